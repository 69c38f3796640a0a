"""TEST INFRASTRUCTURE (oracle) -- Python front of the CPU oracle.

Loads an xspn file with the independent Python decoder (xspn_decode.py) and evaluates it with
the C restatement of the reference arithmetic (spn_oracle.c, built by the Makefile beside it)
or with a slow numpy restatement of the same rules (`evaluate_numpy`, used to cross-check the
C code on small cases).  Nothing in the product imports this module; only tests, the smoke
check and the CPU-baseline / reference arm of the benchmark do.
"""
import ctypes
import os
import subprocess

import numpy as np

from . import xspn_decode
from .xspn_decode import KIND_CAT, KIND_GAUSS, KIND_HIST, KIND_PRODUCT, KIND_SUM

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

MODES = {
    "linear_f64": 0,      # the reference's only f64 mode: probabilities + root log
    "log_f64": 1,         # n-ary max-shifted log-sum-exp in double: the high-precision truth
    "log_f32_gpu": 2,     # reference op order, a + log(1 + exp(b - a)) in float
    "log_f32_cpu": 3,     # reference op order, a + log1p(exp(b - a)) in float
    "log_f64_reforder": 4,
    "linear_f32": 5,
}
_F32_MODES = {2, 3, 5}
_DT = {"uint8": 0, "int8": 1, "uint16": 2, "int16": 3, "uint32": 4, "int32": 5, "uint64": 6,
       "int64": 7, "float32": 8, "float64": 9}


class _CModel(ctypes.Structure):
    _fields_ = [("n_nodes", ctypes.c_int32), ("root", ctypes.c_int32), ("num_features", ctypes.c_int32),
                ("pad_", ctypes.c_int32)] + [(n, ctypes.c_void_p) for n in (
                    "kind", "feature", "mean", "stddev", "child_ptr", "child_idx", "weights", "tab_ptr",
                    "tab", "brk_ptr", "brk")]


def build(force=False):
    """Compile libspn_oracle.so with the Makefile beside this file (no-op when up to date)."""
    so = os.path.join(_HERE, "libspn_oracle.so")
    if force or not os.path.exists(so) or any(
            os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(so)
            for f in ("spn_oracle.c", "spn_oracle_body.inc", "Makefile")):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return so


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        for name in ("spn_oracle_eval", "spn_oracle_eval_vec"):
            fn = getattr(_LIB, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.POINTER(_CModel), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                           ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    return _LIB


class OracleModel:
    """A decoded xspn model held as flat arrays, children-before-parents."""

    def __init__(self, decoded):
        d = dict(decoded)
        n = len(d["kind"])
        # the writer lists children first (BinarySerialization.py:160-191); re-sort if a file does not
        cp, ci = d["child_ptr"], d["child_idx"]
        ok = all((ci[cp[v]:cp[v + 1]] < v).all() for v in range(n)) if n < 200000 else \
            bool((ci < np.repeat(np.arange(n), np.diff(cp))).all())
        if not ok:
            d = _toposort(d)
        self.d = d
        self.num_features = int(d["num_features"])
        self.feature_type = d["feature_type"]
        self.support_marginal = bool(d["support_marginal"])
        self.name = d["name"]
        self._keep = {k: np.ascontiguousarray(d[k], dtype=t) for k, t in (
            ("kind", np.int32), ("feature", np.int32), ("mean", np.float64), ("stddev", np.float64),
            ("child_ptr", np.int64), ("child_idx", np.int32), ("weights", np.float64), ("tab_ptr", np.int64),
            ("tab", np.float64), ("brk_ptr", np.int64), ("brk", np.int32))}
        self.c = _CModel(n_nodes=n, root=int(d["root"]), num_features=self.num_features, pad_=0,
                         **{k: v.ctypes.data for k, v in self._keep.items()})

    def validate(self):
        """The reference's verifier rules (mlir/lib/Dialect/HiSPN/HiSPNOps.cpp:33-126)."""
        d = self.d
        kind, _ = xspn_decode.parse_feature_type(d["feature_type"])
        if d["support_marginal"] and kind != "float":
            raise ValueError("Feature data type must be floating-point to support marginal")
        for v in range(len(d["kind"])):
            k = d["kind"][v]
            nc = d["child_ptr"][v + 1] - d["child_ptr"][v]
            if k in (KIND_SUM, KIND_PRODUCT) and nc == 0:
                raise ValueError("Number of operands must be at least one")
            if k == KIND_SUM:
                w = d["weights"][d["child_ptr"][v]:d["child_ptr"][v + 1]]
                if abs(float(np.sum(w)) - 1.0) > 1e-6:
                    raise ValueError("Weights must sum up to 1.0 for normalized SPN")
            if k == KIND_CAT:
                p = d["tab"][d["tab_ptr"][v]:d["tab_ptr"][v + 1]]
                if abs(float(np.sum(p)) - 1.0) > 1e-6:
                    raise ValueError("Category probabilities should sum to 1.0")


def _toposort(d):
    raise ValueError("xspn nodes are not listed children-before-parents")


def load_model(path_or_bytes):
    return OracleModel(xspn_decode.decode_xspn(path_or_bytes))


def evaluate(model, inputs, mode="log_f32_gpu", marginal=None, strict_nan=False, threads=0, chunk=4096,
             vectorized=False):
    """Per-sample joint log-likelihood of `inputs` ([N, F] numpy array) under `model`."""
    x = np.ascontiguousarray(inputs)
    if x.ndim != 2 or x.shape[1] != model.num_features:
        raise ValueError("inputs must be [N, %d]" % model.num_features)
    m = MODES[mode]
    if marginal is None:
        marginal = model.support_marginal
    out = np.empty(x.shape[0], dtype=np.float32 if m in _F32_MODES else np.float64)
    fn = _lib().spn_oracle_eval_vec if vectorized else _lib().spn_oracle_eval
    rc = fn(ctypes.byref(model.c), m, int(bool(marginal)), int(bool(strict_nan)), _DT[str(x.dtype)],
            x.ctypes.data, x.shape[0], out.ctypes.data, int(threads), int(chunk))
    if rc != 0:
        raise RuntimeError("oracle evaluation failed with code %d" % rc)
    return out


def max_threads():
    return int(_lib().spn_oracle_max_threads())


# ------------------------------------------------------------------------------------------
# numpy restatement (slow; samples vectorised, nodes looped in Python) for cross-checks
# ------------------------------------------------------------------------------------------
def _tree(ops, comb):
    if len(ops) == 1:
        return ops[0]
    piv = (len(ops) + 1) // 2
    return comb(_tree(ops[:piv], comb), _tree(ops[piv:], comb))


def evaluate_numpy(model, inputs, mode="log_f32_gpu", marginal=None, strict_nan=False):
    d = model.d
    x = np.asarray(inputs)
    if marginal is None:
        marginal = model.support_marginal
    linear = mode.startswith("linear")
    rt = np.float32 if mode.endswith("f32") or "_f32_" in mode else np.float64
    isflt = x.dtype.kind == "f"
    vals = {}
    NEG, ONE = (rt(0), rt(1)) if linear else (rt(-np.inf), rt(0))

    def logadd(a0, b0):
        gt = a0 > b0
        a, b = np.where(gt, a0, b0), np.where(gt, b0, a0)
        with np.errstate(invalid="ignore", over="ignore"):
            e = np.exp(b - a)
            r = a + (np.log1p(e) if mode == "log_f32_cpu" else np.log(rt(1) + e))
        if not strict_nan:
            r = np.where((a0 == -np.inf) & (b0 == -np.inf), rt(-np.inf), r)
        return r.astype(rt)

    with np.errstate(divide="ignore", invalid="ignore"):
        for v in range(len(d["kind"])):
            k = d["kind"][v]
            ch = d["child_idx"][d["child_ptr"][v]:d["child_ptr"][v + 1]]
            if k == KIND_GAUSS:
                col = x[:, d["feature"][v]].astype(np.float64)
                xr = col.astype(rt)
                sd = float(d["stddev"][v])
                dd = xr - rt(d["mean"][v])
                if linear:
                    g = rt(1.0 / np.sqrt(2.0 * np.pi * sd * sd)) * np.exp((dd * dd) * rt(-1.0 / (2.0 * sd * sd)))
                else:
                    g = rt(-np.log(sd) - 0.5 * np.log(2 * np.pi)) + (dd * dd) * rt(-(1.0 / (2.0 * sd * sd)))
                if marginal:
                    g = np.where(np.isnan(xr), ONE, g)
                vals[v] = g.astype(rt)
            elif k in (KIND_CAT, KIND_HIST):
                col = x[:, d["feature"][v]].astype(np.float64)
                nan = np.isnan(col) if isflt else np.zeros(len(col), bool)
                idx = np.trunc(np.where(nan, -1, col)).astype(np.int64)
                tab = d["tab"][d["tab_ptr"][v]:d["tab_ptr"][v + 1]]
                tv = tab.astype(rt) if linear else np.log(tab).astype(rt)
                if k == KIND_CAT:
                    inr = (idx >= 0) & (idx < len(tab))
                    b = np.where(inr, idx, 0)
                else:
                    brk = d["brk"][d["brk_ptr"][v]:d["brk_ptr"][v + 1]]
                    b = np.searchsorted(brk, idx, side="right") - 1
                    inr = (idx >= brk[0]) & (idx < brk[-1])
                    b = np.where(inr, b, 0)
                r = np.where(inr, tv[b], NEG)
                r = np.where(nan, ONE if marginal else NEG, r)
                vals[v] = r.astype(rt)
            elif k == KIND_PRODUCT:
                vals[v] = _tree([vals[c] for c in ch], (lambda a, b: a * b) if linear else (lambda a, b: a + b))
            else:
                w = d["weights"][d["child_ptr"][v]:d["child_ptr"][v + 1]]
                if mode == "log_f64":
                    t = np.stack([vals[c] + rt(np.log(wi)) for c, wi in zip(ch, w)])
                    mx = t.max(axis=0)
                    mm = np.where(np.isinf(mx) & (mx < 0), 0, mx)
                    vals[v] = mx + np.log(np.exp(t - mm).sum(axis=0))
                elif linear:
                    vals[v] = _tree([vals[c] * rt(wi) for c, wi in zip(ch, w)], lambda a, b: a + b)
                else:
                    vals[v] = _tree([vals[c] + rt(np.log(wi)) for c, wi in zip(ch, w)], logadd)
        r = vals[int(d["root"])]
        return np.log(r) if linear else r
