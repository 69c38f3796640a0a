"""ctypes binding of the C ABI in include/spnb.h (libspnb.so).

There is no fallback: if the library is missing the import fails, and if no CUDA device is
present every execute call returns an error from the library itself."""
import ctypes
import json
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.normpath(os.path.join(_HERE, "..", "..", "lib", "libspnb.so"))


class KernelInfo(ctypes.Structure):
    _fields_ = [("kernel_name", ctypes.c_char * 256), ("query_type", ctypes.c_uint32), ("target", ctypes.c_uint32),
                ("batch_size", ctypes.c_uint32), ("num_features", ctypes.c_uint32),
                ("bytes_per_feature", ctypes.c_uint32), ("num_results", ctypes.c_uint32),
                ("bytes_per_result", ctypes.c_uint32), ("dtype", ctypes.c_char * 16)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError("libspnb.so not found at %s: build it with `make -C spn-compiler_b200/csrc` "
                          "(or __graft_entry__.build())" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    vp, cp, sz = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t
    sig = {
        "spnb_compile": (ctypes.c_int, [cp, ctypes.POINTER(cp), ctypes.POINTER(cp), ctypes.c_int, cp, ctypes.c_char_p, sz,
                                        ctypes.POINTER(KernelInfo)]),
        "spnb_plan_load": (ctypes.c_int, [cp, ctypes.POINTER(vp)]),
        "spnb_plan_info": (ctypes.c_int, [vp, ctypes.POINTER(KernelInfo)]),
        "spnb_plan_stats_json": (cp, [vp]),
        "spnb_plan_source": (cp, [vp]),
        "spnb_execute_host": (ctypes.c_int, [vp, sz, vp, vp]),
        "spnb_execute_device": (ctypes.c_int, [vp, ctypes.c_int, sz, vp, vp, vp]),
        "spnb_execute_device_noalloc": (ctypes.c_int, [vp, ctypes.c_int, sz, vp, vp, vp]),
        "spnb_execute_sharded": (ctypes.c_int, [vp, ctypes.POINTER(ctypes.c_int), ctypes.c_int, sz, vp, vp,
                                                ctypes.POINTER(ctypes.c_double)]),
        "spnb_set_device": (ctypes.c_int, [vp, ctypes.c_int]),
        "spnb_launch_config": (ctypes.c_int, [vp, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                              ctypes.POINTER(sz)]),
        "spnb_device_status": (ctypes.c_int, [vp, ctypes.c_int]),
        "spnb_last_kernel_ms": (ctypes.c_float, [vp]),
        "spnb_plan_free": (None, [vp]),
        "spnb_measure_peak": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(ctypes.c_double)]),
        "spnb_device_count": (ctypes.c_int, []),
        "spnb_last_error": (cp, []),
        "spnb_version": (cp, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()
EXPORTS = ["spnb_compile", "spnb_plan_load", "spnb_plan_info", "spnb_plan_stats_json", "spnb_plan_source",
           "spnb_execute_host", "spnb_execute_device", "spnb_execute_device_noalloc", "spnb_execute_sharded", "spnb_set_device",
           "spnb_launch_config", "spnb_device_status", "spnb_last_kernel_ms", "spnb_plan_free", "spnb_measure_peak", "spnb_device_count", "spnb_last_error",
           "spnb_version"]


class SpnbError(RuntimeError):
    pass


def _check(rc):
    if rc != 0:
        raise SpnbError(lib.spnb_last_error().decode("utf-8", "replace"))


def compile_query(query_path, options, plan_path=None):
    """-> (plan_path, KernelInfo)"""
    keys = (ctypes.c_char_p * len(options))(*[str(k).encode() for k in options])
    vals = (ctypes.c_char_p * len(options))(*[str(v).encode() for v in options.values()])
    out = ctypes.create_string_buffer(4096)
    info = KernelInfo()
    _check(lib.spnb_compile(str(query_path).encode(), keys, vals, len(options),
                            plan_path.encode() if plan_path else None, out, 4096, ctypes.byref(info)))
    return out.value.decode(), info


class Plan:
    def __init__(self, plan_path):
        self._h = ctypes.c_void_p()
        _check(lib.spnb_plan_load(str(plan_path).encode(), ctypes.byref(self._h)))
        self.info = KernelInfo()
        _check(lib.spnb_plan_info(self._h, ctypes.byref(self.info)))
        self.num_features = int(self.info.num_features)
        self.result_dtype = np.dtype(self.info.dtype.decode())
        self.bytes_per_feature = int(self.info.bytes_per_feature)

    def close(self):
        if self._h:
            lib.spnb_plan_free(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stats(self):
        return json.loads(lib.spnb_plan_stats_json(self._h).decode())

    @property
    def source(self):
        return lib.spnb_plan_source(self._h).decode()

    def _check_in(self, x):
        if x.ndim != 2 or x.shape[1] != self.num_features or x.dtype.itemsize != self.bytes_per_feature:
            raise SpnbError("inputs must be [N, %d] with %d-byte elements" % (self.num_features, self.bytes_per_feature))

    def execute_host(self, inputs):
        x = np.ascontiguousarray(inputs)
        self._check_in(x)
        out = np.empty(x.shape[0], dtype=self.result_dtype)
        _check(lib.spnb_execute_host(self._h, x.shape[0], x.ctypes.data, out.ctypes.data))
        return out

    def execute_host_ptr(self, n, in_ptr, out_ptr):
        _check(lib.spnb_execute_host(self._h, n, in_ptr, out_ptr))

    def execute_device(self, device, n, d_in, d_out, stream=0):
        _check(lib.spnb_execute_device(self._h, device, n, d_in, d_out, stream))

    def execute_device_noalloc(self, device, n, d_in, d_out, stream=0):
        """Like execute_device, but through the entry point that never allocates device memory."""
        _check(lib.spnb_execute_device_noalloc(self._h, device, n, d_in, d_out, stream))

    def execute_sharded(self, devices, inputs, want_mean=False):
        x = np.ascontiguousarray(inputs)
        self._check_in(x)
        out = np.empty(x.shape[0], dtype=self.result_dtype)
        devs = (ctypes.c_int * len(devices))(*devices)
        mean = ctypes.c_double(0.0)
        _check(lib.spnb_execute_sharded(self._h, devs, len(devices), x.shape[0], x.ctypes.data, out.ctypes.data,
                                        ctypes.byref(mean) if want_mean else None))
        return (out, mean.value) if want_mean else out

    def set_device(self, device):
        _check(lib.spnb_set_device(self._h, device))

    def launch_config(self, device=0):
        g, b, s = ctypes.c_int(), ctypes.c_int(), ctypes.c_size_t()
        _check(lib.spnb_launch_config(self._h, device, ctypes.byref(g), ctypes.byref(b), ctypes.byref(s)))
        return g.value, b.value, s.value

    def device_status(self, device=0):
        """Waits for the plan's queued work on `device`; raises SpnbError if a kernel gave up on a bounded wait."""
        _check(lib.spnb_device_status(self._h, device))

    @property
    def last_kernel_ms(self):
        return float(lib.spnb_last_kernel_ms(self._h))


def device_count():
    return int(lib.spnb_device_count())


def measure_peak(kind):
    """Instruction rate of the current device: 'fp32', 'ex2', 'lg2' or 'fp64' -> operations per second."""
    v = ctypes.c_double(0.0)
    _check(lib.spnb_measure_peak({"fp32": 0, "ex2": 1, "lg2": 2, "fp64": 3, "fp32x2": 4}[kind], ctypes.byref(v)))
    return v.value
