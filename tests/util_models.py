"""Helpers shared by the tests: seeded models as xspn files, oracle evaluation, error metrics."""
import os
import tempfile

import numpy as np

from oracle import oracle
from spnb import synth

REL_TOL_F32 = 1e-5    # north-star tolerance for f32 log-space results (relative, in log space)
REL_TOL_F64 = 1e-12   # ... and for f64 results


def write_query(spn, support_marginal, batch_size=64, directory=None):
    """Serialise a synth.FlatSPN to a temporary xspn query file and return its path."""
    fd, path = tempfile.mkstemp(suffix=".bin", dir=directory)
    with os.fdopen(fd, "wb") as f:
        f.write(spn.to_xspn_bytes(batch_size=batch_size, support_marginal=support_marginal))
    return path


def max_rel_err(got, want):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    fin = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), fin), "finite/non-finite pattern differs"
    assert np.array_equal(got[~fin], want[~fin]) or (np.isnan(got[~fin]) == np.isnan(want[~fin])).all()
    if not fin.any():
        return 0.0
    # relative in log space; for |ll| < 1 (everything marginalised: ll ~ 0) the bound is absolute
    return float(np.max(np.abs(got[fin] - want[fin]) / np.maximum(np.abs(want[fin]), 1.0)))


def small_configs():
    """(name, FlatSPN, inputs(n), log_space, marginal) at sizes the oracle finishes in seconds."""
    c1 = synth.config1()
    c2 = synth.config2(target_nodes=600)
    c3 = synth.config3(target_nodes=1500)
    c4 = synth.config4(target_nodes=4000)
    return [
        ("cfg1_f64_linear", c1, lambda n: synth.config1_inputs(c1, n), False, False),
        ("cfg1_f32_log", c1, lambda n: synth.config1_inputs(c1, n), True, False),
        ("cfg2_gauss", c2, synth.config2_inputs, True, True),
        ("cfg3_hist_nan", c3, synth.config3_inputs, True, True),
        ("cfg4_mixed", c4, synth.config4_inputs, True, True),
    ]


def oracle_eval(path, x, log_space, mode=None):
    m = oracle.load_model(path)
    if mode is None:
        mode = "log_f64" if log_space else "linear_f64"
    return oracle.evaluate(m, x, mode)
