"""Properties checked at the full BASELINE batch sizes, where the oracle would take too long to evaluate
everything: (1) a random 20 000-sample subset agrees with the oracle; (2) the result does not depend on
how the batch is cut (whole batch through the device entry = two halves = host-path chunks = sharded);
(3) marginalising a feature can only raise the likelihood of a sample (log-space monotonicity) and
marginalising everything gives log 1 = 0."""
import numpy as np
import pytest

from tests.util_models import REL_TOL_F32, max_rel_err, oracle_eval, write_query

pytestmark = pytest.mark.gpu


def _device_run(plan, x, lo=0, hi=None):
    import torch
    hi = x.shape[0] if hi is None else hi
    dx = torch.from_numpy(x[lo:hi]).cuda()
    out = torch.empty(hi - lo, dtype=torch.float32, device="cuda")
    plan.execute_device(0, hi - lo, dx.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("cfg,n", [(2, 10_000_000), (3, 4_000_000)])
def test_full_batch_properties(cfg, n, tmp_path):
    from spnb import capi, synth
    spn = getattr(synth, "config%d" % cfg)()
    gen = getattr(synth, "config%d_inputs" % cfg)
    q = write_query(spn, True, directory=str(tmp_path))
    plan_path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true"})
    plan = capi.Plan(plan_path)
    x = gen(n)
    whole = _device_run(plan, x)
    assert whole.shape == (n,) and np.isfinite(whole).all()
    # (1) subset against the oracle
    idx = np.random.default_rng(5).choice(n, 20000, replace=False)
    assert max_rel_err(whole[idx], oracle_eval(q, x[idx], True)) <= REL_TOL_F32
    # (2) independence of the cut
    cut = n // 2 + 12345
    assert np.array_equal(np.concatenate([_device_run(plan, x, 0, cut), _device_run(plan, x, cut, n)]), whole)
    assert np.array_equal(plan.execute_host(x), whole)
    assert np.array_equal(plan.execute_sharded([0, 0], x), whole)
    # (3) marginalisation
    sub = x[:200000].copy()
    base = whole[:200000]
    sub[:, 0] = np.nan
    more = _device_run(plan, sub)
    if cfg == 3:   # histogram densities are probabilities of single values: marginalising never lowers ll
        assert (more >= base - 1e-3).all()
    sub[:] = np.nan
    assert np.abs(_device_run(plan, sub)).max() <= 1e-4
    plan.close()


def test_layered_batch_larger_than_one_transposition_chunk(tmp_path):
    """The layered path copies the batch feature-major 512 Ki samples at a time: a batch that needs three such
    chunks (the last one ragged) gives the same values as its pieces and as the host path, and a subset agrees
    with the oracle."""
    from spnb import capi, synth
    spn = synth.config5(seed=11, num_features=64, depth=3, repetitions=2, width=32)
    q = write_query(spn, True, directory=str(tmp_path))
    plan_path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true"})
    plan = capi.Plan(plan_path)
    assert plan.stats["strategy"] == "layered"
    n = 2 * 524288 + 70001
    x = synth.config5_inputs(n, 17, num_features=64)
    x[::1013, 7] = np.nan
    whole = _device_run(plan, x)
    plan.device_status(0)
    assert whole.shape == (n,) and np.isfinite(whole).all()
    idx = np.random.default_rng(6).choice(n, 5000, replace=False)
    assert max_rel_err(whole[idx], oracle_eval(q, x[idx], True)) <= REL_TOL_F32
    cut = 524288 + 333
    assert np.array_equal(np.concatenate([_device_run(plan, x, 0, cut), _device_run(plan, x, cut, n)]), whole)
    assert np.array_equal(plan.execute_host(x), whole)
    plan.close()
