"""Properties checked at the full BASELINE batch sizes, where the oracle would take too long to evaluate
everything: (1) a random subset agrees with the oracle; (2) the result does not depend on
how the batch is cut (whole batch through the device entry = two halves = host-path chunks = sharded);
(3) marginalising a feature can only raise the likelihood of a sample (log-space monotonicity) and
marginalising everything gives log 1 = 0.  The two largest configurations (the 53 k-node DAG and the
662 k-node layered model) are additionally compared with the reference-order f32 oracle, and the layered
tensor-core result with the scalar layered kernel."""
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


def _subset_check(q, x, idx, got, chunk):
    """`got` (device results of rows idx) against the f64 oracle and the reference-order f32 oracle."""
    from oracle import oracle
    m = oracle.load_model(q)
    sub = np.ascontiguousarray(x[idx])
    for mode in ("log_f64", "log_f32_gpu"):
        want = oracle.evaluate(m, sub, mode, chunk=chunk)
        err = max_rel_err(got, want)
        assert err <= REL_TOL_F32, (mode, err)


def test_full_batch_config4_mixed_dag(tmp_path):
    """BASELINE configuration 4 at full size: ~53 k nodes over 128 Gaussian + 128 categorical features, default
    options (chunked generated kernel, values crossing chunks through per-CTA scratch), 4 M samples."""
    from spnb import capi, synth
    spn = synth.config4()
    q = write_query(spn, True, directory=str(tmp_path))
    plan_path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true"})
    plan = capi.Plan(plan_path)
    assert plan.stats["nodes"] > 40000
    n = 4_000_000
    x = synth.config4_inputs(n)
    whole = _device_run(plan, x)
    plan.device_status(0)
    assert whole.shape == (n,) and np.isfinite(whole).all()
    idx = np.sort(np.random.default_rng(8).choice(n, 6000, replace=False))
    _subset_check(q, x, idx, whole[idx], 256)
    cut = n // 2 + 4321
    assert np.array_equal(np.concatenate([_device_run(plan, x, 0, cut), _device_run(plan, x, cut, n)]), whole)
    # missing values: Gaussian and categorical columns of a slice marginalised, checked against the oracle
    sub = x[:100000].copy()
    sub[::3, 5] = np.nan
    sub[::4, 200] = np.nan
    got = _device_run(plan, sub)
    pick = np.arange(0, 100000, 50)
    assert max_rel_err(got[pick], oracle_eval(q, sub[pick], True)) <= REL_TOL_F32
    sub[:] = np.nan
    assert np.abs(_device_run(plan, sub[:4096])).max() <= 1e-4
    plan.close()


def test_full_batch_config5_layered(tmp_path):
    """BASELINE configuration 5 at full size: 784 features, depth 4, 16 repetitions, 32 x 1024 dense sums
    (662 529 nodes), 2 M samples on the tensor-core layered kernel; a subset against both oracles and against
    the scalar layered kernel, and the bounded-wait status of the device afterwards."""
    from spnb import capi, synth
    spn = synth.config5()
    q = write_query(spn, True, directory=str(tmp_path))
    plan_path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true"})
    plan = capi.Plan(plan_path)
    assert plan.stats["strategy"] == "layered" and plan.stats["nodes"] > 600000
    n = 2_000_000
    x = synth.config5_inputs(n)
    whole = _device_run(plan, x)
    plan.device_status(0)
    assert whole.shape == (n,) and np.isfinite(whole).all()
    idx = np.sort(np.random.default_rng(9).choice(n, 5000, replace=False))
    _subset_check(q, x, idx, whole[idx], 32)
    scalar_path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "layered-scalar"})
    scalar = capi.Plan(scalar_path)
    sub = np.ascontiguousarray(x[idx])
    assert max_rel_err(whole[idx], scalar.execute_host(sub)) <= REL_TOL_F32
    scalar.close()
    cut = 3 * 524288 + 777   # inside the last 512 Ki-sample transposition chunk
    assert np.array_equal(np.concatenate([_device_run(plan, x, 0, cut), _device_run(plan, x, cut, n)]), whole)
    plan.device_status(0)
    # missing values in a slice
    part = x[:65536].copy()
    part[::5, 100] = np.nan
    part[7, :] = np.nan
    got = _device_run(plan, part)
    assert abs(got[7]) <= 1e-4
    pick = np.arange(0, 65536, 128)
    from oracle import oracle
    want = oracle.evaluate(oracle.load_model(q), np.ascontiguousarray(part[pick]), "log_f64", chunk=32)
    assert max_rel_err(got[pick], want) <= REL_TOL_F32
    plan.close()
