"""GPU parity: the CUDA engine, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Tolerances: 1e-5 relative in log space for f32 results, 1e-12 for f64 results."""
import os

import numpy as np
import pytest

from tests.util_models import (REL_TOL_F32, REL_TOL_F64, max_rel_err, oracle_eval, small_configs, write_query)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from spnb import capi as c
    assert c.device_count() > 0, "GPU tests need a CUDA device"
    return c


def _opts(log_space, **extra):
    o = {"target": "CUDA", "use-log-space": "true" if log_space else "false"}
    o.update({k.replace("_", "-"): str(v) for k, v in extra.items()})
    return o


@pytest.mark.parametrize("kernel", ["unrolled", "interp"])
def test_small_configs_match_oracle(capi, kernel, tmp_path):
    for name, spn, inputs, log_space, marginal in small_configs():
        q = write_query(spn, marginal, directory=str(tmp_path))
        plan_path, info = capi.compile_query(q, _opts(log_space, spnb_kernel=kernel))
        plan = capi.Plan(plan_path)
        # the last size gives every CTA of the generated kernels a row range that ends inside a tile and
        # inside a warp (1.3 to 2 tiles of 1024 rows per CTA on a 148-SM device)
        sizes = (1, 31, 33, 127, 128, 129, 5000) + ((250007,) if kernel == "unrolled" and name.startswith(("cfg1", "cfg2")) else ())
        for n in sizes:
            x = inputs(n)
            got = plan.execute_host(x)
            want = oracle_eval(q, x, log_space)
            assert got.dtype == (np.float32 if log_space else np.float64)
            err = max_rel_err(got, want)
            assert err <= (REL_TOL_F32 if log_space else REL_TOL_F64), (name, kernel, n, err)
        plan.close()
        os.remove(plan_path)


def test_reference_goldens_on_gpu(capi, golden_dir, tmp_path):
    """The stored model/input/output triples of the reference's own tests (NIPS5 is what its CUDA test runs)."""
    from spnb import synth  # noqa: F401
    from oracle import xspn_decode
    for name, dtype in (("NIPS5", np.uint32), ("nltcs", np.float64), ("plants", np.float64)):
        z = np.load(os.path.join(golden_dir, name + "_io.npz"))
        x, ref = z["inputs"].astype(dtype), z["outputs"]
        src = os.path.join(golden_dir, name + ".bin")
        d = xspn_decode.decode_xspn(src)
        q = src
        if not d["is_query"]:
            q = str(tmp_path / (name + "_query.bin"))
            _rewrap_as_query(d, q)
        for log_space, tol in ((True, REL_TOL_F32), (False, REL_TOL_F64)):
            plan_path, _ = capi.compile_query(q, _opts(log_space))
            plan = capi.Plan(plan_path)
            if name == "nltcs" and not log_space:
                # sums with up to 640 addends: the f64 interpreter runs them as loops (the reference's C++
                # default is linear space: compiler/src/option/GlobalOptions.cpp:65)
                assert plan.stats["strategy"] == "interpreter"
            got = plan.execute_host(x)
            assert max_rel_err(got, ref) <= tol, (name, log_space)
            plan.close()
            os.remove(plan_path)


def _rewrap_as_query(d, path):
    """The stored nltcs/plants files carry a bare model header; the reference's tests wrap them in a
    query in Python before compiling.  Do the same with the engine's own writer."""
    from xspn.serialization.binary import wire
    n = len(d["kind"])
    ids = np.arange(n)
    scope_sorted = np.asarray(d["scope"])
    data = wire.encode_flat(
        kind=d["kind"], node_id=ids, child_ptr=d["child_ptr"], child_id=d["child_idx"].astype(np.int32),
        weight=d["weights"], scope_id=np.where(d["feature"] >= 0, scope_sorted[np.maximum(d["feature"], 0)], 0),
        mean=d["mean"], stddev=d["stddev"], tab_ptr=d["tab_ptr"], tab=d["tab"], brk_ptr=d["brk_ptr"], brk=d["brk"],
        root_id=int(d["root"]), scope=list(scope_sorted), feature_type=d["feature_type"], name=d["name"],
        query={"batch_size": 64, "error_kind": 0, "max_error": 0.02, "support_marginal": False})
    with open(path, "wb") as f:
        f.write(data)


def test_chunked_kernels_pass_values_through_scratch(capi, tmp_path):
    """DAGs beyond the chunk size are emitted as several functions; values crossing a chunk boundary go
    through per-CTA scratch memory."""
    for idx in (1, 2, 3, 4):
        name, spn, inputs, log_space, marginal = small_configs()[idx]
        q = write_query(spn, marginal, directory=str(tmp_path))
        for group in (1, 3):   # 3: every chunk runs on three tiles in a row, each with its own scratch slice
            plan_path, _ = capi.compile_query(q, _opts(log_space, spnb_kernel="unrolled", spnb_chunk_nodes=97,
                                                       spnb_table_window=2048, spnb_group_tiles=group))
            plan = capi.Plan(plan_path)
            assert plan.stats["scratch_slots"] > 0 and "st.global" in plan.source
            for n in (1, 1025, 300001):
                x = inputs(n)
                err = max_rel_err(plan.execute_host(x), oracle_eval(q, x, log_space))
                assert err <= REL_TOL_F32, (name, n, group, err)
            plan.close()
            os.remove(plan_path)


def test_scope_local_staging(capi, tmp_path):
    """Models with hundreds of features are cut into chunks whose leaves read few enough features, and every
    chunk stages only its own features from a feature-major copy of the batch (CTAs of 1024 samples).  Checked
    with small staging budgets (many chunks, features staged again and again), with missing values in Gaussian and
    categorical columns (plain and NaN-aware bodies are chosen chunk by chunk), and across the 512 Ki-sample
    pieces the feature-major copy is made in."""
    name, spn, inputs, log_space, marginal = small_configs()[4]
    q = write_query(spn, marginal, directory=str(tmp_path))
    for budget, chunk, ring in ((0, 2000, 0), (64, 300, 0), (16, 97, 0), (40, 300, 4), (0, 2000, 12)):
        # the second variant also ends its chunks where the fewest values are alive and requests the operands
        # of earlier chunks at the top of each function; the third keeps CTA-wide barriers between its chunks (the
        # others let the warps drift apart); the last two copy the operands of earlier chunks into a shared-memory
        # ring ahead of their use
        plan_path, _ = capi.compile_query(q, _opts(True, spnb_kernel="unrolled", spnb_scoped=1, spnb_scope_bytes=budget,
                                                   spnb_chunk_nodes=chunk, spnb_table_window=4096,
                                                   spnb_scope_cut=1 if budget == 64 else 0,
                                                   spnb_hoist_loads=24 if budget == 64 else 0,
                                                   spnb_prefetch_slots=ring,
                                                   spnb_chunk_barrier=1 if budget == 16 else 0))
        plan = capi.Plan(plan_path)
        st = plan.stats
        assert st["scoped_staging"] and st["tile"] == 1024 and st["chunks"] > 1
        for n in (1, 1025, 70001) + ((2 * 524288 + 777,) if budget in (64, 40) else ()):
            x = inputs(n)
            x[::5, 3] = np.nan        # Gaussian column
            x[::7, 200] = np.nan      # categorical column
            x[1 % n, :] = np.nan
            x[::11, 130] = 9.0        # a category outside every table: impossible evidence
            got = plan.execute_host(x)
            if n > 200000:
                idx = np.arange(0, n, 97)
                err = max_rel_err(got[idx], oracle_eval(q, x[idx], True))
            else:
                err = max_rel_err(got, oracle_eval(q, x, True))
            assert err <= REL_TOL_F32, (budget, chunk, n, err)
        plan.close()
        os.remove(plan_path)
    # float64 inputs keep the row-major path (the feature-major copy is single precision)
    x64 = inputs(3000).astype(np.float64)
    spn64 = small_configs()[4][1]
    spn64.feature_type = "float64"
    q64 = write_query(spn64, marginal, directory=str(tmp_path))
    spn64.feature_type = "float32"
    plan_path, _ = capi.compile_query(q64, _opts(True, spnb_kernel="unrolled"))
    plan = capi.Plan(plan_path)
    assert not plan.stats["scoped_staging"]
    assert max_rel_err(plan.execute_host(x64), oracle_eval(q64, x64, True)) <= REL_TOL_F32
    plan.close()


def test_interpreter_spills_values_to_scratch(capi, tmp_path):
    """With fewer shared-memory slots than live values the interpreter keeps the rest in global scratch."""
    for idx in (2, 3, 4):
        name, spn, inputs, log_space, marginal = small_configs()[idx]
        q = write_query(spn, marginal, directory=str(tmp_path))
        plan_path, _ = capi.compile_query(q, _opts(True, spnb_kernel="interp", spnb_interp_slots=6))
        plan = capi.Plan(plan_path)
        assert plan.stats["interp_slots"] > 6
        for n in (1, 257, 200001):
            x = inputs(n)
            err = max_rel_err(plan.execute_host(x), oracle_eval(q, x, True))
            assert err <= REL_TOL_F32, (name, n, err)
        plan.close()
        os.remove(plan_path)


def test_layered_ratspn_kernel(capi, tmp_path):
    """RAT-SPN-style region graphs are recognised and run by the layered kernels (tcgen05 tensor-memory kernel
    by default, mma.sync and scalar FP32 by name); checked against the oracle and against the generic
    interpreter on the same inputs, with missing values and with inputs far outside half-precision range."""
    from spnb import synth
    shapes = [dict(num_features=64, depth=2, repetitions=3, width=4),
              dict(num_features=96, depth=3, repetitions=2, width=8),
              dict(num_features=70, depth=1, repetitions=2, width=32),
              dict(num_features=50, depth=2, repetitions=2, width=6),    # width not a multiple of four
              dict(num_features=192, depth=2, repetitions=2, width=32),  # full-width regions: tensor-core path
              dict(num_features=64, depth=3, repetitions=3, width=32)]
    for sh in shapes:
        spn = synth.config5(seed=7, **sh)
        q = write_query(spn, True, directory=str(tmp_path))
        plans = {}
        for mode in ("layered", "layered-mma", "layered-scalar", "interp"):
            path, _ = capi.compile_query(q, _opts(True, spnb_kernel=mode))
            plans[mode] = (capi.Plan(path), path)
        if sh["width"] == 32:
            # default: two sample tiles per CTA; the one-tile kernel by name and with more warpgroups
            assert plans["layered"][0].stats["tc_tiles"] == 2
            path, _ = capi.compile_query(q, _opts(True, spnb_kernel="layered", spnb_tc_tiles=1))
            plans["layered/1 tile"] = (capi.Plan(path), path)
            assert plans["layered/1 tile"][0].stats["tc_tiles"] == 1
            for wgs in (2, 4):
                path, _ = capi.compile_query(q, _opts(True, spnb_kernel="layered", spnb_tc_warpgroups=wgs))
                plans["layered/%d warpgroups" % wgs] = (capi.Plan(path), path)
        assert plans["layered"][0].stats["strategy"] == "layered"
        for n in (1, 129, 20001):
            x = synth.config5_inputs(n, 31, num_features=sh["num_features"])
            x[::7, ::5] = np.nan
            x[3 % n, :] = np.nan
            x[::11, 3] = 400.0      # squares overflow half precision: the kernel's FP32 path takes the row over
            x[::13, 5] = -1.0e4
            want = oracle_eval(q, x, True)
            for mode, (plan, _) in plans.items():
                err = max_rel_err(plan.execute_host(x), want)
                assert err <= REL_TOL_F32, (sh, n, mode, err)
        for plan, path in plans.values():
            plan.close()
            os.remove(path)
    # a model that is not layered is refused by the layered strategy
    name, spn, inputs, log_space, marginal = small_configs()[2]
    q = write_query(spn, marginal, directory=str(tmp_path))
    with pytest.raises(capi.SpnbError, match="layered"):
        capi.compile_query(q, _opts(True, spnb_kernel="layered"))


def test_layered_kernels_with_raw_scale_gaussians(capi, tmp_path):
    """Leaf means hundreds of standard deviations away from zero and from each other (pixel-scale data with
    narrow components): every layered kernel must evaluate c2 (x - mu)^2 + c1 in the centred form, an expanded
    quadratic loses whole units per leaf here.  Inputs sit near one component's means, so that the
    log-likelihood is moderate and the relative tolerance is a tight absolute one."""
    from spnb import synth
    from xspn.serialization.binary import wire
    spn = synth.config5(seed=23, num_features=64, depth=2, repetitions=2, width=32, mean_dist=(120.0, 40.0), sd_range=(0.05, 0.12))
    q = write_query(spn, True, directory=str(tmp_path))
    a = spn.a
    g = np.nonzero(a["kind"] == wire.K_GAUSS)[0]
    first = {}
    for i in g:                       # the first Gaussian listed for each feature (repetition 0, component 0)
        first.setdefault(int(a["scope_id"][i]), i)
    mu = np.array([a["mean"][first[f]] for f in range(64)])
    sd = np.array([a["stddev"][first[f]] for f in range(64)])
    rng = np.random.default_rng(3)
    n = 4097
    x = (mu[None, :] + rng.standard_normal((n, 64)) * sd[None, :]).astype(np.float32)
    x[::9, 4] = np.nan
    want = oracle_eval(q, x, True)
    assert np.isfinite(want).all() and np.abs(want).max() < 2000.0
    # float32 inputs near 120 carry 4e-6 of rounding into differences of the order of 0.1: the reference's own
    # f32 arithmetic (restated by the oracle's log_f32_gpu mode) is a few 1e-5 away from the f64 value here.
    # The kernels must be as close as that arithmetic allows; the expanded quadratic would be off by 1e-2.
    inherent = max_rel_err(oracle_eval(q, x, True, "log_f32_gpu"), want)
    assert inherent < 2e-4
    for mode in ("layered", "layered-mma", "layered-scalar", "interp"):
        path, _ = capi.compile_query(q, _opts(True, spnb_kernel=mode))
        plan = capi.Plan(path)
        err = max_rel_err(plan.execute_host(x), want)
        assert err <= max(REL_TOL_F32, 4.0 * inherent), (mode, err, inherent)
        plan.close()
        os.remove(path)


def test_bounded_wait_runs_out_and_is_reported(capi, tmp_path):
    """The tensor-core kernels poll their barriers a limited number of times.  A plan compiled with the
    self-test option makes the two-tile kernel leave out one commit; the waiting threads give up, the kernel
    frees its tensor memory and returns normally, spnb_device_status reports the flag (and clears it), the host
    entry point reports it too, and the device keeps working for other plans."""
    import torch
    from spnb import synth
    spn = synth.config5(seed=5, num_features=64, depth=2, repetitions=2, width=32)
    q = write_query(spn, True, directory=str(tmp_path))
    x = synth.config5_inputs(4000, 3, num_features=64)
    good_path, _ = capi.compile_query(q, _opts(True))
    good = capi.Plan(good_path)
    want = good.execute_host(x)
    bad_path, _ = capi.compile_query(q, _opts(True, spnb_selftest_withhold_commit=1, spnb_spin_limit=20000))
    bad = capi.Plan(bad_path)
    assert bad.stats["tc_tiles"] == 2
    dx = torch.from_numpy(x).cuda()
    dout = torch.zeros(x.shape[0], dtype=torch.float32, device="cuda")
    bad.execute_device(0, x.shape[0], dx.data_ptr(), dout.data_ptr(), torch.cuda.current_stream().cuda_stream)
    with pytest.raises(capi.SpnbError, match="bounded wait"):
        bad.device_status(0)
    bad.device_status(0)    # the flag was cleared by the report
    with pytest.raises(capi.SpnbError, match="bounded wait"):
        bad.execute_host(x)
    bad.close()
    # the context is intact: the regular plan still gives the same answers
    assert np.array_equal(good.execute_host(x), want)
    assert max_rel_err(want, oracle_eval(q, x, True)) <= REL_TOL_F32
    good.close()


def test_histogram_buckets_by_arithmetic(capi, tmp_path):
    """Equal-width histograms can bucket their input with multiply-shift instead of the byte table, either with
    the standard special codes (spnb-bucket-arith) or with special codes staged so that one clamp does the rest
    (spnb-bucket-clamp); both must agree with the byte-table path and the oracle, NaN and out-of-range inputs
    included."""
    name, spn, inputs, log_space, marginal = small_configs()[3]
    q = write_query(spn, marginal, directory=str(tmp_path))
    x = inputs(50001)
    x[::13, 7] = 300.0      # outside every histogram
    x[::17, 9] = -5.0
    want = oracle_eval(q, x, True)
    for extra in (dict(spnb_bucket_clamp=1), dict(spnb_bucket_arith=1), dict(spnb_bucket_clamp=1, spnb_scoped=1, spnb_chunk_nodes=200)):
        plan_path, _ = capi.compile_query(q, _opts(True, spnb_kernel="unrolled", **extra))
        plan = capi.Plan(plan_path)
        if "spnb_bucket_clamp" in extra:
            assert "min((" in plan.source
        err = max_rel_err(plan.execute_host(x), want)
        assert err <= REL_TOL_F32, (extra, err)
        plan.close()
        os.remove(plan_path)


def test_fused_leaf_tables(capi, tmp_path):
    """Discrete leaf children of a product read through one table over their combined code must give what the
    one-read-per-leaf kernel gives (to rounding) and what the oracle gives, in both spaces, with codes outside the
    tables and, for floating inputs with marginal support, missing values."""
    name, spn, inputs, _, _ = small_configs()[0]
    for log_space, marginal, ftype in ((False, False, "int32"), (True, False, "int32"), (True, True, "float32"), (False, True, "float64")):
        spn.feature_type = ftype
        q = write_query(spn, marginal, directory=str(tmp_path))
        x = inputs(20011).astype(ftype)
        x[::7, 3] = 7            # a category no table has: impossible evidence
        x[::11, 5] = -1
        if marginal:
            x[::5, 2] = np.nan
            x[::13, :] = np.nan
        want = oracle_eval(q, x, log_space)
        got = {}
        for fuse, entries in ((1, 128), (1, 16), (0, 128)):
            plan_path, _ = capi.compile_query(q, _opts(log_space, spnb_kernel="unrolled", spnb_fuse_leaves=fuse, spnb_fuse_entries=entries))
            plan = capi.Plan(plan_path)
            assert (plan.stats["fused_table_entries"] > 0) == bool(fuse)
            got[(fuse, entries)] = plan.execute_host(x)
            err = max_rel_err(got[(fuse, entries)], want)
            assert err <= (REL_TOL_F32 if log_space else REL_TOL_F64), (log_space, marginal, fuse, entries, err)
            plan.close()
            os.remove(plan_path)
        assert max_rel_err(got[(1, 128)], got[(0, 128)]) <= (2e-6 if log_space else 1e-14)
    spn.feature_type = "int32"


def test_streamed_table_window(capi, tmp_path):
    """Leaf tables larger than the shared-memory window are reloaded piecewise inside the kernel body."""
    for idx in (3, 4, 1):
        name, spn, inputs, log_space, marginal = small_configs()[idx]
        q = write_query(spn, marginal, directory=str(tmp_path))
        plan_path, _ = capi.compile_query(q, _opts(log_space, spnb_kernel="unrolled", spnb_table_window=1024))
        plan = capi.Plan(plan_path)
        assert "win[i] = __ldg" in plan.source and plan.source.count("win[i] = __ldg") > 4
        for n in (1, 1000, 70001):
            x = inputs(n)
            err = max_rel_err(plan.execute_host(x), oracle_eval(q, x, log_space))
            assert err <= REL_TOL_F32, (name, n, err)
        plan.close()
        os.remove(plan_path)


def test_device_pointer_entry_matches_host_entry(capi, tmp_path):
    import torch
    name, spn, inputs, log_space, marginal = small_configs()[2]
    q = write_query(spn, marginal, directory=str(tmp_path))
    plan_path, _ = capi.compile_query(q, _opts(True))
    plan = capi.Plan(plan_path)
    x = inputs(100000)
    host = plan.execute_host(x)
    dx = torch.from_numpy(x).cuda()
    dout = torch.empty(x.shape[0], dtype=torch.float32, device="cuda")
    plan.execute_device(0, x.shape[0], dx.data_ptr(), dout.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    plan.device_status(0)   # no kernel of the plan gave up on a bounded wait
    assert np.array_equal(dout.cpu().numpy(), host)
    assert max_rel_err(host, oracle_eval(q, x, True)) <= REL_TOL_F32
    plan.close()
    # the same through the layered tcgen05 kernel, whose bounded-wait flag only device_status reports here
    from spnb import synth
    spn = synth.config5(seed=9, num_features=96, depth=3, repetitions=2, width=32)
    q = write_query(spn, True, directory=str(tmp_path))
    plan_path, _ = capi.compile_query(q, _opts(True))
    plan = capi.Plan(plan_path)
    assert plan.stats["strategy"] == "layered"
    x = synth.config5_inputs(30001, 5, num_features=96)
    x[::9, 1] = np.nan
    host = plan.execute_host(x)
    dx = torch.from_numpy(x).cuda()
    dout = torch.empty(x.shape[0], dtype=torch.float32, device="cuda")
    plan.execute_device(0, x.shape[0], dx.data_ptr(), dout.data_ptr(), torch.cuda.current_stream().cuda_stream)
    plan.device_status(0)
    assert np.array_equal(dout.cpu().numpy(), host)
    assert max_rel_err(host, oracle_eval(q, x, True)) <= REL_TOL_F32
    plan.close()
