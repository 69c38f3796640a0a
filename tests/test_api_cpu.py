"""Host-side logic that needs no GPU: C-ABI exports, option handling, the xspn writer/reader pair,
planner statistics, the pybind module and the CUDACompiler front."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import oracle
from tests.util_models import small_configs, write_query
from xspn.serialization.binary.BinarySerialization import BinarySerializer
from xspn.structure.Model import SPNModel
from xspn.structure.Nodes import Categorical, Gaussian, Histogram, Product, Sum
from xspn.structure.Query import JointProbability

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from spnb import capi
    header = open(os.path.join(ROOT, "include", "spnb.h")).read()
    declared = set(re.findall(r"\b(spnb_[a-z_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(capi.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), name
    assert declared == set(capi.EXPORTS)


def test_no_gpu_means_a_loud_error_not_a_fallback(tmp_path):
    from spnb import capi
    if capi.device_count() > 0:
        pytest.skip("a GPU is present")
    name, spn, inputs, log_space, marginal = small_configs()[2]
    q = write_query(spn, marginal, directory=str(tmp_path))
    plan_path, info = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true"})
    plan = capi.Plan(plan_path)
    with pytest.raises(capi.SpnbError, match="no CPU fallback"):
        plan.execute_host(inputs(8))


def test_option_handling(tmp_path):
    from spnb import capi
    name, spn, inputs, log_space, marginal = small_configs()[0]
    q = write_query(spn, False, directory=str(tmp_path))
    with pytest.raises(capi.SpnbError, match="Unknown compile option"):
        capi.compile_query(q, {"target": "CUDA", "no-such-option": "1"})
    with pytest.raises(capi.SpnbError, match="target"):
        capi.compile_query(q, {"use-log-space": "true"})
    with pytest.raises(capi.SpnbError, match="spnb-tile"):
        capi.compile_query(q, {"target": "CUDA", "spnb-tile": "100"})
    with pytest.raises(capi.SpnbError, match="CPU"):
        capi.compile_query(q, {"target": "CPU"})
    # every key the reference's Python layer may pass is accepted
    opts = {"target": "CUDA", "use-log-space": "true", "gpu-shared-mem": "false", "dump-ir": "false",
            "search-paths": "/tmp", "maxTaskSize": "10", "optLevel": "3", "cpu-vectorize": "false",
            "vector-library": "None", "use-shuffle": "false", "delete-temps": "true", "opt-repr": "false",
            "collect-graph-stats": "true", "graph-stats-file": str(tmp_path / "stats.json")}
    path, info = capi.compile_query(q, opts)
    assert os.path.isfile(path) and os.path.isfile(tmp_path / "stats.json")
    import json
    gs = json.load(open(tmp_path / "stats.json"))
    # the reference's key set (LoSPNGraphStatsCollection.cpp:83-102) with the engine's own statistics beside it
    for key in ("featureCount", "minDepth", "maxDepth", "averageDepth", "medianDepth", "innerCount", "leafCount",
                "sumCount", "productCount", "categoricalCount", "constantCount", "gaussianCount", "histogramCount"):
        assert key in gs, key
    assert gs["featureCount"] == 16 and gs["gaussianCount"] == 0 and gs["categoricalCount"] == gs["spnb"]["categorical"]
    assert gs["minDepth"] <= gs["medianDepth"] <= gs["maxDepth"] and gs["innerCount"] == gs["sumCount"] + gs["productCount"]
    assert info.dtype == b"float32" and info.bytes_per_result == 4 and info.query_type == 1 and info.target == 2
    path, info = capi.compile_query(q, {"target": "CUDA"})  # reference default: linear space, f64 result
    assert info.dtype == b"float64" and info.bytes_per_result == 8
    # marginal support needs a floating feature type (int32 inputs here)
    qm = write_query(spn, True, directory=str(tmp_path))
    with pytest.raises(capi.SpnbError, match="floating-point to support marginal"):
        capi.compile_query(qm, {"target": "CUDA"})


def test_model_header_is_rejected_like_the_reference(golden_dir):
    from spnb import capi
    with pytest.raises(capi.SpnbError, match="Cannot compile raw models"):
        capi.compile_query(os.path.join(golden_dir, "nltcs.bin"), {"target": "CUDA"})


def test_planner_statistics_and_strategies(tmp_path, golden_dir):
    from spnb import capi
    path, info = capi.compile_query(os.path.join(golden_dir, "NIPS5.bin"), {"target": "CUDA", "use-log-space": "true"})
    st = capi.Plan(path).stats
    assert (st["histogram"], st["products"], st["sums"]) == (10, 2, 1) and st["strategy"] == "unrolled"
    assert st["ops_sfu"] == 3 and st["bytes_per_sample"] == 5 * 4 + 4
    assert info.kernel_name == b"spn_kernel" and info.num_features == 5 and info.bytes_per_feature == 4
    path, _ = capi.compile_query(os.path.join(golden_dir, "speaker_FADG0.bin"),
                                 {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "interp"})
    st = capi.Plan(path).stats
    assert st["strategy"] == "interpreter" and st["gaussian"] == 1326 and st["sum_edges"] == 51


def test_corrupt_files_fail_cleanly(tmp_path, golden_dir):
    from spnb import capi
    data = open(os.path.join(golden_dir, "NIPS5.bin"), "rb").read()
    for cut in (0, 7, 8, 40, len(data) // 2, len(data) - 8):
        p = tmp_path / ("cut%d.bin" % cut)
        p.write_bytes(data[:cut])
        with pytest.raises(capi.SpnbError):
            capi.compile_query(str(p), {"target": "CUDA"})
    rng = np.random.default_rng(0)
    for trial in range(30):
        b = bytearray(data)
        for pos in rng.integers(8, len(b), size=6):
            b[pos] ^= 0xFF
        p = tmp_path / ("flip%d.bin" % trial)
        p.write_bytes(bytes(b))
        try:
            capi.compile_query(str(p), {"target": "CUDA", "use-log-space": "true"})
        except capi.SpnbError:
            pass  # an error message is fine, a crash is not


def _toy_spn():
    g1, g2 = Gaussian(0.5, 1.0, scope=0), Gaussian(0.25, 0.1, scope=1)
    c1, h1 = Categorical([0.35, 0.55, 0.1], scope=2), Histogram([0, 2, 4], [0.25, 0.75], [1, 3], scope=3)
    g3, g4 = Gaussian(-0.5, 2.0, scope=0), Gaussian(1.25, 0.7, scope=1)
    c2, h2 = Categorical([0.2, 0.3, 0.5], scope=2), Histogram([0, 1, 4], [0.4, 0.2], [0.5, 2], scope=3)
    return Sum([0.3, 0.5, 0.2], [Product([g1, g2, c1, h1]), Product([g3, g4, c2, h2]), Product([g1, g4, c2, h1])])


def test_writer_output_is_read_back_by_both_readers(tmp_path):
    from spnb import capi
    q = JointProbability(SPNModel(_toy_spn(), "float32", "toy"), batchSize=64, supportMarginal=True)
    path = str(tmp_path / "toy.bin")
    BinarySerializer(path).serialize_to_file(q)
    m = oracle.load_model(path)
    assert (m.name, m.feature_type, m.num_features, m.support_marginal) == ("toy", "float32", 4, True)
    plan_path, info = capi.compile_query(path, {"target": "CUDA", "use-log-space": "true"})
    st = capi.Plan(plan_path).stats
    # g1, g4, c2 and h1 are shared by two products and must be merged, not duplicated
    assert st["nodes"] == 12 and st["gaussian"] == 4 and st["categorical"] == 2 and st["histogram"] == 2
    assert info.kernel_name == b"toy" and info.batch_size == 64


def test_pybind_module_and_cuda_compiler_front(tmp_path):
    import spnc.spncpy as spncpy
    from spnc.gpu import CUDACompiler
    k = spncpy.Kernel("/tmp/x.plan", "name", 1, 2, 64, 5, 4, 1, 4, "float32")
    assert k.fileName() == "/tmp/x.plan" and k.kernelName() == "name"
    assert spncpy.SPNCompiler.isTargetSupported("CPU") is False
    assert spncpy.SPNCompiler.getHostArchitecture()
    comp = CUDACompiler(computeInLogSpace=True, spnb_kernel="auto") if False else CUDACompiler()
    kernel = comp.compile_ll(_toy_spn(), inputDataType="float32")
    assert os.path.isfile(kernel.fileName()) and kernel.kernelName() == "spn_gpu"
    with pytest.raises(RuntimeError, match="two-dimensional"):
        comp.execute(kernel, np.zeros(4, np.float32))
    with pytest.raises(RuntimeError, match="numpy array"):
        comp.execute(kernel, [[0.0] * 4])
    with pytest.raises(RuntimeError, match="element size"):
        comp.execute(kernel, np.zeros((2, 4), np.float64))
    if not CUDACompiler.isAvailable():
        with pytest.raises(RuntimeError, match="RUNTIME ERROR"):
            comp.execute(kernel, np.zeros((2, 4), np.float32))
    with pytest.raises(RuntimeError, match="COMPILATION ERROR"):
        CUDACompiler(bogus="1").compile_ll(_toy_spn(), inputDataType="float32")
    os.remove(kernel.fileName())


def test_histogram_buckets_can_be_computed_where_that_is_exact(tmp_path):
    """With spnb-bucket-arith=1 near-equal-width histograms get their bucket from a multiply-shift of the
    staged code; the byte table stays for irregular breaks and by default.  (Compilation needs no GPU.)"""
    from spnb import capi
    name, spn, inputs, log_space, marginal = small_configs()[3]
    q = write_query(spn, marginal, directory=str(tmp_path))
    on, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "unrolled",
                                   "spnb-bucket-arith": "1"})
    off, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "unrolled"})
    src_on, src_off = capi.Plan(on).source, capi.Plan(off).source
    assert src_on.count(") >> 16;") > 100 and src_off.count(") >> 16;") == 0
    assert src_off.count("lut_s") > src_on.count("lut_s")
    # a histogram with irregular breaks keeps its byte table
    from spnb import synth
    b = synth.FlatSPN(2, "float32", "two_histograms")
    h0 = b.histogram(0, [0, 3, 50, 51, 200], [0.1, 0.2, 0.3, 0.4])
    h1 = b.histogram(1, [0, 64, 128, 192, 256], [0.25, 0.25, 0.25, 0.25])
    b.root = b.product([h0, h1])
    q2 = write_query(b, True, directory=str(tmp_path))
    p2, _ = capi.compile_query(q2, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "unrolled",
                                    "spnb-bucket-arith": "1"})
    src2 = capi.Plan(p2).source
    assert src2.count(") >> 16;") == 1 and "lut_s" in src2


def test_discrete_leaves_of_a_product_share_a_fused_table(tmp_path):
    """Categorical leaf children of one product are looked up through one table over their combined code
    (fewer shared-memory reads); a leaf with a second consumer, a Gaussian sibling and a chunked kernel keep
    the plain reads.  (Compilation needs no GPU.)"""
    from spnb import capi, synth
    b = synth.FlatSPN(4, "int32", "fusable")
    c0 = b.categorical(0, [0.2, 0.8])
    c1 = b.categorical(1, [0.5, 0.25, 0.25])
    c2 = b.categorical(2, [0.1, 0.9])
    c3 = b.categorical(3, [0.3, 0.7])
    d3 = b.categorical(3, [0.6, 0.4])
    shared = b.categorical(2, [0.4, 0.6])
    p1 = b.product([c0, c1, c2, c3])
    p2 = b.product([b.categorical(0, [0.5, 0.5]), b.categorical(1, [0.1, 0.1, 0.8]), shared, d3])
    p3 = b.product([b.categorical(0, [0.3, 0.7]), b.categorical(1, [0.2, 0.2, 0.6]), shared, b.categorical(3, [0.9, 0.1])])
    b.root = b.sum([p1, p2, p3], [0.5, 0.25, 0.25])
    q = write_query(b, False, directory=str(tmp_path))
    for log_space in ("true", "false"):
        on, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": log_space, "spnb-kernel": "unrolled",
                                       "spnb-fuse-entries": "128"})
        off, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": log_space, "spnb-kernel": "unrolled",
                                        "spnb-fuse-leaves": "0"})
        pon, poff = capi.Plan(on), capi.Plan(off)
        ld = "ld.shared.f32" if log_space == "true" else "ld.shared.f64"
        # 11 leaves read one by one; fused: one group of three per product (4 * 5 * 4 = 80 combined codes each; a
        # fourth leaf would exceed the 128-entry limit), the first product's last leaf and the shared leaf on their own
        assert poff.source.count(ld) == 11 and poff.stats["fused_table_entries"] == 0
        assert pon.source.count(ld) == 3 + 2
        assert pon.stats["fused_table_entries"] == 3 * 80
    small, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "unrolled",
                                      "spnb-fuse-entries": "20"})
    # pairs only: (4 * 5) + (4 * 4) in the first product, (4 * 5) in the other two
    assert capi.Plan(small).stats["fused_table_entries"] == 36 + 20 + 20


def test_staging_schemes_show_in_the_generated_source(tmp_path):
    """Which staging scheme a model gets, read off the generated source.  (Compilation needs no GPU.)"""
    from spnb import capi
    configs = small_configs()
    # 16 int32 features, discrete leaves: asynchronous double-buffered stage, codes digested in registers
    name, spn, inputs, log_space, marginal = configs[0]
    q = write_query(spn, marginal, directory=str(tmp_path))
    plan = capi.Plan(capi.compile_query(q, {"target": "CUDA", "use-log-space": "false", "spnb-kernel": "unrolled"})[0])
    assert "cp.async.ca.shared.global" in plan.source and "int cf0;" in plan.source and "ld.shared.u8" not in plan.source
    sync = capi.Plan(capi.compile_query(q, {"target": "CUDA", "use-log-space": "false", "spnb-kernel": "unrolled",
                                            "spnb-async-stage": "0"})[0])
    assert "cp.async" not in sync.source and "ld.shared.u8" in sync.source
    # 256 mixed features: scope-local staging, no CTA-wide barrier between chunks, codes from the byte plane
    name, spn, inputs, log_space, marginal = configs[4]
    q = write_query(spn, marginal, directory=str(tmp_path))
    base = {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "unrolled", "spnb-scoped": "1", "spnb-chunk-nodes": "300"}
    plan = capi.Plan(capi.compile_query(q, base)[0])
    assert plan.stats["scoped_staging"] and plan.stats["chunks"] > 5
    assert "__any_sync(0xffffffffu, nan)" in plan.source and "__syncthreads_or(nan)" not in plan.source
    assert "srcc[(unsigned long long)__ldg(cf + j) * ld]" in plan.source
    lock = capi.Plan(capi.compile_query(q, dict(base, **{"spnb-chunk-barrier": "1", "spnb-code-plane": "0"}))[0])
    assert "__syncthreads_or(nan)" in lock.source and "__any_sync" not in lock.source
    assert "TOINT(raw)" in lock.source and "srcc[(unsigned long long)__ldg(cf + j) * ld]" not in lock.source
    ring = capi.Plan(capi.compile_query(q, dict(base, **{"spnb-prefetch-slots": "4"}))[0])
    assert "cp.async.wait_group 3; ld.shared.f32" in ring.source


def test_two_tile_tensor_core_program(tmp_path):
    """The plan of a full-width layered model is annotated for the two-tile tensor-core kernel: right operands
    go straight to the operand buffer, left operands wait in registers (sibling = one leaf region) or in an
    a-stack whose depth is the region-tree depth minus one; narrower models stay on the one-tile kernel."""
    from spnb import capi, synth
    for depth in (1, 2, 3, 4):
        spn = synth.config5(seed=3, num_features=16 * 2 ** depth, depth=depth, repetitions=2, width=32)
        q = write_query(spn, True, directory=str(tmp_path))
        path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "layered"})
        st = capi.Plan(path).stats
        assert st["tc_tiles"] == 2
        prog = st["tc_program"]
        assert prog["a_slots"] == max(depth - 1, 1)
        steps = prog["steps"].split()
        assert len(steps) == 2 * (2 ** (depth + 1) - 1)
        # replay: slots are used as a stack, every inner step finds its operands where the program says
        live, regs, operand = [], False, False
        for tok in steps:
            kind = tok[0]
            if kind in "IR":
                src = tok[1]
                assert operand, tok
                operand = False
                if src == "r":
                    assert regs
                    regs = False
                else:
                    assert live and live[-1] == int(src), (tok, live)
                    live.pop()
            dest = tok[1:] if kind == "L" else tok[2:]
            if dest == "o":
                assert not operand
                operand = True
            elif dest == "r":
                assert not regs
                regs = True
            elif dest.startswith("s"):
                assert int(dest[1:]) == len(live)
                live.append(int(dest[1:]))
            else:
                assert dest == "-" and kind == "R"
        assert not live and not regs and not operand
    narrow = synth.config5(seed=3, num_features=32, depth=2, repetitions=2, width=8)
    q = write_query(narrow, True, directory=str(tmp_path))
    path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "layered"})
    assert capi.Plan(path).stats["tc_tiles"] == 1
    path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "layered", "spnb-tc-tiles": "1"})
    with pytest.raises(capi.SpnbError, match="spnb-tc-tiles"):
        capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-tc-tiles": "3"})


def test_bench_batch_is_the_same_for_every_gpu_count():
    """bench.py cuts ONE batch into one shard per rank (strong scaling): the shards of 2, 4 and 8 ranks put
    together are the batch a single rank evaluates."""
    import bench
    from spnb import synth
    spn = synth.config2(target_nodes=300)
    n = 8 * 1000 + 8
    whole = bench.shard_inputs(2, spn, n, 1, 0)
    assert whole.shape == (n, 26)
    for world in (2, 4, 8):
        parts = [bench.shard_inputs(2, spn, n, world, r) for r in range(world)]
        assert np.array_equal(np.concatenate(parts), whole)
        assert sum(len(p) for p in parts) == n
