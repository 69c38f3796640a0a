"""GPU tests written like the reference's own CUDA tests (python-interface/test/cuda/*.py): a small
hand-built SPN, a few dozen random samples through `CUDACompiler().log_likelihood`, results compared
with np.isclose defaults; the expected values come from the CPU oracle instead of SPFlow."""
import os
import tempfile

import numpy as np
import pytest

from oracle import oracle
from xspn.serialization.binary.BinarySerialization import BinarySerializer
from xspn.structure.Model import SPNModel
from xspn.structure.Nodes import Categorical, Gaussian, Histogram, Product, Sum
from xspn.structure.Query import JointProbability

pytestmark = pytest.mark.gpu


def _expected(spn, inputs, marginal, mode):
    with tempfile.NamedTemporaryFile(suffix=".bin") as f:
        BinarySerializer(f.name).serialize_to_file(
            JointProbability(SPNModel(spn, str(inputs.dtype), "ref"), batchSize=64, supportMarginal=marginal))
        return oracle.evaluate(oracle.load_model(f.name), inputs, mode)


def _check(results, reference):
    assert results.shape == reference.shape
    for i, (r, e) in enumerate(zip(results, reference)):
        ok = np.isclose(r, e) or np.isclose(np.exp(r), np.exp(e)) or (np.isinf(e) and r == e)
        assert ok, f"evaluation #{i} failed: result: {r:16.8f}, reference: {e:16.8f}"


def _gaussian_spn():
    g = [Gaussian(mean=m, stdev=s, scope=f) for f, (m, s) in enumerate(
        [(0.11, 1.0), (0.12, 0.75), (0.13, 0.5), (0.14, 0.25), (0.15, 1.0), (0.16, 0.25), (0.17, 0.5), (0.18, 0.75),
         (0.19, 1.0), (0.20, 1.0)])]
    p0 = Product([g[0], g[1]])
    p1 = Product([g[2], g[3], g[4]])
    p2 = Product([g[5], g[6], g[7], g[8], g[9]])
    return Product([p0, p1, p2])


def _categorical_spn():
    c = [Categorical(p=p, scope=f) for f, p in enumerate(
        [[0.35, 0.55, 0.1], [0.25, 0.625, 0.125], [0.5, 0.2, 0.3], [0.6, 0.15, 0.25], [0.7, 0.11, 0.19],
         [0.8, 0.14, 0.06]])]
    p = Product([c[0], Sum([0.3, 0.7], [c[1], Categorical(p=[0.1, 0.8, 0.1], scope=1)]), c[2]])
    q = Product([c[3], c[4], c[5]])
    return Product([p, q])


def _histogram_spn():
    h1 = Histogram([0., 1., 2.], [0.25, 0.75], [1, 1], scope=0)
    h2 = Histogram([0., 1., 2.], [0.45, 0.55], [1, 1], scope=1)
    h3 = Histogram([0., 1., 2.], [0.33, 0.67], [1, 1], scope=0)
    h4 = Histogram([0., 1., 2.], [0.875, 0.125], [1, 1], scope=1)
    return Sum([0.3, 0.7], [Product([h1, h2]), Product([h3, h4])])


def test_cuda_gaussian():
    from spnc.gpu import CUDACompiler
    assert CUDACompiler.isAvailable()
    rng = np.random.default_rng(1)
    inputs = rng.normal(0.5, 1.0, size=(30, 10)).astype(np.float64)
    for log_space, mode in ((True, "log_f64"), (False, "linear_f64")):
        res = CUDACompiler(computeInLogSpace=log_space).log_likelihood(_gaussian_spn(), inputs, supportMarginal=False)
        assert res.dtype == (np.float32 if log_space else np.float64)
        _check(res, _expected(_gaussian_spn(), inputs, False, mode))


def test_marginal_cuda_gaussian():
    from spnc.gpu import CUDACompiler
    rng = np.random.default_rng(2)
    inputs = rng.normal(0.5, 1.0, size=(30, 10)).astype(np.float32)
    inputs[rng.random(inputs.shape) < 0.3] = np.nan
    inputs[0, :] = np.nan
    res = CUDACompiler().log_likelihood(_gaussian_spn(), inputs)
    assert res[0] == 0.0
    _check(res, _expected(_gaussian_spn(), inputs, True, "log_f64"))


def test_cuda_categorical_and_marginal():
    from spnc.gpu import CUDACompiler
    rng = np.random.default_rng(3)
    inputs = rng.integers(0, 3, size=(30, 6)).astype(np.float64)
    res = CUDACompiler().log_likelihood(_categorical_spn(), inputs, supportMarginal=False)
    _check(res, _expected(_categorical_spn(), inputs, False, "log_f64"))
    inputs[rng.random(inputs.shape) < 0.3] = np.nan
    inputs[1, 0] = 7  # outside every table: impossible evidence
    res = CUDACompiler().log_likelihood(_categorical_spn(), inputs, supportMarginal=True)
    assert res[1] == -np.inf
    _check(res, _expected(_categorical_spn(), inputs, True, "log_f64"))
    ints = rng.integers(0, 3, size=(30, 6)).astype(np.int32)
    res = CUDACompiler().log_likelihood(_categorical_spn(), ints, supportMarginal=False)
    _check(res, _expected(_categorical_spn(), ints, False, "log_f64"))
    with pytest.raises(RuntimeError):  # the default supportMarginal=True needs floating inputs
        CUDACompiler().log_likelihood(_categorical_spn(), ints)


def test_cuda_histogram_int_and_float_inputs():
    from spnc.gpu import CUDACompiler
    rng = np.random.default_rng(4)
    ints = rng.integers(0, 2, size=(30, 2)).astype(np.int32)
    res = CUDACompiler().log_likelihood(_histogram_spn(), ints, supportMarginal=False)
    _check(res, _expected(_histogram_spn(), ints, False, "log_f64"))
    flt = ints.astype(np.float32)
    flt[::5, 1] = np.nan
    res = CUDACompiler().log_likelihood(_histogram_spn(), flt)
    _check(res, _expected(_histogram_spn(), flt, True, "log_f64"))


def test_compile_once_execute_many():
    from spnc.gpu import CUDACompiler
    comp = CUDACompiler()
    kernel = comp.compile_ll(_gaussian_spn(), inputDataType="float32", supportMarginal=False)
    rng = np.random.default_rng(5)
    for n in (1, 64, 65, 1000):
        x = rng.normal(size=(n, 10)).astype(np.float32)
        _check(comp.execute(kernel, x), _expected(_gaussian_spn(), x, False, "log_f64"))
    # Fortran-ordered input is made contiguous instead of being read as garbage
    x = np.asfortranarray(rng.normal(size=(50, 10)).astype(np.float32))
    _check(comp.execute(kernel, x), _expected(_gaussian_spn(), np.ascontiguousarray(x), False, "log_f64"))
    os.remove(kernel.fileName())


def test_sharded_entry_on_the_visible_devices(tmp_path):
    from spnb import capi, synth
    from tests.util_models import write_query, max_rel_err, REL_TOL_F32
    spn = synth.config2(target_nodes=600)
    q = write_query(spn, True, directory=str(tmp_path))
    plan_path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true"})
    plan = capi.Plan(plan_path)
    x = synth.config2_inputs(300001, 11)
    devs = list(range(capi.device_count()))
    out, mean = plan.execute_sharded(devs + devs[:1], x, want_mean=True)  # a device may appear twice
    want = oracle.evaluate(oracle.load_model(q), x, "log_f64")
    assert max_rel_err(out, want) <= REL_TOL_F32
    assert abs(mean - want.mean()) <= 1e-4 * abs(want.mean())


def test_partitioned_cuda_NIPS5(golden_dir):
    """The reference's partitioned CUDA test (python-interface/test/examples/NIPS5/test_partitioned_cuda_NIPS5.py:24-42):
    the stored NIPS5 query read back with BinaryDeserializer, compiled with computeInLogSpace=False and
    maxTaskSize=10, i.e. cut into functions of at most ten nodes whose results travel through global scratch."""
    from spnc.gpu import CUDACompiler
    from xspn.serialization.binary.BinarySerialization import BinaryDeserializer
    query = BinaryDeserializer(os.path.join(golden_dir, "NIPS5.bin")).deserialize_from_file()
    spn = query.graph.root
    z = np.load(os.path.join(golden_dir, "NIPS5_io.npz"))
    inputs, reference = z["inputs"].astype(np.int32), z["outputs"].reshape(-1)
    results = CUDACompiler(computeInLogSpace=False, maxTaskSize=10).log_likelihood(spn, inputs, supportMarginal=False)
    assert results.dtype == np.float64
    assert np.all(np.isclose(results, reference)) or np.all(np.isclose(np.exp(results), np.exp(reference)))
    # the option really partitions: the generated source passes values through the scratch area
    kernel = CUDACompiler(computeInLogSpace=False, maxTaskSize=10).compile_ll(spn, "int32", supportMarginal=False)
    from spnb import capi
    plan = capi.Plan(kernel.fileName())
    assert plan.stats["scratch_slots"] > 0 and "st.global" in plan.source
    plan.close()
    os.remove(kernel.fileName())
