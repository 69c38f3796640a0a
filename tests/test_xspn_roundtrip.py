"""Round trip of the xspn binary format through the package's own writer and reader, shaped after the
reference's xspn/test/serialization/binary/test_binary_serialization_roundtrip.py:19-124 (which needs SPFlow
and pycapnp; the node classes of xspn.structure.Nodes stand in for SPFlow's here), plus the stored example
files of the reference read back node for node."""
import os

import numpy as np

from xspn.serialization.binary.BinarySerialization import BinaryDeserializer, BinarySerializer
from xspn.structure.Model import SPNModel
from xspn.structure.Nodes import Categorical, Gaussian, Histogram, Product, Sum, topological_order
from xspn.structure.Query import ErrorKind, ErrorModel, JointProbability


def _count(root, cls=None):
    return sum(1 for n in topological_order(root) if cls is None or isinstance(n, cls))


def _edges(root):
    return sum(len(getattr(n, "children", [])) for n in topological_order(root))


def test_binary_serialization_roundtrip(tmp_path):
    h1 = Histogram([0, 1, 2], [0.25, 0.75], [1, 1], scope=1)
    h2 = Histogram([0, 1, 2], [0.45, 0.55], [1, 1], scope=2)
    h3 = Histogram([0, 1, 2], [0.33, 0.67], [1, 1], scope=1)
    h4 = Histogram([0, 1, 2], [0.875, 0.125], [1, 1], scope=2)
    spn = Sum([0.3, 0.7], [Product(children=[h1, h2]), Product(children=[h3, h4])])
    model = SPNModel(spn, featureValueType="uint32")
    query = JointProbability(model)
    path = str(tmp_path / "test.bin")
    BinarySerializer(path).serialize_to_file(query)
    back = BinaryDeserializer(path).deserialize_from_file()
    assert isinstance(back, JointProbability)
    assert back.batchSize == query.batchSize
    assert back.errorModel.error == query.errorModel.error
    assert back.errorModel.kind == query.errorModel.kind
    assert back.graph.featureType == model.featureType
    assert back.graph.name == model.name
    root = back.graph.root
    assert _count(spn) == _count(root)
    for cls in (Sum, Product, Histogram):
        assert _count(spn, cls) == _count(root, cls)
    assert _edges(spn) == _edges(root)
    assert list(root.weights) == [0.3, 0.7]
    assert root.children[1].children[0].densities == [0.33, 0.67] and root.children[1].children[0].breaks == [0, 1, 2]
    assert root.children[0].children[1].bin_repr_points == [1.0, 1.0]


def test_categorical_leaf_serialization(tmp_path):
    c1 = Categorical(p=[0.35, 0.55, 0.1], scope=1)
    c2 = Categorical(p=[0.25, 0.625, 0.125], scope=2)
    model = SPNModel(Product(children=[c1, c2]), "uint8", "test")
    path = str(tmp_path / "test.bin")
    BinarySerializer(path).serialize_to_file(JointProbability(model))
    back = BinaryDeserializer(path).deserialize_from_file()
    assert isinstance(back, JointProbability) and isinstance(back.graph, SPNModel)
    assert back.graph.featureType == "uint8" and back.graph.name == "test"
    root = back.graph.root
    assert isinstance(root, Product) and len(root.children) == 2
    assert list(root.children[0].p) == c1.p and list(root.children[1].p) == c2.p


def test_gaussian_leaf_serialization(tmp_path):
    g1 = Gaussian(mean=0.5, stdev=1, scope=0)
    g2 = Gaussian(mean=0.125, stdev=0.25, scope=1)
    model = SPNModel(Product(children=[g1, g2]), "float32", "test")
    path = str(tmp_path / "test.bin")
    BinarySerializer(path).serialize_to_file(
        JointProbability(model, batchSize=7, supportMarginal=True, rootError=ErrorModel(ErrorKind.RELATIVE, 0.125)))
    back = BinaryDeserializer(path).deserialize_from_file()
    assert (back.batchSize, back.supportsMarginal(), back.errorModel.kind, back.errorModel.error) == \
        (7, True, ErrorKind.RELATIVE, 0.125)
    a, b = back.graph.root.children
    assert (a.scope, a.mean, a.stdev) == (g1.scope, 0.5, 1.0)
    assert (b.scope, b.mean, b.stdev) == (g2.scope, 0.125, 0.25)


def test_model_header_roundtrip_and_rewrite_is_stable(tmp_path, golden_dir):
    """A stored model of the reference (bare model header) is read, written again and read again: the second
    file is byte-identical to the first rewrite and both readers of this repository agree on it."""
    from oracle import xspn_decode
    for name in ("NIPS5.bin", "nltcs.bin"):
        src = os.path.join(golden_dir, name)
        first = BinaryDeserializer(src).deserialize_from_file()
        a = str(tmp_path / ("a_" + name))
        BinarySerializer(a).serialize_to_file(first)
        second = BinaryDeserializer(a).deserialize_from_file()
        b = str(tmp_path / ("b_" + name))
        BinarySerializer(b).serialize_to_file(second)
        assert open(a, "rb").read() == open(b, "rb").read()
        d0, d1 = xspn_decode.decode_xspn(src), xspn_decode.decode_xspn(a)
        assert d0["is_query"] == d1["is_query"] and d0["feature_type"] == d1["feature_type"]
        assert len(d0["kind"]) == len(d1["kind"])
        assert sorted(d0["kind"].tolist()) == sorted(d1["kind"].tolist())
        assert np.isclose(np.sort(d0["weights"]), np.sort(d1["weights"])).all()
