"""Binary (Cap'n Proto) serialisation of SPN models and queries.

Same surface as the reference's xspn/xspn/serialization/binary/BinarySerialization.py:53-81 and :254-370
(`BinarySerializer(fileName).serialize_to_file(modelOrQuery)`,
`BinaryDeserializer(fileName).deserialize_from_file()`), and the same steps before writing (:106-129):
validity check, file-unique ids, bottom-up scope rebuild, nodes listed children-before-parents.
The encoding and decoding themselves are done by `wire` (no pycapnp).
"""
import numpy as np

from xspn.structure.Model import SPNModel
from xspn.structure.Query import ErrorKind, ErrorModel, JointProbability, Query
from xspn.structure import Nodes
from xspn.serialization.binary import wire

_KIND_CODE = {"product": wire.K_PRODUCT, "sum": wire.K_SUM, "histogram": wire.K_HIST,
              "gaussian": wire.K_GAUSS, "categorical": wire.K_CAT}
# enum ordinals of the schema (spflow.capnp:10-25)
_TYPE_ORD = {"real": 0, "interval": 1, "positive": 2, "categorical": 3, "ordinal": 4, "count": 5, "binary": 6}
_META_ORD = {"real": 0, "binary": 1, "discrete": 2}


def _enum_ord(value, table):
    if value is None:
        return 0
    name = getattr(value, "name", str(value)).lower()
    return table.get(name, 0)


def _item(v):
    return v.item() if type(v).__module__ == np.__name__ else v


class BinarySerializer:
    """Serialise an SPNModel or a Query into an xspn binary file."""

    def __init__(self, fileName, bufferSize=10 * (2 ** 10), clearFile=True):
        self.assignedIDs = {}
        self.fileName = fileName
        self.bufferSize = bufferSize
        if clearFile:
            open(fileName, "w").close()

    def serialize_to_file(self, content):
        data = self.serialize_to_bytes(content)
        with open(self.fileName, "a+b") as f:
            f.write(data)

    def serialize_to_bytes(self, content):
        if isinstance(content, SPNModel):
            return self._encode_model(content, None)
        if isinstance(content, Query):
            if not isinstance(content, JointProbability):
                raise NotImplementedError("No serialization defined for query %r of type %s" % (content, type(content)))
            kind = content.errorModel.kind
            if kind is ErrorKind.ABSOLUTE or kind == ErrorKind.ABSOLUTE:
                ek = 0
            elif kind is ErrorKind.RELATIVE or kind == ErrorKind.RELATIVE:
                ek = 1
            else:
                raise NotImplementedError("No serialization defined for error kind %r" % (kind,))
            q = {"batch_size": int(content.batchSize), "error_kind": ek, "max_error": float(content.errorModel.error),
                 "support_marginal": bool(content.supportsMarginal())}
            return self._encode_model(content.graph, q)
        raise NotImplementedError("No serialization defined for content %r of type %s" % (content, type(content)))

    def _encode_model(self, model, query):
        root = model.root
        Nodes.assign_ids(root, self.assignedIDs)
        Nodes.rebuild_scopes_bottom_up(root)
        ok, why = Nodes.is_valid(root)
        assert ok, "SPN invalid before serialization: %s" % why
        order = Nodes.topological_order(root)
        n = len(order)
        kind = np.zeros(n, np.int64)
        node_id = np.zeros(n, np.int64)
        scope_id = np.zeros(n, np.int64)
        mean = np.zeros(n)
        stddev = np.ones(n)
        hist_type = np.zeros(n, np.uint64)
        hist_meta = np.zeros(n, np.uint64)
        child_ptr, tab_ptr, brk_ptr, repr_ptr = [0], [0], [0], [0]
        child_id, weight, tab, brk, repr_pts = [], [], [], [], []
        for i, nd in enumerate(order):
            k = Nodes.kind_of(nd)
            kind[i] = _KIND_CODE[k]
            node_id[i] = nd.id
            if k in ("sum", "product"):
                child_id.extend(c.id for c in nd.children)
                if k == "sum":
                    weight.extend(float(_item(w)) for w in nd.weights)
                else:
                    weight.extend(0.0 for _ in nd.children)
            else:
                assert len(nd.scope) == 1, "Expecting leaf to be univariate"
                scope_id[i] = int(_item(nd.scope[0]))
                if k == "gaussian":
                    mean[i] = float(_item(nd.mean))
                    stddev[i] = float(_item(nd.stdev))
                elif k == "categorical":
                    tab.extend(float(_item(p)) for p in nd.p)
                else:
                    brk.extend(int(b) for b in nd.breaks)
                    tab.extend(float(_item(d)) for d in nd.densities)
                    repr_pts.extend(float(_item(r)) for r in (nd.bin_repr_points or []))
                    hist_type[i] = _enum_ord(getattr(nd, "type", None), _TYPE_ORD)
                    hist_meta[i] = _enum_ord(getattr(nd, "meta_type", None), _META_ORD)
            child_ptr.append(len(child_id))
            tab_ptr.append(len(tab))
            brk_ptr.append(len(brk))
            repr_ptr.append(len(repr_pts))
        return wire.encode_flat(
            kind=kind, node_id=node_id, child_ptr=child_ptr, child_id=np.asarray(child_id, np.int32),
            weight=np.asarray(weight, np.float64), scope_id=scope_id, mean=mean, stddev=stddev,
            tab_ptr=tab_ptr, tab=np.asarray(tab, np.float64), brk_ptr=brk_ptr, brk=np.asarray(brk, np.int32),
            root_id=root.id, scope=[int(_item(s)) for s in root.scope], feature_type=str(model.featureType),
            name=model.name or "", query=query, repr_ptr=repr_ptr, repr_pts=np.asarray(repr_pts, np.float64),
            hist_type=hist_type, hist_meta=hist_meta)


_TYPE_NAME = {v: k for k, v in _TYPE_ORD.items()}
_META_NAME = {v: k for k, v in _META_ORD.items()}


class BinaryDeserializer:
    """Read an SPNModel or a JointProbability query back from an xspn binary file.

    Nodes come back as xspn.structure.Nodes objects (SPFlow's attribute names), children resolved by id,
    scopes rebuilt bottom-up and the structure checked, as the reference does after reading
    (BinarySerialization.py:295-312).  Histogram `type` / `meta_type` come back as the lower-case names of
    the schema's enumerants."""

    def __init__(self, fileName):
        self.fileName = fileName

    def deserialize_from_file(self):
        with open(self.fileName, "rb") as f:
            return self.deserialize_from_bytes(f.read())

    def deserialize_from_bytes(self, data):
        msg = wire.decode_message(data)
        model = self._model(msg)
        q = msg["query"]
        if q is None:
            return model
        if q["error_kind"] == 0:
            kind = ErrorKind.ABSOLUTE
        elif q["error_kind"] == 1:
            kind = ErrorKind.RELATIVE
        else:
            raise NotImplementedError("Cannot deserialize error kind %r" % (q["error_kind"],))
        return JointProbability(model, q["batch_size"], q["support_marginal"], ErrorModel(kind, q["max_error"]))

    def _model(self, msg):
        by_id, roots = {}, []
        for nd in msg["nodes"]:
            k = nd["kind"]
            if k in (wire.K_PRODUCT, wire.K_SUM):
                kids = [by_id.get(c) for c in nd["children"]]
                assert None not in kids, "Child node ID could not be resolved"
                node = Nodes.Product(children=kids) if k == wire.K_PRODUCT else Nodes.Sum(weights=nd["weights"], children=kids)
            elif k == wire.K_HIST:
                node = Nodes.Histogram(nd["breaks"], nd["densities"], nd["bin_repr_points"], scope=nd["scope"],
                                       type_=_TYPE_NAME.get(nd["type"]), meta_type=_META_NAME.get(nd["meta_type"]))
            elif k == wire.K_GAUSS:
                node = Nodes.Gaussian(nd["mean"], nd["stddev"], nd["scope"])
            else:
                node = Nodes.Categorical(p=nd["probabilities"], scope=nd["scope"])
            node.id = nd["id"]
            by_id[node.id] = node
            if nd["root"]:
                roots.append(node)
        for r in roots:
            Nodes.rebuild_scopes_bottom_up(r)
            ok, why = Nodes.is_valid(r)
            assert ok, "SPN invalid after deserialization: %s" % why
        root = next((r for r in roots if r.id == msg["root_id"]), None)
        if root is None:
            raise ValueError("Did not find serialized root node %d" % msg["root_id"])
        return SPNModel(root, msg["feature_type"], msg["name"] or None)
