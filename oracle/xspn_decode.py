"""TEST INFRASTRUCTURE (oracle) -- independent pure-Python decoder of xspn binary files.

This file belongs to the CPU oracle.  It is used only by the tests, by the smoke
check and by the CPU-baseline leg of the benchmark; the product (the CUDA engine and
its C++ front end) never imports it.  It is deliberately a second, unrelated
implementation of the wire format so that a decoding bug in the product's C++ reader
cannot hide behind an identical bug here.

Format followed: the Cap'n Proto schema of the reference
(xspn/xspn/serialization/binary/capnproto/spflow.capnp:27-101) in the standard
unpacked stream framing, as written by the reference's serialiser
(xspn/xspn/serialization/binary/BinarySerialization.py:71-81).  The semantic steps
(sorted scope -> input column, buckets from breaks/densities, type-string parsing,
default kernel name) follow the reference's front end
(compiler/src/pipeline/steps/frontend/SPFlowToMLIRDeserializer.cpp:74-140,162-258).
"""
import re
import struct

import numpy as np

KIND_PRODUCT, KIND_SUM, KIND_HIST, KIND_GAUSS, KIND_CAT = 0, 1, 2, 3, 4


class _Msg:
    """Random access to the segments of one Cap'n Proto message."""

    def __init__(self, data: bytes):
        self.data = data
        (nseg_m1,) = struct.unpack_from("<I", data, 0)
        nseg = nseg_m1 + 1
        sizes = struct.unpack_from("<%dI" % nseg, data, 4)
        hdr = 4 + 4 * nseg
        hdr = (hdr + 7) & ~7
        self.seg_off = []
        off = hdr
        for s in sizes:
            self.seg_off.append(off)
            off += 8 * s
        self.seg_words = list(sizes)
        if off > len(data):
            raise ValueError("xspn file truncated: segment table exceeds file size")

    def word(self, seg, w):
        if w < 0 or w >= self.seg_words[seg]:
            raise ValueError("pointer outside segment")
        return struct.unpack_from("<Q", self.data, self.seg_off[seg] + 8 * w)[0]

    def byte_off(self, seg, w):
        return self.seg_off[seg] + 8 * w

    # -- pointer resolution -------------------------------------------------
    def resolve(self, seg, w):
        """Follow far pointers. Returns (seg, pointer_word_value, target_word_index) where
        target_word_index is the index of the first content word, or None for null."""
        p = self.word(seg, w)
        if p == 0:
            return None
        kind = p & 3
        if kind != 2:
            off = _s30(p)
            return seg, p, w + 1 + off
        # far pointer
        double = (p >> 2) & 1
        pad = (p >> 3) & 0x1FFFFFFF
        tseg = p >> 32
        if not double:
            q = self.word(tseg, pad)
            if q & 3 == 2:
                raise ValueError("far pointer landing pad is itself far")
            return tseg, q, pad + 1 + _s30(q)
        q = self.word(tseg, pad)          # far pointer to the content
        tag = self.word(tseg, pad + 1)    # describes the content, offset field unused
        if q & 3 != 2 or (q >> 2) & 1:
            raise ValueError("malformed double-far landing pad")
        return q >> 32, tag, (q >> 3) & 0x1FFFFFFF


def _s30(p):
    v = (p >> 2) & 0x3FFFFFFF
    return v - (1 << 30) if v & (1 << 29) else v


class _Struct:
    def __init__(self, msg, seg, w, dwords, pwords):
        self.msg, self.seg, self.w, self.dwords, self.pwords = msg, seg, w, dwords, pwords

    def _get(self, fmt, byte, size):
        if byte + size > 8 * self.dwords:
            return 0  # field beyond the stored data section keeps its default
        return struct.unpack_from(fmt, self.msg.data, self.msg.byte_off(self.seg, self.w) + byte)[0]

    def i32(self, byte):
        return self._get("<i", byte, 4)

    def u16(self, byte):
        return self._get("<H", byte, 2)

    def f64(self, byte):
        v = self._get("<d", byte, 8)
        return float(v)

    def bit(self, byte, bit):
        return (self._get("<B", byte, 1) >> bit) & 1

    def _ptr(self, i):
        if i >= self.pwords:
            return None
        return self.msg.resolve(self.seg, self.w + self.dwords + i)

    def struct(self, i):
        r = self._ptr(i)
        if r is None:
            return None
        seg, p, tw = r
        if p & 3 != 0:
            raise ValueError("expected a struct pointer")
        return _Struct(self.msg, seg, tw, (p >> 32) & 0xFFFF, (p >> 48) & 0xFFFF)

    def prim_list(self, i, dtype):
        r = self._ptr(i)
        if r is None:
            return np.zeros(0, dtype=dtype)
        seg, p, tw = r
        if p & 3 != 1:
            raise ValueError("expected a list pointer")
        esz = (p >> 32) & 7
        cnt = p >> 35
        want = {1: 2, 4: 4, 8: 5}[np.dtype(dtype).itemsize]
        if esz != want:
            raise ValueError("list element size %d does not match %s" % (esz, dtype))
        nbytes = cnt * np.dtype(dtype).itemsize
        if 8 * tw + nbytes > 8 * self.msg.seg_words[seg]:
            raise ValueError("list exceeds its segment")
        return np.frombuffer(self.msg.data, dtype=np.dtype(dtype).newbyteorder("<"), count=cnt,
                             offset=self.msg.byte_off(seg, tw)).astype(dtype)

    def text(self, i):
        b = self.prim_list(i, np.uint8)
        return bytes(b[:-1]).decode("utf-8") if len(b) else ""

    def struct_list(self, i):
        r = self._ptr(i)
        if r is None:
            return []
        seg, p, tw = r
        if p & 3 != 1 or (p >> 32) & 7 != 7:
            raise ValueError("expected an inline-composite list")
        tag = self.msg.word(seg, tw)
        cnt = (tag >> 2) & 0x3FFFFFFF
        dw, pw = (tag >> 32) & 0xFFFF, (tag >> 48) & 0xFFFF
        step = dw + pw
        if tw + 1 + cnt * step > self.msg.seg_words[seg]:
            raise ValueError("struct list exceeds its segment")
        return [_Struct(self.msg, seg, tw + 1 + k * step, dw, pw) for k in range(cnt)]


def parse_feature_type(text):
    """numpy dtype name -> (kind, bits); kind is 'int' (signedness dropped, as in the
    reference, SPFlowToMLIRDeserializer.cpp:226-248) or 'float'."""
    m = re.fullmatch(r"(u?)int([1-9]+)", text)
    if m:
        return ("uint" if m.group(1) else "int"), int(m.group(2))
    m = re.fullmatch(r"float([1-9]+)", text)
    if m and int(m.group(1)) in (16, 32, 64):
        return "float", int(m.group(1))
    raise ValueError("Unsupported feature data type " + text)


def decode_xspn(path_or_bytes):
    """Decode an xspn file into a dict of flat numpy arrays (nodes in file order)."""
    data = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
    msg = _Msg(bytes(data))
    r = msg.resolve(0, 0)
    if r is None:
        raise ValueError("empty message")
    seg, p, tw = r
    header = _Struct(msg, seg, tw, (p >> 32) & 0xFFFF, (p >> 48) & 0xFFFF)
    out = {"is_query": bool(header.u16(0) == 1), "batch_size": 1, "error_kind": 0, "max_error": 0.0,
           "support_marginal": False}
    if out["is_query"]:
        q = header.struct(0)
        out["batch_size"] = q.i32(0)
        out["error_kind"] = q.u16(4)
        out["max_error"] = q.f64(8)
        joint = q.struct(0)
        if joint is None:
            raise ValueError("Can only deserialize joint queries")
        out["support_marginal"] = bool(joint.bit(0, 0))
        model = joint.struct(0)
        if model is None:
            raise ValueError("No model attached to query")
    else:
        model = header.struct(0)
    root_id = model.i32(0)
    out["num_features"] = model.i32(4)
    out["name"] = model.text(0) or "spn_kernel"
    out["feature_type"] = model.text(1)
    scope = np.sort(model.prim_list(2, np.int32))
    col_of = {int(s): i for i, s in enumerate(scope)}
    out["scope"] = scope

    nodes = model.struct_list(3)
    n = len(nodes)
    kind = np.zeros(n, np.int32)
    feature = np.full(n, -1, np.int32)
    mean = np.zeros(n, np.float64)
    stddev = np.ones(n, np.float64)
    child_ptr = np.zeros(n + 1, np.int64)
    tab_ptr = np.zeros(n + 1, np.int64)
    brk_ptr = np.zeros(n + 1, np.int64)
    children, weights, tabs, brks = [], [], [], []
    index_of = {}
    for k, nd in enumerate(nodes):
        nid = nd.i32(0)
        index_of[nid] = k
        which = nd.u16(6)
        body = nd.struct(0)
        kind[k] = which
        if which == KIND_PRODUCT:
            children.append(body.prim_list(0, np.int32))
            weights.append(np.zeros(len(children[-1])))
        elif which == KIND_SUM:
            children.append(body.prim_list(0, np.int32))
            weights.append(body.prim_list(1, np.float64))
            if len(weights[-1]) != len(children[-1]):
                raise ValueError("Number of weights must match the number of addends!")
        else:
            children.append(np.zeros(0, np.int32))
            weights.append(np.zeros(0))
        if which == KIND_HIST:
            b = body.prim_list(0, np.int32)
            d = body.prim_list(1, np.float64)
            feature[k] = col_of[body.i32(4)]
            brks.append(b)
            tabs.append(d[: max(len(b) - 1, 0)])
        elif which == KIND_GAUSS:
            mean[k], stddev[k] = body.f64(0), body.f64(8)
            feature[k] = col_of[body.i32(16)]
            brks.append(np.zeros(0, np.int32))
            tabs.append(np.zeros(0))
        elif which == KIND_CAT:
            feature[k] = col_of[body.i32(0)]
            brks.append(np.zeros(0, np.int32))
            tabs.append(body.prim_list(0, np.float64))
        else:
            brks.append(np.zeros(0, np.int32))
            tabs.append(np.zeros(0))
        child_ptr[k + 1] = child_ptr[k] + len(children[-1])
        tab_ptr[k + 1] = tab_ptr[k] + len(tabs[-1])
        brk_ptr[k + 1] = brk_ptr[k] + len(brks[-1])
    cat = np.concatenate(children) if children else np.zeros(0, np.int32)
    try:
        child_idx = np.array([index_of[int(c)] for c in cat], np.int32)
    except KeyError as e:
        raise ValueError("No definition found for node with ID: %s" % e)
    out.update(kind=kind, feature=feature, mean=mean, stddev=stddev, child_ptr=child_ptr,
               child_idx=child_idx, weights=np.concatenate(weights) if weights else np.zeros(0),
               tab_ptr=tab_ptr, tab=np.concatenate(tabs) if tabs else np.zeros(0),
               brk_ptr=brk_ptr, brk=np.concatenate(brks).astype(np.int32) if brks else np.zeros(0, np.int32),
               root=index_of[root_id])
    return out
