"""Cap'n Proto encoder and decoder for xspn files, written against the reference's schema
(xspn/xspn/serialization/binary/capnproto/spflow.capnp:27-101) without pycapnp.

The whole message is laid out in ONE segment in the standard unpacked stream framing
(u32 segment count - 1, u32 segment size in words, then the segment), which every Cap'n Proto
reader accepts.  All per-node work is vectorised with numpy so that models with 10^5..10^6
nodes and 10^7 edges serialise in seconds.

Node kinds use the schema's union order: 0 product, 1 sum, 2 histogram, 3 gaussian, 4 categorical.
"""
import numpy as np

K_PRODUCT, K_SUM, K_HIST, K_GAUSS, K_CAT = 0, 1, 2, 3, 4


def _struct_ptr(off, dwords, pwords):
    return ((np.asarray(off, np.int64) << 2) & 0xFFFFFFFC).astype(np.uint64) \
        | (np.uint64(dwords) << np.uint64(32)) | (np.uint64(pwords) << np.uint64(48))


def _list_ptr(off, esz, count):
    return (((np.asarray(off, np.int64) << 2) & 0xFFFFFFFC) | 1).astype(np.uint64) \
        | (np.uint64(esz) << np.uint64(32)) | (np.asarray(count, np.uint64) << np.uint64(35))


def _text_words(s):
    b = s.encode("utf-8") + b"\0"
    pad = (-len(b)) % 8
    return np.frombuffer(b + b"\0" * pad, dtype="<u8"), len(b)


def encode_flat(*, kind, node_id, child_ptr, child_id, weight, scope_id, mean, stddev, tab_ptr, tab,
                brk_ptr, brk, root_id, scope, feature_type, name="", query=None,
                repr_ptr=None, repr_pts=None, hist_type=None, hist_meta=None):
    """Encode a model given as flat arrays.  `query` is None (model header) or a dict
    {batch_size, error_kind (0 absolute / 1 relative), max_error, support_marginal}."""
    kind = np.asarray(kind, np.int64)
    n = len(kind)
    node_id = np.asarray(node_id, np.int64)
    child_ptr = np.asarray(child_ptr, np.int64)
    tab_ptr = np.asarray(tab_ptr, np.int64)
    brk_ptr = np.asarray(brk_ptr, np.int64)
    k = np.diff(child_ptr)
    nt = np.diff(tab_ptr)
    nb = np.diff(brk_ptr)
    if repr_ptr is None:
        repr_ptr = np.zeros(n + 1, np.int64)
        repr_pts = np.zeros(0)
    repr_ptr = np.asarray(repr_ptr, np.int64)
    nr = np.diff(repr_ptr)
    cw = (k + 1) // 2
    bw = (nb + 1) // 2
    body = np.select([kind == K_PRODUCT, kind == K_SUM, kind == K_HIST, kind == K_GAUSS, kind == K_CAT],
                     [1 + cw, 2 + cw + k, 4 + bw + nt + nr, np.full(n, 3), 2 + nt])

    # ---- fixed head ------------------------------------------------------------------
    head = []  # list of (word index, value) filled below; simple python, tiny
    is_query = query is not None
    w_header = 1
    pos = 3
    if is_query:
        w_query = pos; pos += 3
        w_joint = pos; pos += 2
    w_model = pos; pos += 5
    name_words, name_len = _text_words(name or "")
    ft_words, ft_len = _text_words(feature_type)
    scope = np.asarray(scope, np.int32)
    w_name = pos; pos += len(name_words)
    w_ft = pos; pos += len(ft_words)
    w_scope = pos; pos += (len(scope) + 1) // 2
    w_nodes = pos; pos += 1 + 2 * n
    base = pos + np.concatenate(([0], np.cumsum(body)[:-1])) if n else np.zeros(0, np.int64)
    total = int(pos + body.sum())
    if total >= (1 << 29):
        raise ValueError("model too large for a single-segment xspn file")
    W = np.zeros(total, dtype=np.uint64)

    W[0] = _struct_ptr(0, 1, 1)
    W[w_header] = np.uint64(1 if is_query else 0)
    if is_query:
        W[w_header + 1] = _struct_ptr(w_query - (w_header + 2), 2, 1)
        W[w_query] = np.uint64(int(query["batch_size"]) & 0xFFFFFFFF) | (np.uint64(int(query["error_kind"])) << np.uint64(32))
        W[w_query + 1] = np.array([float(query["max_error"])], "<f8").view("<u8")[0]
        W[w_query + 2] = _struct_ptr(w_joint - (w_query + 3), 1, 1)
        W[w_joint] = np.uint64(1 if query["support_marginal"] else 0)
        W[w_joint + 1] = _struct_ptr(w_model - (w_joint + 2), 1, 4)
    else:
        W[w_header + 1] = _struct_ptr(w_model - (w_header + 2), 1, 4)
    W[w_model] = np.uint64(int(root_id) & 0xFFFFFFFF) | (np.uint64(len(scope)) << np.uint64(32))
    W[w_model + 1] = _list_ptr(w_name - (w_model + 2), 2, name_len)
    W[w_model + 2] = _list_ptr(w_ft - (w_model + 3), 2, ft_len)
    W[w_model + 3] = _list_ptr(w_scope - (w_model + 4), 4, len(scope))
    W[w_model + 4] = _list_ptr(w_nodes - (w_model + 5), 7, 2 * n)
    W[w_name:w_name + len(name_words)] = name_words
    W[w_ft:w_ft + len(ft_words)] = ft_words
    W32 = W.view("<u4")
    W32[2 * w_scope:2 * w_scope + len(scope)] = scope.view(np.uint32)
    # tag word of the node list: element count in the offset field, 1 data word, 1 pointer
    W[w_nodes] = _struct_ptr(n, 1, 1)
    if n == 0:
        return _frame(W)

    # ---- node headers ----------------------------------------------------------------
    idx = np.arange(n, dtype=np.int64)
    w_data = w_nodes + 1 + 2 * idx
    is_root = (node_id == int(root_id)).astype(np.uint64)
    W[w_data] = (node_id & 0xFFFFFFFF).astype(np.uint64) | (is_root << np.uint64(32)) | (kind.astype(np.uint64) << np.uint64(48))
    dws = np.select([kind == K_PRODUCT, kind == K_SUM, kind == K_HIST, kind == K_GAUSS, kind == K_CAT], [0, 0, 1, 3, 1])
    pws = np.select([kind == K_PRODUCT, kind == K_SUM, kind == K_HIST, kind == K_GAUSS, kind == K_CAT], [1, 2, 3, 0, 1])
    W[w_data + 1] = (((base - (w_data + 2)) << 2) & 0xFFFFFFFC).astype(np.uint64) \
        | (dws.astype(np.uint64) << np.uint64(32)) | (pws.astype(np.uint64) << np.uint64(48))

    child_id = np.asarray(child_id, np.int32)
    weight = np.asarray(weight, np.float64)
    Wf = W.view("<f8")

    def edge_positions(mask, list_word, ptr):
        cnt = np.diff(ptr)[mask]
        if cnt.sum() == 0:
            return None, None
        lo = ptr[:-1][mask]
        src = np.repeat(lo, cnt) + _ranges(cnt)
        dst_base = np.repeat(list_word[mask], cnt)
        return src, (dst_base, _ranges(cnt))

    # products
    m = kind == K_PRODUCT
    if m.any():
        W[base[m]] = _list_ptr(0, 4, k[m])
        src, d = edge_positions(m, base + 1, child_ptr)
        if src is not None:
            W32[2 * d[0] + d[1]] = child_id[src].view(np.uint32)
    # sums
    m = kind == K_SUM
    if m.any():
        W[base[m]] = _list_ptr(1, 4, k[m])
        W[base[m] + 1] = _list_ptr(cw[m], 5, k[m])
        src, d = edge_positions(m, base + 2, child_ptr)
        if src is not None:
            W32[2 * d[0] + d[1]] = child_id[src].view(np.uint32)
        src, d = edge_positions(m, base + 2 + cw, child_ptr)
        if src is not None:
            Wf[d[0] + d[1]] = weight[src]
    # gaussians
    m = kind == K_GAUSS
    if m.any():
        Wf[base[m]] = np.asarray(mean, np.float64)[m]
        Wf[base[m] + 1] = np.asarray(stddev, np.float64)[m]
        W[base[m] + 2] = (np.asarray(scope_id, np.int64)[m] & 0xFFFFFFFF).astype(np.uint64)
    # categoricals
    tab = np.asarray(tab, np.float64)
    m = kind == K_CAT
    if m.any():
        W[base[m]] = (np.asarray(scope_id, np.int64)[m] & 0xFFFFFFFF).astype(np.uint64)
        W[base[m] + 1] = _list_ptr(0, 5, nt[m])
        src, d = edge_positions(m, base + 2, tab_ptr)
        if src is not None:
            Wf[d[0] + d[1]] = tab[src]
    # histograms
    m = kind == K_HIST
    if m.any():
        ht = np.zeros(n, np.uint64) if hist_type is None else np.asarray(hist_type, np.uint64)
        hm = np.zeros(n, np.uint64) if hist_meta is None else np.asarray(hist_meta, np.uint64)
        W[base[m]] = ht[m] | (hm[m] << np.uint64(16)) | ((np.asarray(scope_id, np.int64)[m] & 0xFFFFFFFF).astype(np.uint64) << np.uint64(32))
        W[base[m] + 1] = _list_ptr(2, 4, nb[m])
        W[base[m] + 2] = _list_ptr(1 + bw[m], 5, nt[m])
        W[base[m] + 3] = _list_ptr(bw[m] + nt[m], 5, nr[m])
        brk = np.asarray(brk, np.int32)
        src, d = edge_positions(m, base + 4, brk_ptr)
        if src is not None:
            W32[2 * d[0] + d[1]] = brk[src].view(np.uint32)
        src, d = edge_positions(m, base + 4 + bw, tab_ptr)
        if src is not None:
            Wf[d[0] + d[1]] = tab[src]
        src, d = edge_positions(m, base + 4 + bw + nt, repr_ptr)
        if src is not None:
            Wf[d[0] + d[1]] = np.asarray(repr_pts, np.float64)[src]
    return _frame(W)


def _ranges(cnt):
    """concatenate(arange(c) for c in cnt), vectorised"""
    cnt = np.asarray(cnt, np.int64)
    tot = int(cnt.sum())
    ends = np.cumsum(cnt)
    return np.arange(tot, dtype=np.int64) - np.repeat(ends - cnt, cnt)


def _frame(W):
    hdr = np.array([0, len(W)], dtype="<u4").tobytes()
    return hdr + W.astype("<u8").tobytes()


# ------------------------------------------------------------------------------------------------
# Reader.  Accepts any framing a Cap'n Proto writer may produce for the schema: several segments,
# far and double-far pointers, structs stored shorter than the schema (missing fields read as zero).
# ------------------------------------------------------------------------------------------------
import struct as _st


class _View:
    """The segments of one unpacked Cap'n Proto stream message."""

    def __init__(self, data):
        self.data = bytes(data)
        if len(self.data) < 8:
            raise ValueError("not an xspn file: shorter than a segment table")
        nseg = _st.unpack_from("<I", self.data, 0)[0] + 1
        if nseg > 4096 or 4 + 4 * nseg > len(self.data):
            raise ValueError("not an xspn file: bad segment count")
        words = _st.unpack_from("<%dI" % nseg, self.data, 4)
        at = (4 + 4 * nseg + 7) & ~7
        self.start, self.words = [], list(words)
        for w in words:
            self.start.append(at)
            at += 8 * w
        if at > len(self.data):
            raise ValueError("xspn file truncated")

    def u64(self, seg, w):
        if not (0 <= seg < len(self.words)) or not (0 <= w < self.words[seg]):
            raise ValueError("pointer leaves its segment")
        return _st.unpack_from("<Q", self.data, self.start[seg] + 8 * w)[0]

    def follow(self, seg, w):
        """Pointer at (seg, w) -> (seg, pointer value describing the object, first content word) or None."""
        p = self.u64(seg, w)
        if p == 0:
            return None
        if p & 3 != 2:
            off = (p >> 2) & 0x3FFFFFFF
            off -= (off & (1 << 29)) << 1
            return seg, p, w + 1 + off
        pad_seg, pad = p >> 32, (p >> 3) & 0x1FFFFFFF
        if not (p >> 2) & 1:
            return self.follow_pad(pad_seg, pad)
        far, tag = self.u64(pad_seg, pad), self.u64(pad_seg, pad + 1)
        if far & 3 != 2:
            raise ValueError("malformed double-far pointer")
        return far >> 32, tag, (far >> 3) & 0x1FFFFFFF

    def follow_pad(self, seg, w):
        r = self.follow(seg, w)
        if r is None or self.u64(seg, w) & 3 == 2:
            raise ValueError("malformed far pointer")
        return r


class _Rec:
    """One struct: `dw` data words followed by `pw` pointers."""

    def __init__(self, view, seg, w, dw, pw):
        self.v, self.seg, self.w, self.dw, self.pw = view, seg, w, dw, pw
        if w < 0 or w + dw + pw > view.words[seg]:
            raise ValueError("struct leaves its segment")

    def scalar(self, fmt, byte):
        size = _st.calcsize(fmt)
        if byte + size > 8 * self.dw:
            return 0
        return _st.unpack_from(fmt, self.v.data, self.v.start[self.seg] + 8 * self.w + byte)[0]

    def _target(self, i):
        return None if i >= self.pw else self.v.follow(self.seg, self.w + self.dw + i)

    def child(self, i):
        t = self._target(i)
        if t is None:
            return None
        seg, p, w = t
        if p & 3 != 0:
            raise ValueError("expected a struct pointer")
        return _Rec(self.v, seg, w, (p >> 32) & 0xFFFF, (p >> 48) & 0xFFFF)

    def array(self, i, dtype):
        t = self._target(i)
        if t is None:
            return np.zeros(0, dtype)
        seg, p, w = t
        size_code = {1: 2, 2: 3, 4: 4, 8: 5}[np.dtype(dtype).itemsize]
        if p & 3 != 1 or (p >> 32) & 7 != size_code:
            raise ValueError("expected a list of %s" % np.dtype(dtype).name)
        count = p >> 35
        if 8 * w + count * np.dtype(dtype).itemsize > 8 * self.v.words[seg] or w < 0:
            raise ValueError("list leaves its segment")
        return np.frombuffer(self.v.data, np.dtype(dtype).newbyteorder("<"), count, self.v.start[seg] + 8 * w).astype(dtype)

    def text(self, i):
        b = self.array(i, np.uint8)
        return bytes(b[:-1]).decode("utf-8") if len(b) else ""

    def records(self, i):
        t = self._target(i)
        if t is None:
            return []
        seg, p, w = t
        if p & 3 != 1 or (p >> 32) & 7 != 7:
            raise ValueError("expected a list of structs")
        tag = self.v.u64(seg, w)
        count, dw, pw = (tag >> 2) & 0x3FFFFFFF, (tag >> 32) & 0xFFFF, (tag >> 48) & 0xFFFF
        return [_Rec(self.v, seg, w + 1 + k * (dw + pw), dw, pw) for k in range(count)]


def decode_message(data):
    """Decode an xspn file (bytes) into plain Python data:
    {"query": None | {batch_size, error_kind, max_error, support_marginal}, "root_id", "num_features", "name",
     "feature_type", "scope": [...], "nodes": [{"id", "root", "kind", ...kind-specific fields...}]}.
    Field positions follow spflow.capnp:27-101 of the reference."""
    view = _View(data)
    t = view.follow(0, 0)
    if t is None or t[1] & 3 != 0:
        raise ValueError("xspn file has no header struct")
    header = _Rec(view, t[0], t[2], (t[1] >> 32) & 0xFFFF, (t[1] >> 48) & 0xFFFF)
    out = {"query": None}
    which = header.scalar("<H", 0)
    if which == 1:
        q = header.child(0)
        if q is None:
            raise ValueError("query header without a query")
        joint = q.child(0)
        if joint is None:
            raise ValueError("Can only deserialize joint queries")
        out["query"] = {"batch_size": q.scalar("<i", 0), "error_kind": q.scalar("<H", 4), "max_error": float(q.scalar("<d", 8)),
                        "support_marginal": bool(joint.scalar("<B", 0) & 1)}
        model = joint.child(0)
    elif which == 0:
        model = header.child(0)
    else:
        raise NotImplementedError("No deserialization defined for header content %d" % which)
    if model is None:
        raise ValueError("No model attached")
    out.update(root_id=model.scalar("<i", 0), num_features=model.scalar("<I", 4), name=model.text(0),
               feature_type=model.text(1), scope=[int(s) for s in model.array(2, np.int32)], nodes=[])
    for rec in model.records(3):
        kind = rec.scalar("<H", 6)
        node = {"id": rec.scalar("<i", 0), "root": bool(rec.scalar("<B", 4) & 1), "kind": kind}
        body = rec.child(0)
        if body is None:
            raise ValueError("node %d has no content" % node["id"])
        if kind == K_PRODUCT:
            node["children"] = [int(c) for c in body.array(0, np.int32)]
        elif kind == K_SUM:
            node["children"] = [int(c) for c in body.array(0, np.int32)]
            node["weights"] = [float(w) for w in body.array(1, np.float64)]
        elif kind == K_HIST:
            node.update(type=body.scalar("<H", 0), meta_type=body.scalar("<H", 2), scope=body.scalar("<i", 4),
                        breaks=[int(b) for b in body.array(0, np.int32)],
                        densities=[float(d) for d in body.array(1, np.float64)],
                        bin_repr_points=[float(r) for r in body.array(2, np.float64)])
        elif kind == K_GAUSS:
            node.update(mean=float(body.scalar("<d", 0)), stddev=float(body.scalar("<d", 8)), scope=body.scalar("<i", 16))
        elif kind == K_CAT:
            node.update(scope=body.scalar("<i", 0), probabilities=[float(p) for p in body.array(0, np.float64)])
        else:
            raise NotImplementedError("No deserialization defined for node kind %d" % kind)
        out["nodes"].append(node)
    return out
