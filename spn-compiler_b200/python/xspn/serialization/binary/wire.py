"""Cap'n Proto encoder for xspn files, written against the reference's schema
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
