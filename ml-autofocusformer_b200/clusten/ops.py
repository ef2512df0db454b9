"""Tensor-level calls into libclusten_b200: one function per C entry point.

Inputs must be contiguous CUDA tensors of one floating dtype plus an int64
index tensor; outputs are allocated here with torch.empty (the kernels write
every element) and the kernels run on torch's current stream.
"""
import collections
import os

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16,
           torch.float64: _lib.F64}


def _dt(t):
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"clusten: unsupported dtype {t.dtype}") from None


def _chk(name, t, dtype=None, dim=None):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise RuntimeError(f"{name} must have {dim} dimensions, got {t.dim()}")


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


# ----------------------------------------------------------------------------- inverse index
class _InverseCache:
    """Inverse indices of the most recently used nbhd_idx tensors.

    All blocks of a stage, and the QK and AV operators inside each block,
    receive the same nbhd_idx tensor (models/aff_transformer.py:480-495 of the
    reference), so one inverse serves many backward calls.  An entry keeps a
    reference to its index tensor, which pins the storage: a later tensor can
    only match an entry by being that very storage, unmodified.
    """

    def __init__(self, capacity):
        self.capacity = capacity
        self.entries = collections.OrderedDict()

    @staticmethod
    def _key(idx, n_targets):
        return (idx.data_ptr(), tuple(idx.shape), idx.device.index, n_targets)

    def get(self, idx, n_targets):
        key = self._key(idx, n_targets)
        ent = self.entries.get(key)
        if ent is not None and ent[1] == idx._version and ent[0]._version == idx._version:
            self.entries.move_to_end(key)
            return ent[2]
        return None

    def put(self, idx, n_targets, inv):
        key = self._key(idx, n_targets)
        self.entries[key] = (idx, idx._version, inv)
        self.entries.move_to_end(key)
        while len(self.entries) > self.capacity:
            self.entries.popitem(last=False)

    def clear(self):
        self.entries.clear()


_cache = _InverseCache(int(os.environ.get("CLUSTEN_INVERSE_CACHE", "4")))


_order_cache = _InverseCache(int(os.environ.get("CLUSTEN_INVERSE_CACHE", "4")))
_ORDER_MAX_ROWS = 4096     # clusten_wf_order_build sorts one batch element in shared memory


def clear_inverse_cache():
    """Drop every cached inverse index and row order (and the index tensors they pin)."""
    _cache.clear()
    _order_cache.clear()


def build_inverse(nbhd_idx, n_targets):
    """Inverse of nbhd_idx [b, rows, m] over n_targets tokens -> opaque int32 buffer."""
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, rows, m = nbhd_idx.shape
    lib = _lib.load()
    nbytes = lib.clusten_inverse_bytes(b, rows, m, n_targets)
    if nbytes == 0:
        _lib.check(lib.clusten_inverse_build(None, b, rows, m, n_targets, None, 0, None))
        raise RuntimeError("clusten: inverse index not available for these sizes")
    inv = torch.empty(nbytes // 4, dtype=torch.int32, device=nbhd_idx.device)
    with torch.cuda.device_of(nbhd_idx):
        _lib.check(lib.clusten_inverse_build(nbhd_idx.data_ptr(), b, rows, m, n_targets, inv.data_ptr(),
                                             nbytes, _stream(nbhd_idx)))
    return inv


def inverse_for(nbhd_idx, n_targets):
    """Cached build_inverse."""
    if _cache.capacity <= 0:
        return build_inverse(nbhd_idx, n_targets)
    inv = _cache.get(nbhd_idx, n_targets)
    if inv is None:
        inv = build_inverse(nbhd_idx, n_targets)
        _cache.put(nbhd_idx, n_targets, inv)
    return inv


def build_row_order(nbhd_idx):
    """Row order for the WF kernels: int32 [b, n_out] permutation that puts rows with nearby
    neighbourhoods next to each other; None when n_out is more than the sort handles."""
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, rows, m = nbhd_idx.shape
    if rows > _ORDER_MAX_ROWS:
        return None
    lib = _lib.load()
    nbytes = lib.clusten_wf_order_bytes(b, rows)
    order = torch.empty(nbytes // 4, dtype=torch.int32, device=nbhd_idx.device)
    with torch.cuda.device_of(nbhd_idx):
        _lib.check(lib.clusten_wf_order_build(nbhd_idx.data_ptr(), b, rows, m, order.data_ptr(), nbytes,
                                              _stream(nbhd_idx)))
    return order.view(b, rows)


def row_order_for(nbhd_idx):
    """Cached build_row_order."""
    if _order_cache.capacity <= 0 or nbhd_idx.shape[1] > _ORDER_MAX_ROWS:
        return build_row_order(nbhd_idx)
    order = _order_cache.get(nbhd_idx, "order")
    if order is None:
        order = build_row_order(nbhd_idx)
        _order_cache.put(nbhd_idx, "order", order)
    return order


def _order_ptr(row_order, nbhd_idx):
    """row_order argument -> (tensor kept alive, pointer): None = cached order, False = storage order."""
    if row_order is None:
        row_order = row_order_for(nbhd_idx)
    if row_order is None or row_order is False:
        return None, None
    if row_order.dtype != torch.int32 or row_order.numel() != nbhd_idx.shape[0] * nbhd_idx.shape[1] \
            or not row_order.is_contiguous() or row_order.device != nbhd_idx.device:
        raise RuntimeError("clusten: row_order must be a contiguous int32 [b, n_out] tensor on the inputs' device")
    return row_order, row_order.data_ptr()


# ----------------------------------------------------------------------------- neighbourhood search
def knn2d(query, database, k, return_dist=False):
    """Indices [b, n_query, k] (int64) of the k database points nearest to every query, ascending distance,
    ties towards the lower index; 2-D fp32 positions [b, n_query, 2] and [b, n, 2]."""
    _chk("query", query, torch.float32, 3)
    _chk("database", database, torch.float32, 3)
    b, nq, d = query.shape
    if d != 2 or database.shape[0] != b or database.shape[2] != 2:
        raise RuntimeError("clusten: knn2d needs [b, n, 2] positions")
    n = database.shape[1]
    nn_idx = torch.empty((b, nq, k), dtype=torch.int64, device=query.device)
    nn_dist = torch.empty((b, nq, k), dtype=torch.float32, device=query.device) if return_dist else None
    with torch.cuda.device_of(query):
        _lib.check(_lib.load().clusten_knn2d(query.data_ptr(), database.data_ptr(), b, nq, n, k, nn_idx.data_ptr(),
                                             nn_dist.data_ptr() if return_dist else None, _stream(query)))
    return (nn_idx, nn_dist) if return_dist else nn_idx


def nbhd_build(pos, member_idx, cluster_mask, nearest_cluster, rel_pos_width, table_width):
    """(nbhd_idx, nbhd_mask or None, pe_idx), each int64 [b, n, nnc * cs]: the members of every token's
    nearest clusters, their mask bits, and their offsets' rows in the position-embedding table
    (models/aff_transformer.py:476-487 of the reference in one kernel).  pos fp32 [b, n, 2];
    member_idx / cluster_mask int64 [b, k, cs]; nearest_cluster int64 [b, n, nnc]."""
    _chk("pos", pos, torch.float32, 3)
    _chk("member_idx", member_idx, torch.int64, 3)
    _chk("nearest_cluster", nearest_cluster, torch.int64, 3)
    b, n, d = pos.shape
    _, k, cs = member_idx.shape
    nnc = nearest_cluster.shape[2]
    if d != 2 or member_idx.shape[0] != b or nearest_cluster.shape[:2] != (b, n):
        raise RuntimeError("clusten: nbhd_build shape mismatch")
    if cluster_mask is not None:
        _chk("cluster_mask", cluster_mask, torch.int64, 3)
        if cluster_mask.shape != member_idx.shape:
            raise RuntimeError("clusten: cluster_mask must have member_idx's shape")
    m = nnc * cs
    nbhd_idx = torch.empty((b, n, m), dtype=torch.int64, device=pos.device)
    pe_idx = torch.empty((b, n, m), dtype=torch.int64, device=pos.device)
    nbhd_mask = torch.empty((b, n, m), dtype=torch.int64, device=pos.device) if cluster_mask is not None else None
    with torch.cuda.device_of(pos):
        _lib.check(_lib.load().clusten_nbhd_build(
            pos.data_ptr(), member_idx.data_ptr(), cluster_mask.data_ptr() if cluster_mask is not None else None,
            nearest_cluster.data_ptr(), nbhd_idx.data_ptr(), nbhd_mask.data_ptr() if nbhd_mask is not None else None,
            pe_idx.data_ptr(), b, n, k, cs, nnc, int(rel_pos_width), int(table_width), _stream(pos)))
    return nbhd_idx, nbhd_mask, pe_idx


def merge_weights(weights_table, pe_idx, learned_prob=None, nbhd_idx=None, nbhd_mask=None):
    """weights [b, n_out, m, ic] = weights_table[pe_idx] * (learned_prob[b, nbhd_idx] * nbhd_mask): the first
    argument of CLUSTENWF as ClusterMerging builds it (models/aff_transformer.py:340-358 of the reference), in one
    kernel.  weights_table [rows, ic]; learned_prob [b, n] or [b, n, 1] (None = 1); int64 [b, n_out, m] tables.
    Table and scores are brought to their common dtype first, as the reference's product does."""
    _chk("pe_idx", pe_idx, torch.int64, 3)
    b, n_out, m = pe_idx.shape
    dtype = weights_table.dtype
    n = 1
    if learned_prob is not None:
        dtype = torch.promote_types(dtype, learned_prob.dtype)
        learned_prob = learned_prob.reshape(b, -1).to(dtype).contiguous()
        n = learned_prob.shape[1]
        if nbhd_idx is None:
            raise RuntimeError("clusten: merge_weights needs nbhd_idx with learned_prob")
        _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
        if nbhd_idx.shape != pe_idx.shape:
            raise RuntimeError("clusten: nbhd_idx must have pe_idx's shape")
    weights_table = weights_table.to(dtype).contiguous()
    _chk("weights_table", weights_table, None, 2)
    rows, ic = weights_table.shape
    if nbhd_mask is not None:
        _chk("nbhd_mask", nbhd_mask, torch.int64, 3)
        if nbhd_mask.shape != pe_idx.shape:
            raise RuntimeError("clusten: nbhd_mask must have pe_idx's shape")
    out = torch.empty((b, n_out, m, ic), dtype=dtype, device=pe_idx.device)
    with torch.cuda.device_of(pe_idx):
        _lib.check(_lib.load().clusten_merge_weights(
            weights_table.data_ptr(), pe_idx.data_ptr(), learned_prob.data_ptr() if learned_prob is not None else None,
            nbhd_idx.data_ptr() if learned_prob is not None else None,
            nbhd_mask.data_ptr() if nbhd_mask is not None else None, out.data_ptr(), b, n_out, n, m, ic, rows,
            _dt(out), _stream(pe_idx)))
    return out


# ----------------------------------------------------------------------------- QK
def qk_forward(query, key, nbhd_idx):
    """attn[b,h,i,j] = <query[b,h,i], key[b,h,nbhd_idx[b,i,j]]>"""
    _chk("query", query, dim=4)
    _chk("key", key, query.dtype, 4)
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, h, n, c = query.shape
    m = nbhd_idx.shape[2]
    if key.shape != query.shape or nbhd_idx.shape[:2] != (b, n):
        raise RuntimeError("clusten: QK shape mismatch")
    attn = torch.empty((b, h, n, m), dtype=query.dtype, device=query.device)
    with torch.cuda.device_of(query):
        _lib.check(_lib.load().clusten_qk_forward(query.data_ptr(), key.data_ptr(), nbhd_idx.data_ptr(),
                                                  attn.data_ptr(), b, h, n, m, c, _dt(query), _stream(query)))
    return attn


def _row_view(t):
    """Can the kernels read this [b, h, n, 32] tensor in place?  Rows contiguous, every other stride and the
    base address a multiple of 16 bytes."""
    es = t.element_size()
    return (t.is_cuda and t.dim() == 4 and t.shape[3] == 32 and t.stride(3) == 1 and t.data_ptr() % 16 == 0
            and all(s > 0 and (s * es) % 16 == 0 for s in t.stride()[:3]))


def _strides3(t):
    import ctypes
    return (ctypes.c_longlong * 3)(*t.stride()[:3])


def strided_forward_ok(a, b_, nbhd_idx):
    """QK: both operands; AV: the value operand (attn must be contiguous) -- see qk/av_forward_views."""
    return (a.dtype == b_.dtype and a.dtype in (torch.float32, torch.float16, torch.bfloat16)
            and 1 <= nbhd_idx.shape[2] <= 48 and nbhd_idx.is_contiguous())


def qk_forward_views(query, key, nbhd_idx):
    """qk_forward on views of query and key (permuted Linear outputs): no copies.  None when the views do not
    qualify (the caller then makes them contiguous)."""
    if not (_row_view(query) and _row_view(key) and strided_forward_ok(query, key, nbhd_idx)):
        return None
    b, h, n, c = query.shape
    m = nbhd_idx.shape[2]
    if key.shape != query.shape or nbhd_idx.shape[:2] != (b, n) or nbhd_idx.dtype != torch.int64:
        raise RuntimeError("clusten: QK shape mismatch")
    attn = torch.empty((b, h, n, m), dtype=query.dtype, device=query.device)
    with torch.cuda.device_of(query):
        st = _lib.load().clusten_qk_forward_strided(query.data_ptr(), _strides3(query), key.data_ptr(), _strides3(key),
                                                    nbhd_idx.data_ptr(), attn.data_ptr(), b, h, n, m, c, _dt(query),
                                                    _stream(query))
    if st == -6:
        return None
    _lib.check(st)
    return attn


def av_forward_views(attn, value, nbhd_idx):
    """av_forward with value read in place through a view; attn must be contiguous.  None when not possible."""
    if not (attn.is_contiguous() and _row_view(value) and strided_forward_ok(attn, value, nbhd_idx)):
        return None
    b, h, n, m = attn.shape
    c = value.shape[3]
    if value.shape[:3] != (b, h, n) or nbhd_idx.shape != (b, n, m) or nbhd_idx.dtype != torch.int64:
        raise RuntimeError("clusten: AV shape mismatch")
    feat = torch.empty((b, h, n, c), dtype=attn.dtype, device=attn.device)
    with torch.cuda.device_of(attn):
        st = _lib.load().clusten_av_forward_strided(attn.data_ptr(), value.data_ptr(), _strides3(value),
                                                    nbhd_idx.data_ptr(), feat.data_ptr(), b, h, n, m, c, _dt(attn),
                                                    _stream(attn))
    if st == -6:
        return None
    _lib.check(st)
    return feat


def local_attention_forward(query, key, value, nbhd_idx, pos_bias=None, pe_table=None, pe_idx=None, mask=None,
                            blank_k=None, blank_v=None):
    """Fused forward of the local attention chain (scores + position bias + mask + blank token + softmax +
    output); see clusten_local_attention_forward in the header.  query must already be scaled.  query / key /
    value may be views with contiguous rows (key and value with equal strides).  Inference only: no autograd."""
    for name, t in (("query", query), ("key", key), ("value", value)):
        if not t.is_cuda or t.dim() != 4 or t.dtype != query.dtype:
            raise RuntimeError(f"clusten: {name} must be a 4-d CUDA tensor of query's dtype")
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, h, n, c = query.shape
    m = nbhd_idx.shape[2]
    if key.shape != query.shape or value.shape != query.shape or nbhd_idx.shape[:2] != (b, n):
        raise RuntimeError("clusten: local attention shape mismatch")
    if not _row_view(query):
        query = query.contiguous()
    if not (_row_view(key) and _row_view(value) and key.stride() == value.stride()):
        key, value = key.contiguous(), value.contiguous()
    def opt(name, t, dtype, shape):
        if t is None:
            return None
        _chk(name, t, dtype)
        if tuple(t.shape) != shape:
            raise RuntimeError(f"clusten: {name} must have shape {shape}, got {tuple(t.shape)}")
        return t
    pos_bias = opt("pos_bias", pos_bias, query.dtype, (b, h, n, m))
    pe_idx = opt("pe_idx", pe_idx, torch.int64, (b, n, m))
    mask = opt("mask", mask, torch.int64, (b, n, m))
    blank_k = opt("blank_k", blank_k, query.dtype, (h, c))
    blank_v = opt("blank_v", blank_v, query.dtype, (h, c))
    rows = 0
    if pe_table is not None:
        _chk("pe_table", pe_table, query.dtype, 2)
        if pe_table.shape[1] != h or pe_idx is None:
            raise RuntimeError("clusten: pe_table must be [rows, heads] and come with pe_idx")
        rows = pe_table.shape[0]
    out = torch.empty((b, h, n, c), dtype=query.dtype, device=query.device)
    ptr = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device_of(query):
        _lib.check(_lib.load().clusten_local_attention_forward(
            query.data_ptr(), _strides3(query), key.data_ptr(), value.data_ptr(), _strides3(key), nbhd_idx.data_ptr(),
            ptr(pos_bias), ptr(pe_table), ptr(pe_idx), rows, ptr(mask), ptr(blank_k), ptr(blank_v), out.data_ptr(),
            b, h, n, m, c, _dt(query), _stream(query)))
    return out


def qk_backward(d_attn, query, key, nbhd_idx, inverse=None):
    _chk("d_attn", d_attn, query.dtype, 4)
    _chk("query", query, dim=4)
    _chk("key", key, query.dtype, 4)
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, h, n, c = query.shape
    m = nbhd_idx.shape[2]
    if d_attn.shape != (b, h, n, m) or key.shape != query.shape:
        raise RuntimeError("clusten: QK backward shape mismatch")
    if inverse is None:
        inverse = inverse_for(nbhd_idx, n)
    d_query = torch.empty_like(query)
    d_key = torch.empty_like(key)
    with torch.cuda.device_of(query):
        _lib.check(_lib.load().clusten_qk_backward(
            d_attn.data_ptr(), query.data_ptr(), key.data_ptr(), nbhd_idx.data_ptr(), inverse.data_ptr(),
            d_query.data_ptr(), d_key.data_ptr(), b, h, n, m, c, _dt(query), _stream(query)))
    return d_query, d_key


# ----------------------------------------------------------------------------- AV
def av_forward(attn, value, nbhd_idx):
    """feat[b,h,i,:] = sum_j attn[b,h,i,j] * value[b,h,nbhd_idx[b,i,j],:]"""
    _chk("attn", attn, dim=4)
    _chk("v", value, attn.dtype, 4)
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, h, n, m = attn.shape
    c = value.shape[3]
    if value.shape[:3] != (b, h, n) or nbhd_idx.shape != (b, n, m):
        raise RuntimeError("clusten: AV shape mismatch")
    feat = torch.empty((b, h, n, c), dtype=attn.dtype, device=attn.device)
    with torch.cuda.device_of(attn):
        _lib.check(_lib.load().clusten_av_forward(attn.data_ptr(), value.data_ptr(), nbhd_idx.data_ptr(),
                                                  feat.data_ptr(), b, h, n, m, c, _dt(attn), _stream(attn)))
    return feat


def av_backward(d_feat, attn, value, nbhd_idx, inverse=None):
    _chk("d_feat", d_feat, attn.dtype, 4)
    _chk("attn", attn, dim=4)
    _chk("v", value, attn.dtype, 4)
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, h, n, m = attn.shape
    c = value.shape[3]
    if d_feat.shape != value.shape or nbhd_idx.shape != (b, n, m):
        raise RuntimeError("clusten: AV backward shape mismatch")
    if inverse is None:
        inverse = inverse_for(nbhd_idx, n)
    d_attn = torch.empty_like(attn)
    d_value = torch.empty_like(value)
    with torch.cuda.device_of(attn):
        _lib.check(_lib.load().clusten_av_backward(
            d_feat.data_ptr(), attn.data_ptr(), value.data_ptr(), nbhd_idx.data_ptr(), inverse.data_ptr(),
            d_attn.data_ptr(), d_value.data_ptr(), b, h, n, m, c, _dt(attn), _stream(attn)))
    return d_attn, d_value


# ----------------------------------------------------------------------------- WF
def wf_forward(weights, feat, nbhd_idx, row_order=None):
    """feat_new[b,i,ic,:] = sum_j weights[b,i,j,ic] * feat[b,nbhd_idx[b,i,j],:]

    row_order: None = the cached order of nbhd_idx, False = storage order, or a build_row_order tensor."""
    _chk("weights", weights, dim=4)
    _chk("feat", feat, weights.dtype, 3)
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, n_out, m, ic = weights.shape
    n, c = feat.shape[1], feat.shape[2]
    if feat.shape[0] != b or nbhd_idx.shape != (b, n_out, m):
        raise RuntimeError("clusten: WF shape mismatch")
    feat_new = torch.empty((b, n_out, ic, c), dtype=weights.dtype, device=weights.device)
    order, order_ptr = _order_ptr(row_order, nbhd_idx)
    with torch.cuda.device_of(weights):
        _lib.check(_lib.load().clusten_wf_forward(
            weights.data_ptr(), feat.data_ptr(), nbhd_idx.data_ptr(), order_ptr, feat_new.data_ptr(),
            b, n_out, n, m, ic, c, _dt(weights), _stream(weights)))
    return feat_new


def wf_backward(d_feat_new, weights, feat, nbhd_idx, inverse=None, row_order=None):
    _chk("d_feat_new", d_feat_new, weights.dtype, 4)
    _chk("weights", weights, dim=4)
    _chk("feat", feat, weights.dtype, 3)
    _chk("nbhd_idx", nbhd_idx, torch.int64, 3)
    b, n_out, m, ic = weights.shape
    n, c = feat.shape[1], feat.shape[2]
    if d_feat_new.shape != (b, n_out, ic, c) or nbhd_idx.shape != (b, n_out, m):
        raise RuntimeError("clusten: WF backward shape mismatch")
    if inverse is None:
        inverse = inverse_for(nbhd_idx, n)
    d_weights = torch.empty_like(weights)
    d_feat = torch.empty_like(feat)
    order, order_ptr = _order_ptr(row_order, nbhd_idx)
    with torch.cuda.device_of(weights):
        _lib.check(_lib.load().clusten_wf_backward(
            d_feat_new.data_ptr(), weights.data_ptr(), feat.data_ptr(), nbhd_idx.data_ptr(),
            inverse.data_ptr(), order_ptr, d_weights.data_ptr(), d_feat.data_ptr(),
            b, n_out, n, m, ic, c, _dt(weights), _stream(weights)))
    return d_weights, d_feat
