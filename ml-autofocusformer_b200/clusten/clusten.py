"""The three CLUSTEN autograd operators, on libclusten_b200.

Same names, argument order, output layouts and gradient contract as
clusten/clusten.py of apple/ml-autofocusformer (`CLUSTENQKFunction` :17-40,
`CLUSTENAVFunction` :43-66, `CLUSTENWFFunction` :69-92), so that
models/aff_transformer.py (:11, :120, :154, :361) imports this package
unchanged.  As there, the second tensor is converted to the first tensor's
dtype and the index receives no gradient.  Differences: bf16 is accepted, key
is not transposed, the scatter-side gradients are deterministic, and the
forward passes read query / key / value in place when they arrive as views with
contiguous rows (the reference copies them, clusten/clusten.py:23-24,50); the
backward passes copy such views, as the reference does.
"""
from torch.autograd import Function

from . import _lib, ops

_lib.load()  # fail at import, like the reference (clusten/clusten.py:8-14), when the library is missing


def _normalise(first, second, nbhd_idx):
    first = first.contiguous()
    second = second.contiguous()
    if second.dtype != first.dtype:
        second = second.to(first.dtype)
    return first, second, nbhd_idx.contiguous()


class CLUSTENQKFunction(Function):
    """attn = query x gathered neighbour keys:  [b,h,n,c], [b,h,n,c], [b,n,m] -> [b,h,n,m]"""

    @staticmethod
    def forward(ctx, query, key, nbhd_idx):
        nbhd_idx = nbhd_idx.contiguous()
        if key.dtype == query.dtype:
            # the model's query / key are permuted views of Linear outputs: read them where they are
            attn = ops.qk_forward_views(query, key, nbhd_idx)
            if attn is not None:
                ctx.save_for_backward(query, key, nbhd_idx)
                return attn
        query, key, nbhd_idx = _normalise(query, key, nbhd_idx)
        ctx.save_for_backward(query, key, nbhd_idx)
        return ops.qk_forward(query, key, nbhd_idx)

    @staticmethod
    def backward(ctx, grad_attn):
        query, key, nbhd_idx = ctx.saved_tensors
        query, key = query.contiguous(), key.contiguous()
        d_query, d_key = ops.qk_backward(grad_attn.contiguous().to(query.dtype), query, key, nbhd_idx)
        return d_query, d_key, None


class CLUSTENAVFunction(Function):
    """feat = attn x gathered neighbour values:  [b,h,n,m], [b,h,n,c], [b,n,m] -> [b,h,n,c]"""

    @staticmethod
    def forward(ctx, attn, v, nbhd_idx):
        nbhd_idx = nbhd_idx.contiguous()
        attn = attn.contiguous()          # the [..., :-1] slice of the softmax output: rows of m + 1, copied
        if v.dtype == attn.dtype:
            feat = ops.av_forward_views(attn, v, nbhd_idx)     # v: a view of the kv Linear output, read in place
            if feat is not None:
                ctx.save_for_backward(attn, v, nbhd_idx)
                return feat
        attn, v, nbhd_idx = _normalise(attn, v, nbhd_idx)
        ctx.save_for_backward(attn, v, nbhd_idx)
        return ops.av_forward(attn, v, nbhd_idx)

    @staticmethod
    def backward(ctx, grad_feat):
        attn, v, nbhd_idx = ctx.saved_tensors
        d_attn, d_v = ops.av_backward(grad_feat.contiguous().to(attn.dtype), attn, v.contiguous(), nbhd_idx)
        return d_attn, d_v, None


class CLUSTENWFFunction(Function):
    """feat_new = weights^T x gathered neighbour features:
    [b,n_,m,ic], [b,n,c], [b,n_,m] -> [b,n_,ic,c]"""

    @staticmethod
    def forward(ctx, weights, feat, nbhd_idx):
        weights, feat, nbhd_idx = _normalise(weights, feat, nbhd_idx)
        ctx.save_for_backward(weights, feat, nbhd_idx)
        return ops.wf_forward(weights, feat, nbhd_idx)

    @staticmethod
    def backward(ctx, grad_feat_new):
        weights, feat, nbhd_idx = ctx.saved_tensors
        d_weights, d_feat = ops.wf_backward(grad_feat_new.contiguous().to(weights.dtype), weights, feat,
                                            nbhd_idx)
        return d_weights, d_feat, None
