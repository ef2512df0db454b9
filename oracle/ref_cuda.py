"""Loader for the reference's own CUDA extension (oracle/_ref/, built by build_ref.py).

TEST INFRASTRUCTURE ONLY.  The wrappers call the extension the way
clusten/clusten.py of the reference does (contiguous inputs; QK forward receives
the key transposed to [b,h,c,n], clusten/clusten.py:28-31), so their results are
the reference operators' results.  fp64 / fp32 / fp16 only: the reference has no
bf16 dispatch (clusten/src/clustenqk_cuda_kernel.cu:78).
"""
import importlib
import os
import sys

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_mods = {}


def available():
    try:
        _load("clustenqk_cuda")
        return True
    except Exception:
        return False


def _load(name):
    if name not in _mods:
        import torch  # noqa: F401  (the extension links against libtorch)
        if _DIR not in sys.path:
            sys.path.insert(0, _DIR)
        _mods[name] = importlib.import_module(name)
    return _mods[name]


def qk_forward(q, k, idx):
    return _load("clustenqk_cuda").forward(q.contiguous(), k.permute(0, 1, 3, 2).contiguous(), idx.contiguous())


def qk_backward(d_attn, q, k, idx):
    return _load("clustenqk_cuda").backward(d_attn.contiguous(), q.contiguous(), k.contiguous(), idx.contiguous())


def av_forward(attn, v, idx):
    return _load("clustenav_cuda").forward(attn.contiguous(), v.contiguous(), idx.contiguous())


def av_backward(d_feat, attn, v, idx):
    return _load("clustenav_cuda").backward(d_feat.contiguous(), attn.contiguous(), v.contiguous(), idx.contiguous())


def wf_forward(w, feat, idx):
    return _load("clustenwf_cuda").forward(w.contiguous(), feat.contiguous(), idx.contiguous())


def wf_backward(d_out, w, feat, idx):
    return _load("clustenwf_cuda").backward(d_out.contiguous(), w.contiguous(), feat.contiguous(), idx.contiguous())
