"""Drop-in for the reference's `clustenav_cuda` extension module (clusten/src/clustenav_cuda.cpp:48-51):
`forward(attn, v, nbhd_idx)` and `backward(d_feat, attn, v, nbhd_idx)` on libclusten_b200."""
from clusten import ops


def forward(attn, v, nbhd_idx):
    return ops.av_forward(attn, v, nbhd_idx)


def backward(d_feat, attn, v, nbhd_idx):
    d_attn, d_v = ops.av_backward(d_feat, attn, v, nbhd_idx)
    return [d_attn, d_v]
