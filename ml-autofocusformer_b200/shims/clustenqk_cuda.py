"""Drop-in for the reference's `clustenqk_cuda` extension module (clusten/src/clustenqk_cuda.cpp:48-51):
`forward(query, key_t, nbhd_idx)` and `backward(d_attn, query, key, nbhd_idx)` on libclusten_b200.

With this directory on sys.path the reference's own clusten/clusten.py (which does `import clustenqk_cuda`,
clusten/clusten.py:8-11) runs unchanged on the B200 kernels.  As there, forward receives the key
pre-transposed to [b, h, c, n] (clusten/clusten.py:30) and backward the key as [b, h, n, c] (:37-38).
"""
from clusten import ops


def forward(query, key_t, nbhd_idx):
    # the B200 kernel reads key rows, so the reference wrapper's transpose is undone here
    return ops.qk_forward(query, key_t.permute(0, 1, 3, 2).contiguous(), nbhd_idx)


def backward(d_attn, query, key, nbhd_idx):
    d_query, d_key = ops.qk_backward(d_attn, query, key, nbhd_idx)
    return [d_query, d_key]
