"""Drop-in for the reference's `clustenwf_cuda` extension module (clusten/src/clustenwf_cuda.cpp:48-51):
`forward(weights, feat, nbhd_idx)` and `backward(d_feat_new, weights, feat, nbhd_idx)` on libclusten_b200."""
from clusten import ops


def forward(weights, feat, nbhd_idx):
    return ops.wf_forward(weights, feat, nbhd_idx)


def backward(d_feat_new, weights, feat, nbhd_idx):
    d_weights, d_feat = ops.wf_backward(d_feat_new, weights, feat, nbhd_idx)
    return [d_weights, d_feat]
