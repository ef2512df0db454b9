"""Seeded synthetic inputs for the CLUSTEN operators.

Neighbourhood tables (`nbhd_idx`) in the three regimes the kernels must handle:

  shared_cluster_rows   random 2-D positions, tokens numbered along a Hilbert curve,
                        grouped 8 at a time; every member of a cluster gets the same
                        row: the m tokens nearest the cluster centroid.
  model_like_rows       what AutoFocusFormer builds (models/aff_transformer.py:476-482,
                        models/point_utils.py:189-206 of the reference): each token takes
                        its m/8 nearest clusters and its row is the concatenation of those
                        clusters' member runs [8j .. 8j+7]; slots past the last token point
                        at token 0.
  random_rows           uniform random indices with repeats, as in the reference's kernel
                        tests (clusten/test_qk_kernel.py:25).

and the operand tensors with the distributions of the benchmark configurations:
N(0,1) features and gradients, softmax-normalised attention and merge weights.
Everything is generated with torch on the device asked for, from an explicit seed.
"""
import math

import torch

CLUSTER = 8


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def hilbert_key(x, y, order):
    """Index along a Hilbert curve of side 2**order for integer coordinates (tensors)."""
    x = x.clone().long()
    y = y.clone().long()
    d = torch.zeros_like(x)
    s = 1 << (order - 1)
    while s > 0:
        rx = ((x & s) > 0).long()
        ry = ((y & s) > 0).long()
        d += s * s * ((3 * rx) ^ ry)
        # rotate the quadrant
        flip = (ry == 0) & (rx == 1)
        x = torch.where(flip, s - 1 - x, x)
        y = torch.where(flip, s - 1 - y, y)
        swap = ry == 0
        x, y = torch.where(swap, y, x), torch.where(swap, x, y)
        x &= s - 1
        y &= s - 1
        s >>= 1
    return d


def sorted_positions(b, n, seed, device="cpu"):
    """[b, n, 2] uniform positions in [0, sqrt(n))^2, ordered along a Hilbert curve."""
    side = math.sqrt(n)
    pos = torch.rand(b, n, 2, generator=_gen(seed, device), device=device) * side
    order = 10
    q = (pos / side * (1 << order)).long().clamp_(0, (1 << order) - 1)
    key = hilbert_key(q[..., 0], q[..., 1], order)
    perm = torch.argsort(key, dim=1, stable=True)
    return pos.gather(1, perm.unsqueeze(-1).expand(-1, -1, 2))


def _centroids(pos):
    b, n, _ = pos.shape
    k = (n + CLUSTER - 1) // CLUSTER
    pad = k * CLUSTER - n
    p = torch.cat([pos, pos.new_zeros(b, pad, 2)], 1).view(b, k, CLUSTER, 2)
    cnt = torch.full((k,), float(CLUSTER), device=pos.device)
    if pad:
        cnt[-1] = CLUSTER - pad
    return p.sum(2) / cnt.view(1, k, 1)


def shared_cluster_rows(b, n, m, seed, device="cpu", batch_chunk=16):
    """nbhd_idx [b, n, m] int64; the 8 tokens of a cluster share one row."""
    pos = sorted_positions(b, n, seed, device)
    rows = []
    for s in range(0, b, batch_chunk):
        p = pos[s:s + batch_chunk]
        d = torch.cdist(_centroids(p), p)                       # [bc, k, n]
        nn = d.topk(min(m, n), dim=2, largest=False, sorted=True)[1]
        if m > n:
            nn = torch.cat([nn, nn[..., :1].expand(-1, -1, m - n)], 2)
        rows.append(nn.repeat_interleave(CLUSTER, dim=1)[:, :n])
    return torch.cat(rows, 0).contiguous()


def model_like_rows(b, n, m, seed, device="cpu", batch_chunk=16):
    """nbhd_idx [b, n, m] int64 made of m/8 aligned runs of 8 token ids per token."""
    if m % CLUSTER:
        raise ValueError("model_like_rows needs m to be a multiple of 8")
    nnc = m // CLUSTER
    pos = sorted_positions(b, n, seed, device)
    k = (n + CLUSTER - 1) // CLUSTER
    member = torch.arange(k * CLUSTER, device=device).view(k, CLUSTER)
    member = torch.where(member < n, member, torch.zeros_like(member))   # pads point at token 0
    rows = []
    for s in range(0, b, batch_chunk):
        p = pos[s:s + batch_chunk]
        d = torch.cdist(p, _centroids(p))                       # [bc, n, k]
        near = d.topk(min(nnc, k), dim=2, largest=False, sorted=True)[1]
        if nnc > k:
            near = torch.cat([near, near[..., :1].expand(-1, -1, nnc - k)], 2)
        rows.append(member[near].reshape(p.shape[0], n, m))
    return torch.cat(rows, 0).contiguous()


def random_rows(b, n_rows, n, m, seed, device="cpu"):
    """nbhd_idx [b, n_rows, m] int64, uniform in [0, n) with repeats."""
    return torch.randint(n, (b, n_rows, m), generator=_gen(seed, device), device=device)


def select_rows(nbhd_idx, n_out, seed):
    """Rows of `n_out` distinct tokens per batch element, in no particular order: the
    merge centres of the adaptive downsampling (models/aff_transformer.py:320-336 picks
    them with an unsorted top-k)."""
    b, n, m = nbhd_idx.shape
    device = nbhd_idx.device
    score = torch.rand(b, n, generator=_gen(seed, device), device=device)
    pick = score.topk(n_out, dim=1, sorted=False)[1]
    return nbhd_idx.gather(1, pick.unsqueeze(-1).expand(-1, -1, m)).contiguous()


def make_index(regime, b, n, m, seed, device="cpu"):
    if regime == "shared":
        return shared_cluster_rows(b, n, m, seed, device)
    if regime == "model":
        return model_like_rows(b, n, m, seed, device)
    if regime == "random":
        return random_rows(b, n, n, m, seed, device)
    raise ValueError(regime)


def attention_operands(b, h, n, m, c, dtype, seed, device="cpu"):
    """(query, key, value, attn, grad_attn, grad_feat): N(0,1) except attn = softmax(N(0,1))."""
    g = _gen(seed, device)

    def rn(*shape):
        return torch.randn(*shape, generator=g, device=device).to(dtype)

    q, k, v = rn(b, h, n, c), rn(b, h, n, c), rn(b, h, n, c)
    attn = torch.softmax(torch.randn(b, h, n, m, generator=g, device=device), -1).to(dtype)
    return q, k, v, attn, rn(b, h, n, m), rn(b, h, n, c)


def merge_operands(b, n_out, n, m, ic, c, dtype, seed, device="cpu"):
    """(weights, feat, grad_feat_new): weights softmax-normalised over the m neighbours."""
    g = _gen(seed, device)
    w = torch.softmax(torch.randn(b, n_out, m, ic, generator=g, device=device), 2).to(dtype)
    feat = torch.randn(b, n, c, generator=g, device=device).to(dtype)
    grad = torch.randn(b, n_out, ic, c, generator=g, device=device).to(dtype)
    return w, feat, grad


# --------------------------------------------------------------------------- bytes
def algorithmic_bytes(op, direction, *, b, n, m, c, s, h=1, n_out=0, ic=1):
    """Bytes an ideal implementation moves: every input read once, every output written once,
    int64 indices, nothing for workspaces.  s = element size."""
    if op in ("qk", "av"):
        bhnc, bhnm, bnm8 = b * h * n * c * s, b * h * n * m * s, b * n * m * 8
        if direction == "fwd":
            return 2 * bhnc + bnm8 + bhnm
        if op == "qk":
            return bhnm + 4 * bhnc + bnm8
        return 2 * bhnm + 3 * bhnc + bnm8
    if op == "wf":
        w, f, i8, o = b * n_out * m * ic * s, b * n * c * s, b * n_out * m * 8, b * n_out * ic * c * s
        if direction == "fwd":
            return w + f + i8 + o
        return o + 2 * w + 2 * f + i8
    raise ValueError(op)
