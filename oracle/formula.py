"""The pure-PyTorch gather formulation of the three CLUSTEN operators.

TEST INFRASTRUCTURE ONLY.  These are the expressions the reference's own kernel
tests print their error norms against:
  QK  clusten/test_qk_kernel.py:39-40   gather keys, broadcast-multiply with the query, sum over c
  AV  clusten/test_av_kernel.py:39-40   gather values, multiply by attn, sum over the m neighbours
  WF  clusten/test_wf_kernel.py:40-41   gather features, weights^T @ gathered
Gradients come from autograd.  Works on any device and dtype; `chunk` bounds the
size of the gathered [.., m, c] intermediate by looping over the batch.
"""
import torch


def _gather_rows(x, nbhd_idx):
    """x [b,h,n,c], nbhd_idx [b,n,m] -> [b,h,n,m,c]"""
    b, h, n, c = x.shape
    m = nbhd_idx.shape[2]
    index = nbhd_idx.reshape(b, 1, n * m, 1).expand(-1, h, -1, c)
    return x.gather(index=index, dim=2).reshape(b, h, n, m, c)


def qk(query, key, nbhd_idx):
    return (query.unsqueeze(3) * _gather_rows(key, nbhd_idx)).sum(-1)


def av(attn, value, nbhd_idx):
    return (attn.unsqueeze(4) * _gather_rows(value, nbhd_idx)).sum(3)


def wf(weights, feat, nbhd_idx):
    b, n_out, m, _ = weights.shape
    c = feat.shape[2]
    gathered = feat.gather(index=nbhd_idx.reshape(b, n_out * m, 1).expand(-1, -1, c), dim=1)
    return weights.transpose(-1, -2) @ gathered.reshape(b, n_out, m, c)


_OPS = {"qk": qk, "av": av, "wf": wf}


def forward(op, a, b_, nbhd_idx, chunk=None):
    """out = op(a, b_, nbhd_idx), optionally evaluated `chunk` batch elements at a time."""
    fn = _OPS[op]
    if chunk is None or chunk >= a.shape[0]:
        return fn(a, b_, nbhd_idx)
    outs = [fn(a[s:s + chunk], b_[s:s + chunk], nbhd_idx[s:s + chunk]) for s in range(0, a.shape[0], chunk)]
    return torch.cat(outs, 0)


def forward_backward(op, a, b_, nbhd_idx, grad_out, chunk=None):
    """(out, grad_a, grad_b) with autograd, optionally chunked over the batch."""
    fn = _OPS[op]
    step = a.shape[0] if chunk is None else chunk
    outs, ga, gb = [], [], []
    for s in range(0, a.shape[0], step):
        x = a[s:s + step].detach().clone().requires_grad_(True)
        y = b_[s:s + step].detach().clone().requires_grad_(True)
        o = fn(x, y, nbhd_idx[s:s + step])
        o.backward(grad_out[s:s + step])
        outs.append(o.detach())
        ga.append(x.grad)
        gb.append(y.grad)
    return torch.cat(outs, 0), torch.cat(ga, 0), torch.cat(gb, 0)


def nbhd_tables(pos, member_idx, cluster_mask, nearest_cluster, rel_pos_width, table_width):
    """(nbhd_idx, nbhd_mask or None, pe_idx): the neighbourhood tables of a stage as the reference's
    BasicLayer.forward builds them (models/aff_transformer.py:476-487): members of the nearest clusters,
    their mask bits, and the rows of their offsets in the position-embedding table."""
    b, n, d = pos.shape
    cs = member_idx.shape[2]
    nnc = nearest_cluster.shape[2]
    m = nnc * cs
    pick = nearest_cluster.reshape(b, -1, 1).expand(-1, -1, cs)
    nbhd_idx = member_idx.gather(index=pick, dim=1).reshape(b, n, m)
    nbhd_mask = None if cluster_mask is None else cluster_mask.gather(index=pick, dim=1).reshape(b, n, m)
    there = pos.gather(index=nbhd_idx.reshape(b, -1, 1).expand(-1, -1, d), dim=1).reshape(b, n, m, d)
    rel = there - (pos.unsqueeze(2) - rel_pos_width)
    pe_idx = (rel[..., 1] * table_width + rel[..., 0]).long()
    return nbhd_idx, nbhd_mask, pe_idx


def merge_weights(weights_table, pe_idx, learned_prob, nbhd_idx, nbhd_mask):
    """weights [b, n_out, m, ic] as the reference's ClusterMerging.forward builds them before CLUSTENWF
    (models/aff_transformer.py:340-358): table rows by pe_idx, times the neighbours' importance scores, times
    the mask.  learned_prob [b, n, 1] or None, nbhd_mask int64 [b, n_out, m] or None."""
    b, n_out, m = pe_idx.shape
    ic = weights_table.shape[-1]
    weights = weights_table.gather(index=pe_idx.reshape(-1, 1).expand(-1, ic), dim=0).reshape(b, n_out, m, ic)
    if learned_prob is not None:
        lp = learned_prob.gather(index=nbhd_idx.reshape(b, -1, 1), dim=1).reshape(b, n_out, m, 1)
        if nbhd_mask is not None:
            lp = lp * nbhd_mask.unsqueeze(3)
        weights = weights * lp
    elif nbhd_mask is not None:
        weights = weights * nbhd_mask.unsqueeze(3)
    return weights
