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
