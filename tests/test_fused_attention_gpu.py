"""Fused local attention (clusten_local_attention_forward) against the chain it replaces, evaluated in fp64 with
the PyTorch gather formulation on the dtype-rounded inputs (models/aff_transformer.py:120-155 of the reference:
QK, position embedding, mask, blank token, softmax, AV, blank value)."""
import pytest
import torch

import workloads
from helpers import TOL, rel_err
from oracle import formula

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _chain(q, k, v, idx, pos_bias=None, pe_table=None, pe_idx=None, mask=None, blank_k=None, blank_v=None):
    q, k, v = q.double(), k.double(), v.double()
    b, h, n, c = q.shape
    attn = formula.qk(q, k, idx)
    if pos_bias is not None:
        attn = attn + pos_bias.double()
    if pe_table is not None:
        attn = attn + pe_table.double()[pe_idx].permute(0, 3, 1, 2)
    if mask is not None:
        attn = attn + (1 - mask.double()).unsqueeze(1) * -100
    if blank_k is not None:
        blank = (q * blank_k.double().reshape(1, h, 1, c)).sum(-1, keepdim=True)
        attn = torch.cat([attn, blank], -1)
    attn = attn.softmax(-1)
    if blank_k is not None:
        pb, attn = attn[..., -1:], attn[..., :-1]
    out = formula.av(attn, v, idx)
    if blank_k is not None:
        out = out + pb * blank_v.double().reshape(1, h, 1, c)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("regime", ["shared", "model", "random"])
@pytest.mark.parametrize("shape", [(2, 4, 200, 48), (2, 2, 73, 48), (1, 3, 96, 24), (2, 2, 64, 13)],
                         ids=lambda s: "x".join(map(str, s)))
def test_full_chain(lib, shape, regime, dtype):
    from clusten import ops
    b, h, n, m = shape
    c = 32
    if regime == "model" and m % 8:
        regime = "random"
    idx = workloads.make_index(regime, b, n, m, 400 + n).to(DEV)
    if regime == "random":
        idx[:, :, -3:] = 0                                   # repeated neighbours inside a row
    g = torch.Generator(device=DEV).manual_seed(401)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV).to(dtype)
    q, k, v = rn(b, h, n, c) * c ** -0.5, rn(b, h, n, c), rn(b, h, n, c)
    pos_bias = rn(b, h, n, m)
    table = rn(111, h)
    pe_idx = torch.randint(0, 111, (b, n, m), generator=g, device=DEV)
    mask = (torch.rand(b, n, m, generator=g, device=DEV) > 0.1).long()
    blank_k, blank_v = rn(h, c), rn(h, c)
    tol = TOL[dtype]
    got = ops.local_attention_forward(q, k, v, idx, pos_bias, table, pe_idx, mask, blank_k, blank_v)
    want = _chain(q, k, v, idx, pos_bias, table, pe_idx, mask, blank_k, blank_v)
    assert got.dtype == dtype and got.shape == (b, h, n, c)
    assert rel_err(got, want) <= tol, ("all terms", rel_err(got, want))
    # every optional term on its own, and none
    for kw in (dict(), dict(pos_bias=pos_bias), dict(pe_table=table, pe_idx=pe_idx), dict(mask=mask),
               dict(blank_k=blank_k, blank_v=blank_v)):
        got = ops.local_attention_forward(q, k, v, idx, **kw)
        want = _chain(q, k, v, idx, **kw)
        assert rel_err(got, want) <= tol, (sorted(kw), rel_err(got, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_on_model_style_views_and_against_the_separate_operators(lib, dtype):
    """query / key / value as views of the q and kv Linear outputs; the result agrees with the chain run through
    the separate operators of this package."""
    from clusten import ops
    b, h, n, m, c = 2, 4, 392, 48, 32
    idx = workloads.make_index("model", b, n, m, 410).to(DEV)
    g = torch.Generator(device=DEV).manual_seed(411)
    qlin = (torch.randn(b, n, h * c, generator=g, device=DEV) * c ** -0.5).to(dtype)
    kvlin = torch.randn(b, n, 2 * h * c, generator=g, device=DEV).to(dtype)
    q = qlin.reshape(b, n, h, c).permute(0, 2, 1, 3)
    kv = kvlin.view(b, n, h, 2, c).permute(3, 0, 2, 1, 4)
    key, v = kv[0], kv[1]
    table = torch.randn(111, h, generator=g, device=DEV).to(dtype)
    pe_idx = torch.randint(0, 111, (b, n, m), generator=g, device=DEV)
    blank_k = torch.randn(h, c, generator=g, device=DEV).to(dtype)
    blank_v = torch.randn(h, c, generator=g, device=DEV).to(dtype)
    got = ops.local_attention_forward(q, key, v, idx, pe_table=table, pe_idx=pe_idx, blank_k=blank_k, blank_v=blank_v)
    assert rel_err(got, _chain(q, key, v, idx, pe_table=table, pe_idx=pe_idx, blank_k=blank_k, blank_v=blank_v)) <= TOL[dtype]
    # the same chain through qk_forward / torch / av_forward
    attn = ops.qk_forward(q.contiguous(), key.contiguous(), idx).float() + table.float()[pe_idx].permute(0, 3, 1, 2)
    blank = (q.float() * blank_k.float().reshape(1, h, 1, c)).sum(-1, keepdim=True)
    attn = torch.cat([attn, blank], -1).softmax(-1)
    sep = ops.av_forward(attn[..., :-1].contiguous().to(dtype), v.contiguous(), idx).float() \
        + attn[..., -1:] * blank_v.float().reshape(1, h, 1, c)
    assert rel_err(got, sep) <= 2 * TOL[dtype]


def test_argument_checks(lib):
    p = 256
    call = lib.clusten_local_attention_forward
    assert call(p, None, p, p, None, p, None, p, None, 5, None, None, None, p, 1, 1, 8, 4, 32, 0, None) == -3   # table without indices
    assert call(p, None, p, p, None, p, None, None, None, 0, None, p, None, p, 1, 1, 8, 4, 32, 0, None) == -3   # blank_k without blank_v
    assert call(p, None, p, p, None, p, None, None, None, 0, None, None, None, p, 1, 1, 8, 64, 32, 0, None) == -6  # m above 48
    assert call(p, None, p, p, None, p, None, None, None, 0, None, None, None, p, 1, 1, 8, 4, 16, 0, None) == -6   # head dim
