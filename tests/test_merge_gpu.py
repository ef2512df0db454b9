"""clusten_merge_weights against the gather formulation of models/aff_transformer.py:340-358 (table rows by
pe_idx, times the neighbours' importance scores, times the mask): one rounding per element, so bit-exact."""
import pytest
import torch

from oracle import formula

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(b, n_out, n, m, ic, dtype, seed, rows=12321):
    g = torch.Generator(device=DEV).manual_seed(seed)
    table = torch.randn(rows, ic, generator=g, device=DEV).to(dtype)
    pe = torch.randint(rows, (b, n_out, m), generator=g, device=DEV)
    prob = torch.rand(b, n, 1, generator=g, device=DEV).to(dtype)
    idx = torch.randint(n, (b, n_out, m), generator=g, device=DEV)
    mask = torch.randint(2, (b, n_out, m), generator=g, device=DEV)
    return table, pe, prob, idx, mask


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["fp32", "bf16", "fp16"])
@pytest.mark.parametrize("b,n_out,n,m,ic", [(2, 784, 3136, 48, 4), (3, 49, 196, 48, 4), (2, 73, 368, 48, 4),
                                            (2, 50, 200, 24, 1), (1, 40, 100, 16, 3)])
def test_weights_match_the_formulation(lib, b, n_out, n, m, ic, dtype):
    from clusten import ops
    table, pe, prob, idx, mask = _case(b, n_out, n, m, ic, dtype, seed=n_out + ic)
    for p_, m_ in [(prob, mask), (prob, None), (None, mask), (None, None)]:
        got = ops.merge_weights(table, pe, p_, idx if p_ is not None else None, m_)
        want = formula.merge_weights(table, pe, p_, idx, m_)
        assert got.dtype == want.dtype and got.shape == (b, n_out, m, ic)
        assert torch.equal(got, want)


def test_mixed_dtypes_promote_like_the_products(lib):
    """A bf16 table (autocast Linear) with fp32 scores, and the other way round: fp32 weights either way."""
    from clusten import ops
    table, pe, prob, idx, mask = _case(2, 100, 400, 48, 4, torch.float32, seed=7)
    for t, p_ in [(table.bfloat16(), prob), (table, prob.bfloat16())]:
        got = ops.merge_weights(t, pe, p_, idx, mask)
        want = formula.merge_weights(t, pe, p_, idx, mask)
        assert got.dtype == torch.float32 == want.dtype
        assert torch.equal(got, want)


def test_feeds_the_merge_operator(lib):
    """The weights are CLUSTENWF's first argument: same merged features as with the formulation's weights."""
    from clusten import ops
    b, n_out, n, m, ic, c = 2, 196, 784, 48, 4, 64
    table, pe, prob, idx, mask = _case(b, n_out, n, m, ic, torch.float32, seed=11)
    feat = torch.randn(b, n, c, device=DEV)
    got = ops.wf_forward(ops.merge_weights(table, pe, prob, idx, mask), feat, idx)
    want = ops.wf_forward(formula.merge_weights(table, pe, prob, idx, mask).contiguous(), feat, idx)
    assert torch.equal(got, want)


def test_rows_and_tokens_out_of_range_give_zero(lib):
    from clusten import ops
    table, pe, prob, idx, mask = _case(1, 8, 32, 8, 4, torch.float32, seed=2, rows=50)
    pe[0, 0, 0] = 50
    pe[0, 0, 1] = -1
    idx[0, 1, 0] = 32
    got = ops.merge_weights(table, pe, prob, idx, None)
    assert bool((got[0, 0, 0] == 0).all()) and bool((got[0, 0, 1] == 0).all()) and bool((got[0, 1, 0] == 0).all())
    assert bool((got[0, 2] != 0).any())


def test_argument_checks(lib):
    p = 256
    assert lib.clusten_merge_weights(p, p, None, None, None, p, 0, 4, 4, 4, 4, 10, 0, None) == -2
    assert lib.clusten_merge_weights(None, p, None, None, None, p, 1, 4, 4, 4, 4, 10, 0, None) == -3
    assert lib.clusten_merge_weights(p, p, p, None, None, p, 1, 4, 4, 4, 4, 10, 0, None) == -3   # scores without tokens
    assert lib.clusten_merge_weights(p, p, None, None, None, p, 1, 4, 4, 4, 4, 10, 3, None) == -1  # fp64
