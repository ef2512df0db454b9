"""CPU checks of the oracle itself: the C restatement against the PyTorch gather
formulation of the reference's tests, against a literal per-element loop, and
against stored outputs of the reference's own CUDA extension."""
import glob
import os

import numpy as np
import pytest
import torch

import workloads
from helpers import rel_err
from oracle import c_oracle, formula

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _case(regime, b, h, n, m, c, seed):
    idx = workloads.make_index(regime, b, n, m, seed)
    q, k, v, attn, g_attn, g_feat = workloads.attention_operands(b, h, n, m, c, torch.float32, seed + 1)
    return idx, q, k, v, attn, g_attn, g_feat


@pytest.mark.parametrize("regime", ["shared", "model", "random"])
def test_c_oracle_matches_formula_attention(regime):
    idx, q, k, v, attn, g_attn, g_feat = _case(regime, 2, 3, 136, 16, 32, 3)
    out, gq, gk = formula.forward_backward("qk", q, k, idx, g_attn)
    assert rel_err(c_oracle.qk_forward(q, k, idx), out) < 2e-6
    dq, dk = c_oracle.qk_backward(g_attn, q, k, idx)
    assert rel_err(dq, gq) < 2e-6 and rel_err(dk, gk) < 2e-6
    out, ga, gv = formula.forward_backward("av", attn, v, idx, g_feat)
    assert rel_err(c_oracle.av_forward(attn, v, idx), out) < 2e-6
    da, dv = c_oracle.av_backward(g_feat, attn, v, idx)
    assert rel_err(da, ga) < 2e-6 and rel_err(dv, gv) < 2e-6


@pytest.mark.parametrize("ic", [1, 4])
def test_c_oracle_matches_formula_wf(ic):
    b, n, n_out, m, c = 2, 136, 40, 16, 24
    idx = workloads.select_rows(workloads.make_index("shared", b, n, m, 5), n_out, 6)
    w, feat, g = workloads.merge_operands(b, n_out, n, m, ic, c, torch.float32, 7)
    out, gw, gf = formula.forward_backward("wf", w, feat, idx, g)
    assert rel_err(c_oracle.wf_forward(w, feat, idx), out) < 2e-6
    dw, df = c_oracle.wf_backward(g, w, feat, idx)
    assert rel_err(dw, gw) < 2e-6 and rel_err(df, gf) < 2e-6


def test_c_oracle_against_literal_loops():
    """The defining sums written out element by element on a tiny case (fp64, exact)."""
    torch.manual_seed(0)
    b, h, n, m, c = 1, 2, 6, 4, 3
    q, k, v = (torch.randn(b, h, n, c, dtype=torch.float64) for _ in range(3))
    attn = torch.randn(b, h, n, m, dtype=torch.float64)
    idx = torch.tensor([[[0, 0, 5, 2], [1, 1, 1, 1], [5, 4, 3, 2], [0, 1, 2, 3], [2, 2, 4, 4], [3, 0, 0, 3]]])
    qk = torch.zeros(b, h, n, m, dtype=torch.float64)
    av = torch.zeros(b, h, n, c, dtype=torch.float64)
    dk = torch.zeros_like(k)
    for z in range(h):
        for i in range(n):
            for j in range(m):
                t = idx[0, i, j]
                qk[0, z, i, j] = sum(q[0, z, i, cc] * k[0, z, t, cc] for cc in range(c))
                av[0, z, i] += attn[0, z, i, j] * v[0, z, t]
                dk[0, z, t] += q[0, z, i] * attn[0, z, i, j]
    assert torch.allclose(c_oracle.qk_forward(q, k, idx), qk, rtol=0, atol=1e-14)
    assert torch.allclose(c_oracle.av_forward(attn, v, idx), av, rtol=0, atol=1e-14)
    assert torch.allclose(c_oracle.qk_backward(attn, q, k, idx)[1], dk, rtol=0, atol=1e-14)


def test_formula_chunking_is_transparent():
    idx, q, k, v, attn, g_attn, g_feat = _case("shared", 4, 2, 72, 8, 16, 11)
    whole = formula.forward_backward("av", attn, v, idx, g_feat)
    parts = formula.forward_backward("av", attn, v, idx, g_feat, chunk=1)
    for a, b_ in zip(whole, parts):
        assert torch.equal(a, b_)


def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "ref_cuda_*.npz")))


@pytest.mark.parametrize("path", _golden_files() or [None])
def test_oracle_against_reference_cuda_outputs(path):
    """tests/golden/ref_cuda_*.npz hold inputs and the outputs of the reference's own CUDA
    extension (unmodified, run on a B200 by tests/golden/make_golden.py)."""
    if path is None:
        pytest.skip("no golden vectors stored yet")
    z = np.load(path)
    op = str(z["op"])
    t = {k_: torch.from_numpy(z[k_]) for k_ in z.files if k_ != "op"}
    tol = 1e-5
    if op == "qk":
        assert rel_err(c_oracle.qk_forward(t["q"], t["k"], t["idx"]), t["attn"]) < tol
        dq, dk = c_oracle.qk_backward(t["g"], t["q"], t["k"], t["idx"])
        assert rel_err(dq, t["dq"]) < tol and rel_err(dk, t["dk"]) < tol
        assert rel_err(formula.qk(t["q"], t["k"], t["idx"]), t["attn"]) < tol
    elif op == "av":
        assert rel_err(c_oracle.av_forward(t["attn"], t["v"], t["idx"]), t["feat"]) < tol
        da, dv = c_oracle.av_backward(t["g"], t["attn"], t["v"], t["idx"])
        assert rel_err(da, t["dattn"]) < tol and rel_err(dv, t["dv"]) < tol
        assert rel_err(formula.av(t["attn"], t["v"], t["idx"]), t["feat"]) < tol
    else:
        assert rel_err(c_oracle.wf_forward(t["w"], t["feat"], t["idx"]), t["out"]) < tol
        dw, df = c_oracle.wf_backward(t["g"], t["w"], t["feat"], t["idx"])
        assert rel_err(dw, t["dw"]) < tol and rel_err(df, t["dfeat"]) < tol
        assert rel_err(formula.wf(t["w"], t["feat"], t["idx"]), t["out"]) < tol
