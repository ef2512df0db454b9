"""Parity of the CUDA operators (called through the C ABI) with the oracle on the
same seeded inputs.  Integer/index work must be exact; floating results are
compared with max|x - ref| / max|ref| against the fp64 oracle evaluated on the
dtype-rounded inputs, tolerance per dtype in helpers.TOL (fp32 1e-5, bf16 2e-2)."""
import pytest
import torch

import workloads
from helpers import TOL, assert_close, exact, rel_err
from oracle import formula, ref_cuda

pytestmark = pytest.mark.gpu

DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16, torch.float16]


@pytest.fixture(scope="module")
def ops(lib):
    from clusten import ops as _ops
    return _ops


def _attention_case(regime, b, h, n, m, c, dtype, seed):
    if regime == "model" and (m % 8 or n < 8):
        regime = "random"
    idx = workloads.make_index(regime, b, n, m, seed).to(DEV)
    t = workloads.attention_operands(b, h, n, m, c, dtype, seed + 1)
    return (idx,) + tuple(x.to(DEV) for x in t)


# (b, h, n, m, c): cluster-structured stages, the reference tests' shape, a padded stage (n % 8 != 0),
# m = n = 49 (every token is a neighbour), head_dim 32 with m below 48 (the kernels' runtime-sized variants),
# m = 144, head dims other than 32, n < m
ATT_SHAPES = [
    (2, 2, 392, 48, 32),
    (3, 4, 196, 48, 32),
    (2, 3, 73, 48, 32),
    (2, 2, 49, 49, 32),
    (2, 2, 100, 24, 32),
    (1, 3, 64, 40, 32),
    (2, 2, 57, 13, 32),
    (1, 2, 160, 144, 32),
    (2, 2, 64, 16, 16),
    (1, 1, 40, 9, 24),
    (1, 2, 96, 24, 64),
    (1, 1, 5, 12, 7),
    # config 0 of the benchmark (QK forward on CPU there), the stage shapes of the per-stage sweep at small
    # batch (h = 8 / n = 196, h = 16 / n = 49 with m = 49) and the padded stages of the 384 x 384 model
    (2, 2, 3136, 48, 32),
    (2, 8, 196, 48, 32),
    (2, 16, 49, 49, 32),
    (1, 16, 368, 48, 32),
    (2, 32, 73, 48, 32),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("regime", ["shared", "model", "random"])
@pytest.mark.parametrize("shape", ATT_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_qk_av_forward_backward(ops, shape, regime, dtype):
    b, h, n, m, c = shape
    idx, q, k, v, attn, g_attn, g_feat = _attention_case(regime, b, h, n, m, c, dtype, 100 + n)
    out = ops.qk_forward(q, k, idx)
    assert out.dtype == dtype and out.is_contiguous()
    assert_close(out, exact("qk", "forward", q, k, idx), dtype, "qk forward")
    dq, dk = ops.qk_backward(g_attn, q, k, idx)
    rq, rk = exact("qk", "backward", g_attn, q, k, idx)
    assert_close(dq, rq, dtype, "d_query")
    assert_close(dk, rk, dtype, "d_key")

    feat = ops.av_forward(attn, v, idx)
    assert_close(feat, exact("av", "forward", attn, v, idx), dtype, "av forward")
    da, dv = ops.av_backward(g_feat, attn, v, idx)
    ra, rv = exact("av", "backward", g_feat, attn, v, idx)
    assert_close(da, ra, dtype, "d_attn")
    assert_close(dv, rv, dtype, "d_value")


def test_fp64_is_accepted(ops):
    idx, q, k, v, attn, g_attn, g_feat = _attention_case("random", 2, 2, 64, 16, 32, torch.float64, 5)
    assert_close(ops.qk_forward(q, k, idx), exact("qk", "forward", q, k, idx), torch.float64, "qk f64")
    da, dv = ops.av_backward(g_feat, attn, v, idx)
    ra, rv = exact("av", "backward", g_feat, attn, v, idx)
    assert_close(da, ra, torch.float64, "d_attn f64")
    assert_close(dv, rv, torch.float64, "d_value f64")


# (b, n_out, n, m, ic, c)
WF_SHAPES = [
    (2, 98, 392, 48, 1, 64),
    (2, 98, 392, 48, 4, 64),
    (3, 64, 196, 48, 4, 32),
    (2, 36, 184, 48, 4, 128),
    (1, 14, 73, 48, 4, 256),
    (2, 51, 392, 48, 2, 64),
    (2, 40, 160, 24, 4, 64),
    (1, 33, 90, 13, 2, 128),
    (1, 20, 100, 16, 3, 24),
    (1, 7, 30, 5, 2, 9),
    # m above 48 on the tiled d_feat path; ic = 3 and ic = 16 with 32-channel slabs on the tiled scatter path
    (1, 20, 100, 80, 4, 64),
    (1, 20, 100, 16, 3, 32),
    (1, 12, 60, 24, 16, 32),
    # odd row counts (the walks take rows two at a time), one neighbour, 17 neighbours, 192 channels, a single row
    (3, 5, 40, 1, 4, 64),
    (1, 7, 30, 17, 4, 192),
    (2, 1, 16, 48, 4, 64),
    # the merges of the 384 x 384 model at 1/5 retention: 1843 -> 368 and 368 -> 73 rows
    (1, 368, 1843, 48, 4, 64),
    (2, 73, 368, 48, 4, 128),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("regime", ["shared", "model", "random"])
@pytest.mark.parametrize("shape", WF_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_wf_forward_backward(ops, shape, regime, dtype):
    b, n_out, n, m, ic, c = shape
    if regime == "model" and m % 8:
        regime = "random"
    if regime == "random":
        idx = workloads.random_rows(b, n_out, n, m, 7).to(DEV)
    else:
        idx = workloads.select_rows(workloads.make_index(regime, b, n, m, 9), n_out, 10).to(DEV)
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, c, dtype, 11))
    out = ops.wf_forward(w, feat, idx)
    assert out.shape == (b, n_out, ic, c) and out.dtype == dtype
    assert_close(out, exact("wf", "forward", w, feat, idx), dtype, "wf forward")
    dw, df = ops.wf_backward(g, w, feat, idx)
    rw, rf = exact("wf", "backward", g, w, feat, idx)
    assert_close(dw, rw, dtype, "d_weights")
    assert_close(df, rf, dtype, "d_feat")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("regime", ["shared", "model", "random"])
@pytest.mark.parametrize("shape", [(2, 98, 392, 48, 4, 64), (1, 50, 200, 24, 1, 128), (2, 73, 368, 48, 4, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_wf_forward_both_kernels(ops, shape, regime, dtype, monkeypatch):
    """WF forward has two kernels: the walk over the neighbours (default) and the tiled one (selected by
    CLUSTEN_WF_FORWARD_TILED, which the library reads at every call).  Both against the oracle, and the walk
    twice for bit-reproducibility."""
    b, n_out, n, m, ic, c = shape
    if regime == "random":
        idx = workloads.random_rows(b, n_out, n, m, 7).to(DEV)
    else:
        idx = workloads.select_rows(workloads.make_index(regime, b, n, m, 9), n_out, 10).to(DEV)
    w, feat, _ = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, c, dtype, 11))
    want = exact("wf", "forward", w, feat, idx)
    walk = ops.wf_forward(w, feat, idx)
    assert torch.equal(walk, ops.wf_forward(w, feat, idx))
    assert_close(walk, want, dtype, "wf forward (walk)")
    assert_close(ops.wf_forward(w, feat, idx, row_order=False), want, dtype, "wf forward (walk, storage order)")
    monkeypatch.setenv("CLUSTEN_WF_FORWARD_TILED", "1")
    tiled = ops.wf_forward(w, feat, idx)
    monkeypatch.delenv("CLUSTEN_WF_FORWARD_TILED")
    assert_close(tiled, want, dtype, "wf forward (tiled)")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("regime", ["shared", "model", "random", "shared-hot"])
@pytest.mark.parametrize("shape", [(2, 99, 392, 48, 4, 128), (1, 200, 800, 48, 1, 64), (2, 50, 200, 24, 2, 64)],
                         ids=lambda s: "x".join(map(str, s)))
def test_wf_d_feat_both_kernels(ops, shape, regime, dtype, monkeypatch):
    """d_feat has two kernels: gradient rows staged in shared memory and multiplied on the tensor cores, or read
    straight into registers and added with FMAs (CLUSTEN_WF_DFEAT = staged | rows, read at every call).  Both
    against the oracle, for both dtypes; "shared-hot" makes one token a neighbour of every row, so that its entry
    list spans several chunks."""
    b, n_out, n, m, ic, c = shape
    if regime == "random":
        idx = workloads.random_rows(b, n_out, n, m, 7).to(DEV)
    else:
        idx = workloads.select_rows(workloads.make_index(regime.split("-")[0], b, n, m, 9), n_out, 10).to(DEV)
    if regime.endswith("hot"):
        idx[:, :, -1] = 5
        idx[:, ::2, -2] = 5          # ... twice in every other row
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, c, dtype, 11))
    _, rf = exact("wf", "backward", g, w, feat, idx)
    for kind in ("rows", "staged"):
        monkeypatch.setenv("CLUSTEN_WF_DFEAT", kind)
        _, df = ops.wf_backward(g, w, feat, idx)
        assert_close(df, rf, dtype, f"d_feat ({kind})")
        assert torch.equal(df, ops.wf_backward(g, w, feat, idx)[1])
    monkeypatch.delenv("CLUSTEN_WF_DFEAT")


@pytest.mark.parametrize("regime", ["shared", "model", "random"])
def test_wf_d_weights_fp32_both_kernels(ops, regime, monkeypatch):
    """fp32 d_weights with ic = 4: the walk with the 16-lane butterfly (default) and the tiled kernel
    (CLUSTEN_WF_DWEIGHTS_TILED), both against the oracle; a row with absent neighbours takes the checked path."""
    b, n_out, n, m, ic, c = 2, 99, 392, 48, 4, 128
    if regime == "random":
        idx = workloads.random_rows(b, n_out, n, m, 7).to(DEV)
    else:
        idx = workloads.select_rows(workloads.make_index(regime, b, n, m, 9), n_out, 10).to(DEV)
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, c, torch.float32, 11))
    rw, _ = exact("wf", "backward", g, w, feat, idx)
    dw, _ = ops.wf_backward(g, w, feat, idx)
    assert_close(dw, rw, torch.float32, "d_weights (walk)")
    assert torch.equal(dw, ops.wf_backward(g, w, feat, idx)[0])
    monkeypatch.setenv("CLUSTEN_WF_DWEIGHTS_TILED", "1")
    dw_t, _ = ops.wf_backward(g, w, feat, idx)
    monkeypatch.delenv("CLUSTEN_WF_DWEIGHTS_TILED")
    assert_close(dw_t, rw, torch.float32, "d_weights (tiled)")
    bad = idx.clone()
    bad[0, 3, 5] = -1
    bad[1, 7, 40] = n + 3
    mask = ((bad >= 0) & (bad < n)).float().unsqueeze(-1)
    dw_b, _ = ops.wf_backward(g, w, feat, bad)
    _, rw_b, _ = formula.forward_backward("wf", w * mask, feat, bad.clamp(0, n - 1), g)
    assert_close(dw_b, rw_b * mask, torch.float32, "d_weights (walk) with bad indices")


# (n, m, n_targets): one warp per chunk of rows with m <= 32, <= 64 and > 64; few rows; and a target count
# whose per-chunk counters do not fit in shared memory (32 rows at a time instead)
INVERSE_SHAPES = [(203, 48, 203), (203, 24, 203), (77, 80, 77), (5, 12, 5), (203, 48, 17500)]


@pytest.mark.parametrize("shape", INVERSE_SHAPES + [(648, 48, 648), (200, 16, 200)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("regime", ["shared", "model", "random", "shared-repeats", "model-repeats", "shared-hot"])
def test_inverse_index_is_exact(ops, regime, shape):
    """Every (row, slot) appears exactly once under its target, rows ascending; repeated
    targets of a row are folded into one flagged entry.  Cluster-shared and run-structured tables take
    the structured build, also when a cluster's row repeats a token, a row names a run twice, or one
    token is named by every cluster (a list too long for one thread to sort)."""
    b = 3
    n, m, nt = shape
    regime, _, variant = regime.partition("-")
    if n < m or (regime == "model" and m % 8):
        regime = "random"
    idx = workloads.make_index(regime, b, n, m, 21) if regime != "random" else workloads.random_rows(b, n, n, m, 21)
    if regime == "random":
        idx[:, :, -3:] = 0          # padded-stage pattern: several slots of a row point at token 0
        idx[0, 0, 1] = idx[0, 0, m - 2]     # a repeat across the 32-slot batches of a row
    elif variant == "repeats" and regime == "shared":
        idx[:, :, 1] = idx[:, :, 0]                   # still one row per cluster, but it names a token twice
        idx[1, :, m - 1] = idx[1, :, 2]
    elif variant == "repeats" and m >= 16:
        idx[:, ::3, 8:16] = idx[:, ::3, 0:8]          # every third row names its first run twice
    elif variant == "hot":
        idx[:, :, m - 1] = 5                          # every cluster names token 5
        idx[2, :, m - 2] = 5                          # ... twice in the last batch element
    inv = ops.build_inverse(idx.to(DEV), nt).cpu()
    hdr = inv[:64]
    assert hdr[1] == b and hdr[2] == n and hdr[3] == m and hdr[4] == nt and hdr[5] == 0
    pad = lambda x: (x + 63) // 64 * 64
    o = 64
    rowptr = inv[o:o + b * (nt + 1)].view(b, nt + 1); o += pad(b * (nt + 1))
    seglen = inv[o:o + b * nt].view(b, nt); o += pad(b * nt)
    entries = inv[o:o + b * n * m].view(b, n * m)
    for bi in range(b):
        counts = torch.bincount(idx[bi].flatten(), minlength=nt)
        room = rowptr[bi, 1:] - rowptr[bi, :-1]
        assert rowptr[bi, 0] == 0 and bool((room >= seglen[bi]).all()) and bool((room <= counts.int()).all())
        assert bool((seglen[bi, n:] == 0).all())
        for t in range(n):
            seg = entries[bi, rowptr[bi, t]:rowptr[bi, t] + seglen[bi, t]].long()
            flagged = seg < 0
            rows = torch.where(flagged, (seg & 0x7fffffff) // m, seg // m)
            want_rows = (idx[bi] == t).any(1).nonzero().flatten()
            assert torch.equal(rows, want_rows), (bi, t)
            mult = (idx[bi][rows] == t).sum(1)
            assert torch.equal(flagged, mult > 1)
            slots = seg[~flagged] % m
            assert (idx[bi][rows[~flagged], slots] == t).all()


@pytest.mark.parametrize("shape", [(1, 2, 64, 16, 32), (2, 2, 104, 48, 32)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("regime", ["random", "model"])
def test_out_of_range_indices_are_ignored(ops, regime, shape):
    b, h, n, m, c = shape
    idx, q, k, v, attn, g_attn, g_feat = _attention_case(regime, b, h, n, m, c, torch.float32, 31)
    bad = idx.clone()
    bad[0, ::3, 5] = n + 7
    bad[0, 1::3, 2] = -1
    mask = ((bad >= 0) & (bad < n)).float().unsqueeze(1)             # [b,1,n,m]
    safe = bad.clamp(0, n - 1)
    ref = formula.qk(q, k, safe) * mask
    assert_close(ops.qk_forward(q, k, bad), ref, torch.float32, "qk with bad indices")
    ref = formula.av(attn * mask, v, safe)
    assert_close(ops.av_forward(attn, v, bad), ref, torch.float32, "av with bad indices")
    da, dv = ops.av_backward(g_feat, attn, v, bad)
    _, ra, rv = formula.forward_backward("av", attn * mask, v, safe, g_feat)
    assert_close(da, ra * mask, torch.float32, "d_attn with bad indices")
    assert_close(dv, rv, torch.float32, "d_value with bad indices")
    assert ops.build_inverse(bad, n)[5].item() == int((mask == 0).sum())


def test_wf_out_of_range_indices_are_ignored(ops):
    b, n_out, n, m, ic, c = 2, 37, 120, 48, 4, 64
    idx = workloads.select_rows(workloads.make_index("model", b, n, m, 9), n_out, 10).to(DEV)
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, c, torch.float32, 11))
    bad = idx.clone()
    bad[0, ::3, 5] = n + 7
    bad[1, 1::3, 2] = -1
    bad[1, 4, :] = -5                                                # a row without any neighbour
    mask = ((bad >= 0) & (bad < n)).float().unsqueeze(-1)            # [b,n_out,m,1]
    safe = bad.clamp(0, n - 1)
    assert_close(ops.wf_forward(w, feat, bad), formula.wf(w * mask, feat, safe), torch.float32, "wf with bad indices")
    dw, df = ops.wf_backward(g, w, feat, bad)
    _, rw, rf = formula.forward_backward("wf", w * mask, feat, safe, g)
    assert_close(dw, rw * mask, torch.float32, "d_weights with bad indices")
    assert_close(df, rf, torch.float32, "d_feat with bad indices")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_wf_row_order_variants(ops, dtype):
    """The row order only groups the rows: storage order, the built order, any permutation and a stage
    with more rows than the order kernel sorts give the same results."""
    b, n_out, n, m, ic, c = 2, 203, 812, 48, 4, 64
    idx = workloads.select_rows(workloads.make_index("shared", b, n, m, 9), n_out, 10).to(DEV)
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, c, dtype, 11))
    order = ops.build_row_order(idx)
    assert order.dtype == torch.int32 and order.shape == (b, n_out)
    assert torch.equal(order.long().sort(dim=1).values, torch.arange(n_out, device=DEV).expand(b, n_out))
    first = idx[:, :, 0].gather(1, order.long())
    assert bool((first[:, 1:] >= first[:, :-1]).all())
    ref_out = exact("wf", "forward", w, feat, idx)
    ref_dw, ref_df = exact("wf", "backward", g, w, feat, idx)
    perm = torch.stack([torch.randperm(n_out, device=DEV) for _ in range(b)]).int().contiguous()
    for ro in (None, False, order, perm):
        assert_close(ops.wf_forward(w, feat, idx, ro), ref_out, dtype, "wf forward")
        dw, df = ops.wf_backward(g, w, feat, idx, None, ro)
        assert_close(dw, ref_dw, dtype, "d_weights")
        assert_close(df, ref_df, dtype, "d_feat")
    with pytest.raises(RuntimeError):
        ops.wf_forward(w, feat, idx, order[:, :-1].contiguous())
    big = torch.randint(0, 64, (1, 4100, 8), device=DEV)
    assert ops.build_row_order(big) is None
    w2, feat2, g2 = (x.to(DEV) for x in workloads.merge_operands(1, 4100, 64, 8, 1, 64, dtype, 12))
    assert_close(ops.wf_forward(w2, feat2, big), exact("wf", "forward", w2, feat2, big), dtype, "wf forward, no order")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_backward_is_bit_reproducible(ops, dtype):
    """No atomics on floating data: two runs give identical bits, also with repeated indices."""
    idx, q, k, v, attn, g_attn, g_feat = _attention_case("random", 4, 4, 196, 48, 32, dtype, 41)
    idx[:, :, -5:] = 0
    first = ops.qk_backward(g_attn, q, k, idx) + ops.av_backward(g_feat, attn, v, idx)
    ops.clear_inverse_cache()
    again = ops.qk_backward(g_attn, q, k, idx) + ops.av_backward(g_feat, attn, v, idx)
    for a, b_ in zip(first, again):
        assert torch.equal(a, b_)


def test_autograd_functions_on_model_style_views(ops):
    """The operators as the model calls them (models/aff_transformer.py:117-120,145-154 of the
    reference): q/k/v are permuted views of Linear outputs, attn a [..., :-1] slice."""
    from clusten import CLUSTENAVFunction, CLUSTENQKFunction, CLUSTENWFFunction
    torch.manual_seed(3)
    b, h, n, m, c = 2, 4, 200, 48, 32
    idx = workloads.model_like_rows(b, n, m, 51).to(DEV)
    qlin = torch.randn(b, n, h * c, device=DEV, requires_grad=True)
    kvlin = torch.randn(b, n, 2 * h * c, device=DEV, requires_grad=True)

    def run(qk_fn, av_fn):
        q = qlin.reshape(b, n, h, c).permute(0, 2, 1, 3)
        kv = kvlin.view(b, n, h, 2, c).permute(3, 0, 2, 1, 4)
        key, v = kv[0], kv[1]
        attn = qk_fn(q, key, idx)
        attn = torch.cat([attn, attn.new_zeros(b, h, n, 1)], -1).softmax(-1)[..., :-1]
        feat = av_fn(attn, v, idx).permute(0, 2, 1, 3).reshape(b, n, h * c)
        loss = (feat * torch.linspace(-1, 1, h * c, device=DEV)).sum()
        gq, gkv = torch.autograd.grad(loss, [qlin, kvlin])
        return feat, gq, gkv

    got = run(CLUSTENQKFunction.apply, CLUSTENAVFunction.apply)
    want = run(formula.qk, formula.av)
    for g_, w_, name in zip(got, want, ["feat", "grad q", "grad kv"]):
        assert rel_err(g_, w_) < 2e-5, name

    w = torch.randn(b, 50, m, 4, device=DEV, requires_grad=True)
    f = torch.randn(b, n, 64, device=DEV, dtype=torch.float16, requires_grad=True)   # cast to weights' dtype
    idx_w = workloads.select_rows(idx, 50, 52)
    out = CLUSTENWFFunction.apply(w, f, idx_w)
    assert out.dtype == torch.float32 and out.shape == (b, 50, 4, 64)
    gw, gf = torch.autograd.grad(out.square().sum(), [w, f])
    ref = formula.wf(w, f.float(), idx_w)
    rgw, rgf = torch.autograd.grad(ref.square().sum(), [w, f])
    assert rel_err(out, ref) < 2e-5 and rel_err(gw, rgw) < 2e-5 and rel_err(gf, rgf) < 2e-3
    assert gf.dtype == torch.float16
    with torch.no_grad():
        assert torch.equal(CLUSTENWFFunction.apply(w, f, idx_w), out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["float32", "float16"])
def test_against_the_reference_cuda_extension(ops, dtype):
    """The reference's own kernels (compiled unmodified into oracle/_ref) on the same inputs."""
    if not ref_cuda.available():
        pytest.skip("oracle/_ref is not built")
    tol = 1e-5 if dtype == torch.float32 else 1e-2   # the reference accumulates fp16 sums in fp16
    b, h, n, m, c = 4, 4, 196, 48, 32
    idx, q, k, v, attn, g_attn, g_feat = _attention_case("random", b, h, n, m, c, dtype, 61)
    assert rel_err(ops.qk_forward(q, k, idx), ref_cuda.qk_forward(q, k, idx)) < tol
    for mine, ref in zip(ops.qk_backward(g_attn, q, k, idx), ref_cuda.qk_backward(g_attn, q, k, idx)):
        assert rel_err(mine, ref) < tol
    assert rel_err(ops.av_forward(attn, v, idx), ref_cuda.av_forward(attn, v, idx)) < tol
    for mine, ref in zip(ops.av_backward(g_feat, attn, v, idx), ref_cuda.av_backward(g_feat, attn, v, idx)):
        assert rel_err(mine, ref) < tol
    n_out, ic, cw = 64, 4, 32
    idx_w = workloads.random_rows(b, n_out, n, m, 62).to(DEV)
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, cw, dtype, 63))
    assert rel_err(ops.wf_forward(w, feat, idx_w), ref_cuda.wf_forward(w, feat, idx_w)) < tol
    for mine, ref in zip(ops.wf_backward(g, w, feat, idx_w), ref_cuda.wf_backward(g, w, feat, idx_w)):
        assert rel_err(mine, ref) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("regime", ["shared", "model"])
def test_full_size_adjoint_identities(ops, regime, dtype):
    """Stage-1 shapes of the benchmark (b=128, h=2, n=3136, m=48, c=32; WF n_=784, c=64, ic=4),
    where the oracle is too slow: each operator is bilinear, so <op(x, y), g> must equal
    <x, grad_x> and <y, grad_y>, which ties forward, both gradients and the inverse index
    together at full size.  Two batch elements are also compared, forward and all gradients, with the
    gather formulation evaluated in fp32 on the GPU."""
    b, h, n, m, c = 128, 2, 3136, 48, 32
    idx = workloads.make_index(regime, b, n, m, 71, DEV)
    q, k, v, attn, g_attn, g_feat = workloads.attention_operands(b, h, n, m, c, dtype, 72, DEV)
    eps = 2.0 ** -23 if dtype == torch.float32 else 2.0 ** -8

    def dot(x, y):
        return (x.double() * y.double()).sum().item()

    def same_product(lhs_pair, *rhs_pairs):
        """<a, b> of every pair agrees with the first one up to the rounding of the outputs: each output
        element carries a relative error of about eps, so the sums differ by about eps * |terms|_2."""
        a, b_ = lhs_pair
        lhs = dot(a, b_)
        scale = (a.double() * b_.double()).pow(2).sum().sqrt().item()
        for x, y in rhs_pairs:
            scale_r = (x.double() * y.double()).pow(2).sum().sqrt().item()
            assert abs(dot(x, y) - lhs) <= 8 * eps * max(scale, scale_r) + 1e-5 * abs(lhs), (dot(x, y), lhs, scale)

    sl = slice(5, 7)
    f32 = lambda *ts: [t[sl].float() for t in ts]
    out = ops.qk_forward(q, k, idx)
    dq, dk = ops.qk_backward(g_attn, q, k, idx)
    same_product((out, g_attn), (q, dq), (k, dk))
    ro, rq, rk = formula.forward_backward("qk", *f32(q, k), idx[sl], g_attn[sl].float())
    assert rel_err(out[sl], ro) <= TOL[dtype] and rel_err(dq[sl], rq) <= TOL[dtype] and rel_err(dk[sl], rk) <= TOL[dtype]
    feat = ops.av_forward(attn, v, idx)
    da, dv = ops.av_backward(g_feat, attn, v, idx)
    same_product((feat, g_feat), (attn, da), (v, dv))
    ro, ra, rv = formula.forward_backward("av", *f32(attn, v), idx[sl], g_feat[sl].float())
    assert rel_err(feat[sl], ro) <= TOL[dtype] and rel_err(da[sl], ra) <= TOL[dtype] and rel_err(dv[sl], rv) <= TOL[dtype]

    n_out, ic, cw = 784, 4, 64
    idx_w = workloads.select_rows(idx, n_out, 73)
    w, f, g = workloads.merge_operands(b, n_out, n, m, ic, cw, dtype, 74, DEV)
    out = ops.wf_forward(w, f, idx_w)
    dw, df = ops.wf_backward(g, w, f, idx_w)
    same_product((out, g), (w, dw), (f, df))
    ro, rw, rf = formula.forward_backward("wf", *f32(w, f), idx_w[sl], g[sl].float())
    assert rel_err(out[sl], ro) <= TOL[dtype] and rel_err(dw[sl], rw) <= TOL[dtype] and rel_err(df[sl], rf) <= TOL[dtype]


# ----------------------------------------------------------------------------- paths that ordinary tables do not reach
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("repeats", [1, 3])
def test_hot_token_segments_span_several_chunks(ops, repeats, dtype):
    """Every row names token 0 (once, or three times as the padded stages do, models/point_utils.py:189-206
    of the reference), so the tile of targets 0..7 has far more edges than the scatter kernels take at a
    time: later chunks accumulate onto what earlier ones wrote."""
    b, h, n, m, c = 2, 2, 648, 48, 32
    for regime in ("shared", "model", "random"):
        idx, q, k, v, attn, g_attn, g_feat = _attention_case(regime, b, h, n, m, c, dtype, 300 + repeats)
        idx[:, :, -repeats:] = 0
        dq, dk = ops.qk_backward(g_attn, q, k, idx)
        rq, rk = exact("qk", "backward", g_attn, q, k, idx)
        assert_close(dq, rq, dtype, f"d_query ({regime})")
        assert_close(dk, rk, dtype, f"d_key ({regime})")
        da, dv = ops.av_backward(g_feat, attn, v, idx)
        ra, rv = exact("av", "backward", g_feat, attn, v, idx)
        assert_close(da, ra, dtype, f"d_attn ({regime})")
        assert_close(dv, rv, dtype, f"d_value ({regime})")
    # the merge operator with 408 rows that all name token 0
    n_out, ic, cw = 408, 4, 64
    idx_w = workloads.select_rows(workloads.make_index("model", b, n, m, 310), n_out, 311).to(DEV)
    idx_w[:, :, -repeats:] = 0
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, cw, dtype, 312))
    assert_close(ops.wf_forward(w, feat, idx_w), exact("wf", "forward", w, feat, idx_w), dtype, "wf forward")
    dw, df = ops.wf_backward(g, w, feat, idx_w)
    rw, rf = exact("wf", "backward", g, w, feat, idx_w)
    assert_close(dw, rw, dtype, "d_weights")
    assert_close(df, rf, dtype, "d_feat")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("regime", ["shared", "model", "random"])
def test_token_ids_beyond_8192(ops, regime, dtype):
    """Stage 1 of the 384 x 384 model has 9216 tokens: the ids of one tile of random rows then span more
    than the de-duplication bitmap covers (one slot per edge instead), and the merge gathers from
    9216 tokens into 1843 rows (1/5 retention, not a multiple of 8)."""
    b, h, n, m, c = 1, 4, 9216, 48, 32
    idx, q, k, v, attn, g_attn, g_feat = _attention_case(regime, b, h, n, m, c, dtype, 320)
    assert_close(ops.qk_forward(q, k, idx), exact("qk", "forward", q, k, idx), dtype, "qk forward")
    dq, dk = ops.qk_backward(g_attn, q, k, idx)
    rq, rk = exact("qk", "backward", g_attn, q, k, idx)
    assert_close(dq, rq, dtype, "d_query")
    assert_close(dk, rk, dtype, "d_key")
    assert_close(ops.av_forward(attn, v, idx), exact("av", "forward", attn, v, idx), dtype, "av forward")
    da, dv = ops.av_backward(g_feat, attn, v, idx)
    ra, rv = exact("av", "backward", g_feat, attn, v, idx)
    assert_close(da, ra, dtype, "d_attn")
    assert_close(dv, rv, dtype, "d_value")
    n_out, ic, cw = 1843, 4, 128
    idx_w = workloads.select_rows(idx.cpu(), n_out, 321).to(DEV) if regime != "random" else \
        workloads.random_rows(b, n_out, n, m, 321).to(DEV)
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, cw, dtype, 322))
    assert_close(ops.wf_forward(w, feat, idx_w), exact("wf", "forward", w, feat, idx_w), dtype, "wf forward")
    dw, df = ops.wf_backward(g, w, feat, idx_w)
    rw, rf = exact("wf", "backward", g, w, feat, idx_w)
    assert_close(dw, rw, dtype, "d_weights")
    assert_close(df, rf, dtype, "d_feat")


def test_wf_rows_that_repeat_a_neighbour(ops):
    """Merge rows that name one token several times, on the tiled paths with ic = 3, ic = 16 and m = 80."""
    for (b, n_out, n, m, ic, c) in [(1, 20, 100, 16, 3, 32), (1, 12, 60, 24, 16, 32), (1, 20, 100, 80, 4, 64)]:
        idx = workloads.random_rows(b, n_out, n, m, 330).to(DEV)
        idx[:, :, 1] = idx[:, :, 0]
        idx[:, ::2, -1] = idx[:, ::2, 2]
        w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, c, torch.float32, 331))
        assert_close(ops.wf_forward(w, feat, idx), exact("wf", "forward", w, feat, idx), torch.float32, "wf forward")
        dw, df = ops.wf_backward(g, w, feat, idx)
        rw, rf = exact("wf", "backward", g, w, feat, idx)
        assert_close(dw, rw, torch.float32, "d_weights")
        assert_close(df, rf, torch.float32, "d_feat")


def test_fp32_products_with_widely_spread_magnitudes(ops, capsys):
    """FP32 inputs are multiplied as three TF32 passes (high x high, high x low, low x high).  With
    magnitudes spread over 2^-20 .. 2^20 the error must still stay inside the fp32 tolerance; the margin
    is printed."""
    b, h, n, m, c = 2, 2, 392, 48, 32
    idx, q, k, v, attn, g_attn, g_feat = _attention_case("shared", b, h, n, m, c, torch.float32, 340)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(341)

    def spread(t):
        e = torch.randint(-20, 21, t.shape, generator=gen, device=DEV).float()
        return t * torch.exp2(e)

    q, k, v, g_attn, g_feat = (spread(t) for t in (q, k, v, g_attn, g_feat))
    errs = {"qk forward": rel_err(ops.qk_forward(q, k, idx), exact("qk", "forward", q, k, idx)),
            "av forward": rel_err(ops.av_forward(attn, v, idx), exact("av", "forward", attn, v, idx))}
    dq, dk = ops.qk_backward(g_attn, q, k, idx)
    rq, rk = exact("qk", "backward", g_attn, q, k, idx)
    da, dv = ops.av_backward(g_feat, attn, v, idx)
    ra, rv = exact("av", "backward", g_feat, attn, v, idx)
    errs.update({"d_query": rel_err(dq, rq), "d_key": rel_err(dk, rk), "d_attn": rel_err(da, ra),
                 "d_value": rel_err(dv, rv)})
    with capsys.disabled():
        print("\nfp32 three-pass TF32 products, inputs scaled by 2^[-20, 20]:",
              {k_: f"{e:.2e} ({TOL[torch.float32] / max(e, 1e-30):.1f}x inside)" for k_, e in errs.items()})
    assert max(errs.values()) <= TOL[torch.float32], errs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_more_targets_than_fit_in_shared_memory(ops, dtype):
    """n = 20000 tokens (a 640 x 640 input): the inverse build keeps its per-target counters in global
    memory; the reference's atomicAdd scatter has no size limit (clusten/src/clustenqk_cuda_kernel.cu:125)."""
    b, h, n, m, c = 1, 2, 20000, 16, 32
    for regime in ("model", "random"):
        idx, q, k, v, attn, g_attn, g_feat = _attention_case(regime, b, h, n, m, c, dtype, 350)
        if regime == "random":
            idx[:, :, -2:] = 0
        dq, dk = ops.qk_backward(g_attn, q, k, idx)
        rq, rk = exact("qk", "backward", g_attn, q, k, idx)
        assert_close(dq, rq, dtype, f"d_query ({regime})")
        assert_close(dk, rk, dtype, f"d_key ({regime})")
        da, dv = ops.av_backward(g_feat, attn, v, idx)
        ra, rv = exact("av", "backward", g_feat, attn, v, idx)
        assert_close(da, ra, dtype, f"d_attn ({regime})")
        assert_close(dv, rv, dtype, f"d_value ({regime})")
    n_out, ic, cw = 4000, 4, 64
    idx_w = workloads.random_rows(b, n_out, n, m, 351).to(DEV)
    w, feat, g = (x.to(DEV) for x in workloads.merge_operands(b, n_out, n, m, ic, cw, dtype, 352))
    dw, df = ops.wf_backward(g, w, feat, idx_w)
    rw, rf = exact("wf", "backward", g, w, feat, idx_w)
    assert_close(dw, rw, dtype, "d_weights")
    assert_close(df, rf, dtype, "d_feat")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("case", ["shared-repeats", "model-repeats", "mixed-batch", "m40", "m16"])
def test_structured_tiles_with_irregularities(ops, case, dtype):
    """The lean scatter kernel works on tiles that the structured inverse build marks; tables that are
    structured except for a repeated token, a run named twice, or one batch element of random rows must
    come out the same as everything else: through the flagged entries and the general kernel."""
    b, h, n, m, c = 3, 2, 392, 48, 32
    if case == "m40":
        m = 40
    if case == "m16":
        m = 16
    regime = "shared" if case.startswith("shared") else "model"
    idx, q, k, v, attn, g_attn, g_feat = _attention_case(regime, b, h, n, m, c, dtype, 360)
    if case == "shared-repeats":
        idx[:, 64:128, 1] = idx[:, 64:128, 0]
    elif case == "model-repeats":
        idx[:, ::5, 8:16] = idx[:, ::5, 0:8]
    elif case == "mixed-batch":
        idx[1] = workloads.random_rows(1, n, n, m, 361)[0].to(DEV)
        idx[2] = workloads.make_index("shared", 1, n, m, 362)[0].to(DEV)
    dq, dk = ops.qk_backward(g_attn, q, k, idx)
    rq, rk = exact("qk", "backward", g_attn, q, k, idx)
    assert_close(dq, rq, dtype, "d_query")
    assert_close(dk, rk, dtype, "d_key")
    da, dv = ops.av_backward(g_feat, attn, v, idx)
    ra, rv = exact("av", "backward", g_feat, attn, v, idx)
    assert_close(da, ra, dtype, "d_attn")
    assert_close(dv, rv, dtype, "d_value")
    ops.clear_inverse_cache()
    again = ops.av_backward(g_feat, attn, v, idx)[1]
    assert torch.equal(dv, again), "the summation order is fixed: same bits on a rebuilt inverse"


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("regime", ["shared", "model", "random"])
def test_forward_reads_model_style_views_in_place(ops, regime, dtype):
    """query / key / value as the model hands them over (models/aff_transformer.py:117-119 of the reference:
    permuted views of the q and kv Linear outputs) are read where they are: same bits as on contiguous copies,
    and no copy is made (the strided entry points accept them)."""
    b, h, n, m, c = 2, 4, 200, 48, 32
    idx = workloads.make_index(regime, b, n, m, 370).to(DEV)
    g = torch.Generator(device=DEV).manual_seed(371)
    qlin = torch.randn(b, n, h * c, generator=g, device=DEV).to(dtype)
    kvlin = torch.randn(b, n, 2 * h * c, generator=g, device=DEV).to(dtype)
    q = qlin.reshape(b, n, h, c).permute(0, 2, 1, 3)
    kv = kvlin.view(b, n, h, 2, c).permute(3, 0, 2, 1, 4)
    key, v = kv[0], kv[1]
    assert not q.is_contiguous() and not key.is_contiguous() and not v.is_contiguous()
    attn = ops.qk_forward_views(q, key, idx)
    assert attn is not None, "the views qualify: rows contiguous, strides multiples of 16 bytes"
    assert torch.equal(attn, ops.qk_forward(q.contiguous(), key.contiguous(), idx))
    assert_close(attn, exact("qk", "forward", q, key, idx), dtype, "qk forward on views")
    probs = attn.float().softmax(-1).to(dtype)
    feat = ops.av_forward_views(probs, v, idx)
    assert feat is not None
    assert torch.equal(feat, ops.av_forward(probs, v.contiguous(), idx))
    assert_close(feat, exact("av", "forward", probs, v, idx), dtype, "av forward on a view")
    # views that do not qualify are declined (the autograd operators then copy, like the reference)
    assert ops.qk_forward_views(q[..., :16], key[..., :16], idx) is None
    odd = torch.randn(b, h, n, c + 1, device=DEV).to(dtype)[..., 1:]          # rows start off a 16-byte boundary
    assert ops.av_forward_views(probs, odd, idx) is None
    # and the autograd operators give the same results either way
    from clusten import CLUSTENAVFunction, CLUSTENQKFunction
    assert torch.equal(CLUSTENQKFunction.apply(q, key, idx), attn)
    assert torch.equal(CLUSTENAVFunction.apply(probs, v, idx), feat)
