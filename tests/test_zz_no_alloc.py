"""clusten_av_backward_noalloc: the AV backward for hosts that cannot allocate device memory at call
time (an engine's enqueue callback, a program that owns all device memory through its own pool).
It keeps the inverse neighbour index in an array inside the library instead of a caller buffer, so
it has to agree with the regular entry point, also on a second call that finds the array full of
the first call's data.  Collected last (file name) so that a run stopping at the first failure has
already run everything else."""
import ctypes

import pytest
import torch

import workloads
from helpers import assert_close, exact

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, d_feat, attn, v, idx):
    b, h, n, m = attn.shape
    c = v.shape[3]
    d_attn = torch.full_like(attn, float("nan"))
    d_v = torch.full_like(v, float("nan"))
    dtype = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[attn.dtype]
    status = lib.clusten_av_backward_noalloc(
        d_feat.data_ptr(), attn.data_ptr(), v.data_ptr(), idx.data_ptr(), d_attn.data_ptr(), d_v.data_ptr(),
        b, h, n, m, c, dtype, torch.cuda.current_stream().cuda_stream)
    return status, d_attn, d_v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_noalloc_matches_regular_entry_point_twice(lib, dtype):
    from clusten import ops
    dev = "cuda"
    # two different problems back to back: the second one starts from the first one's leftovers
    cases = [("shared", 4, 2, 392, 48, 11), ("random", 3, 4, 203, 48, 12)]
    for regime, b, h, n, m, seed in cases:
        idx = workloads.make_index(regime, b, n, m, seed).to(dev)
        if regime == "random":
            idx[:, :, -3:] = 0                      # repeated targets inside a row
        _, _, v, attn, _, g_feat = (t.to(dev) for t in workloads.attention_operands(b, h, n, m, 32, dtype, seed + 1))
        status, d_attn, d_v = _call_noalloc(lib, g_feat, attn, v, idx)
        assert status == 0, lib.clusten_status_string(status)
        ref_attn, ref_v = ops.av_backward(g_feat, attn, v, idx)
        assert_close(d_attn, ref_attn, dtype, f"d_attn ({regime})")
        assert_close(d_v, ref_v, dtype, f"d_value ({regime})")
        assert torch.equal(d_v, ref_v), "same kernels, same index: results must be bit-identical"
        want_attn, want_v = exact("av", "backward", g_feat, attn, v, idx)
        assert_close(d_attn, want_attn, dtype, f"d_attn vs the oracle ({regime})")
        assert_close(d_v, want_v, dtype, f"d_value vs the oracle ({regime})")


def test_noalloc_at_and_just_above_its_capacity(lib):
    """The largest stage-1 problem (n = 3136, m = 48) whose inverse index the built-in array holds, and one
    batch element more, which is refused.  A rejected call must leave its outputs untouched."""
    dev = "cuda"
    h, n, m = 2, 3136, 48
    capacity = 3407936 * 4                      # CLUSTEN_NOALLOC_MAX_INTS ints
    b = max(x for x in range(1, 64) if lib.clusten_inverse_bytes(x, n, m, n) <= capacity)
    assert lib.clusten_inverse_bytes(b + 1, n, m, n) > capacity
    idx = workloads.make_index("shared", b + 1, n, m, 21, dev)
    _, _, v, attn, _, g_feat = workloads.attention_operands(b + 1, h, n, m, 32, torch.float16, 22, dev)
    status, d_attn, d_v = _call_noalloc(lib, g_feat[:b].contiguous(), attn[:b].contiguous(), v[:b].contiguous(),
                                        idx[:b].contiguous())
    assert status == 0, lib.clusten_status_string(status)
    from clusten import ops
    ref_attn, ref_v = ops.av_backward(g_feat[:b].contiguous(), attn[:b].contiguous(), v[:b].contiguous(),
                                      idx[:b].contiguous())
    assert torch.equal(d_v, ref_v) and torch.equal(d_attn, ref_attn)
    status, d_attn, d_v = _call_noalloc(lib, g_feat, attn, v, idx)
    assert status == -8
    assert torch.isnan(d_attn).all() and torch.isnan(d_v).all()
    # a NULL output is refused before anything is launched
    st = lib.clusten_av_backward_noalloc(g_feat.data_ptr(), attn.data_ptr(), v.data_ptr(), idx.data_ptr(), None,
                                         d_v.data_ptr(), 2, h, n, m, 32, 1, torch.cuda.current_stream().cuda_stream)
    assert st == -3


def test_noalloc_rejects_sizes_beyond_its_array(lib):
    p = ctypes.c_void_p(256)        # never dereferenced: the size check comes first
    big = lib.clusten_av_backward_noalloc(p, p, p, p, p, p, 128, 2, 3136, 48, 32, 0, None)
    assert big == -8
    assert b"CLUSTEN_NOALLOC_MAX_INTS" in lib.clusten_status_string(big)
