"""Model-level parity on the GPU: the reference's AutoFocusFormer (unmodified, bytecode in
oracle/_ref/aff_model) gives the same logits on this package's operators as on the PyTorch gather
formulation -- and, where the reference's own CUDA extension is built, as on the reference's kernels --
with the same weights, images and neighbourhood stand-ins.  Tolerances (max |x - ref| / max |ref| over the
logits, accumulated over all blocks): fp32 1e-4, bf16 autocast 5e-2."""
import pytest
import torch

import aff_harness

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not aff_harness.available(), reason="oracle/_ref/aff_model is not built")]

DEV = "cuda"


def _rel(x, ref):
    return ((x.double() - ref.double()).abs().max() / ref.double().abs().max()).item()


@pytest.mark.parametrize("config,batch,dtype,tol", [
    ("tiny224", 6, torch.float32, 1e-4),
    ("tiny224", 6, torch.bfloat16, 5e-2),
    ("base384", 2, torch.float32, 1e-4),
    ("base384", 2, torch.bfloat16, 5e-2),
], ids=["tiny224-fp32", "tiny224-bf16", "base384-fp32", "base384-bf16"])
def test_logits_match_the_formula_operators(lib, config, batch, dtype, tol, capsys):
    from clusten import _lib
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    aff_harness.use_implementation("b200")
    model = aff_harness.build_model(config, DEV, seed=0)
    x = aff_harness.synthetic_images(config, batch, DEV, seed=1)
    before = _lib.launch_count()
    got = aff_harness.forward(model, x, dtype)
    launched = _lib.launch_count() - before
    depths = aff_harness.CONFIGS[config]["depths"]
    # every block of a local-attention stage calls QK and AV once, every merge calls WF once
    assert launched >= 2 * sum(depths[:3]) + 3, launched
    aff_harness.use_implementation("formula", formula_chunk=1)
    want = aff_harness.forward(model, x, dtype)
    err = _rel(got, want)
    agree = (got.argmax(1) == want.argmax(1)).float().mean().item()
    with capsys.disabled():
        print(f"\n{config} {dtype}: logits rel err {err:.2e}, top-1 agreement {agree:.2f}, "
              f"{launched} library kernel launches")
    assert got.shape == (batch, 1000) and torch.isfinite(got.float()).all()
    assert err <= tol, err
    aff_harness.use_implementation("b200")


def test_logits_match_the_reference_kernels(lib, capsys):
    if not aff_harness.reference_kernels_available():
        pytest.skip("the reference's CUDA extension (oracle/_ref) is not built")
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    aff_harness.use_implementation("b200")
    model = aff_harness.build_model("tiny224", DEV, seed=3)
    x = aff_harness.synthetic_images("tiny224", 4, DEV, seed=4)
    got = aff_harness.forward(model, x)
    aff_harness.use_implementation("reference")
    want = aff_harness.forward(model, x)
    aff_harness.use_implementation("b200")
    err = _rel(got, want)
    with capsys.disabled():
        print(f"\ntiny224 fp32 vs the reference's kernels: logits rel err {err:.2e}")
    assert err <= 1e-4, err


@pytest.mark.parametrize("config,batch,dtype,tol", [("tiny224", 4, torch.float32, 1e-4), ("base384", 2, torch.bfloat16, 5e-2)],
                         ids=["tiny224-fp32", "base384-bf16"])
def test_fused_attention_variant_of_the_model(lib, config, batch, dtype, tol, capsys):
    """ClusterAttention routed through the fused local-attention kernel (an opt-in that replaces one method of
    the reference's model): same logits as the unmodified model on the gather formulation."""
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    aff_harness.use_implementation("b200")
    model = aff_harness.build_model(config, DEV, seed=0)
    x = aff_harness.synthetic_images(config, batch, DEV, seed=1)
    try:
        aff_harness.use_fused_attention(True)
        got = aff_harness.forward(model, x, dtype)
    finally:
        aff_harness.use_fused_attention(False)
    aff_harness.use_implementation("formula", formula_chunk=1)
    want = aff_harness.forward(model, x, dtype)
    aff_harness.use_implementation("b200")
    err = _rel(got, want)
    with capsys.disabled():
        print(f"\n{config} {dtype} fused attention: logits rel err {err:.2e}")
    assert err <= tol, err


@pytest.mark.parametrize("config,batch,dtype", [("tiny224", 4, torch.float32), ("base384", 2, torch.bfloat16)],
                         ids=["tiny224-fp32", "base384-bf16"])
def test_neighbourhood_tables_variant_of_the_model(lib, config, batch, dtype, capsys):
    """BasicLayer building its neighbourhood tables with clusten_nbhd_build (an opt-in that replaces one method
    of the reference's model): the tables are integer work, so the blocks see the very same inputs; the logits
    may differ only by what the feature reordering's different torch kernel rounds (nothing: it copies)."""
    aff_harness.use_implementation("b200")
    model = aff_harness.build_model(config, DEV, seed=0)
    x = aff_harness.synthetic_images(config, batch, DEV, seed=1)
    want = aff_harness.forward(model, x, dtype)
    try:
        aff_harness.use_fused_neighbourhood(True)
        got = aff_harness.forward(model, x, dtype)
        aff_harness.use_fused_merging(True)
        both = aff_harness.forward(model, x, dtype)
    finally:
        aff_harness.use_fused_neighbourhood(False)
        aff_harness.use_fused_merging(False)
    err, err2 = _rel(got, want), _rel(both, want)
    with capsys.disabled():
        print(f"\n{config} {dtype} neighbourhood tables from one kernel: logits rel err {err:.2e}; "
              f"merge weights too: {err2:.2e}")
    assert err <= 1e-6, err
    # the merge weights are rounded once where the reference's products round after every step (bf16 only)
    assert err2 <= (1e-6 if dtype == torch.float32 else 2e-2), err2


def test_all_hooks_without_reserved_tokens(lib, capsys):
    """reserve_on=False takes the other branch of the merge-centre selection (models/aff_transformer.py:312-326);
    all three opt-in hooks together against the unmodified model."""
    aff_harness.use_implementation("b200")
    model = aff_harness.build_model("tiny224", DEV, seed=0, reserve_on=False)
    x = aff_harness.synthetic_images("tiny224", 3, DEV, seed=2)
    want = aff_harness.forward(model, x, torch.float32)
    try:
        aff_harness.use_fused(True)
        got = aff_harness.forward(model, x, torch.float32)
    finally:
        aff_harness.use_fused(False)
    err = _rel(got, want)
    with capsys.disabled():
        print(f"\ntiny224 fp32, reserve_on=False, all hooks: logits rel err {err:.2e}")
    assert err <= 1e-4, err
