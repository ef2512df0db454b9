"""The model-level harness without a GPU: the stand-ins behave as documented and the reference's
AutoFocusFormer (bytecode from oracle/build_ref.py) runs on the gather-formulation operators."""
import pytest
import torch

import aff_harness


def test_knn_standin_matches_brute_force():
    g = torch.Generator().manual_seed(0)
    q = torch.rand(3, 40, 2, generator=g) * 20
    d = torch.rand(3, 25, 2, generator=g) * 20
    idx, dist = aff_harness.knn(q, d, 6, return_dist=True, chunk_elems=40 * 25 * 2)   # forces two chunks
    full = ((q[:, :, None, :] - d[:, None, :, :]) ** 2).sum(-1).sqrt()
    want_dist, want_idx = full.sort(dim=2)
    assert torch.equal(idx, want_idx[:, :, :6])
    assert torch.allclose(dist, want_dist[:, :, :6])
    assert aff_harness.knn(q.half(), d.half(), 2).dtype == torch.int64


def test_drop_path_standin():
    dp = aff_harness.DropPath(0.5)
    x = torch.ones(4000, 3)
    assert torch.equal(dp.eval()(x), x)
    y = dp.train()(x)
    kept = (y[:, 0] != 0)
    assert torch.equal(y[kept], torch.full_like(y[kept], 2.0)) and 0.4 < kept.float().mean() < 0.6
    assert bool((y[~kept] == 0).all())


@pytest.mark.skipif(not aff_harness.available(), reason="oracle/_ref/aff_model is not built")
def test_reference_model_runs_on_the_formula_operators():
    aff_harness.use_implementation("formula", formula_chunk=1)
    model = aff_harness.build_model("tiny224", "cpu", seed=0)
    x = aff_harness.synthetic_images("tiny224", 2, "cpu", seed=1)
    y = aff_harness.forward(model, x)
    assert y.shape == (2, 1000) and torch.isfinite(y).all()
    # stage shapes of the configuration: 3136 / 784 / 196 / 49 tokens, m = 48, last stage global attention
    assert model.layers[0].nbhd_size == 48 and model.layers[3].nbhd_size == 49
    aff_harness.use_implementation("formula", formula_chunk=2)
    assert torch.equal(aff_harness.forward(model, x), y)
