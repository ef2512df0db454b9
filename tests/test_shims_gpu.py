"""The reference's own clusten/clusten.py (bytecode from oracle/build_ref.py), unchanged, on top of the three
shim modules that carry the names of its extension modules: forward and backward of the three operators
match this package's autograd operators bit for bit (same kernels underneath)."""
import importlib.machinery
import importlib.util
import os
import sys

import pytest
import torch

import workloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BYTECODE = os.path.join(ROOT, "oracle", "_ref", "ref_clusten", "clusten", "clusten.bytecode")
SHIMS = os.path.join(ROOT, "ml-autofocusformer_b200", "shims")

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(BYTECODE), reason="oracle/_ref is not built")]
DEV = "cuda"


@pytest.fixture(scope="module")
def reference_wrappers(lib):
    saved = {k: sys.modules.pop(k, None) for k in ("clustenqk_cuda", "clustenav_cuda", "clustenwf_cuda")}
    sys.path.insert(0, SHIMS)
    try:
        loader = importlib.machinery.SourcelessFileLoader("reference_clusten_on_shims", BYTECODE)
        spec = importlib.util.spec_from_loader("reference_clusten_on_shims", loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        for name in ("clustenqk_cuda", "clustenav_cuda", "clustenwf_cuda"):
            assert sys.modules[name].__file__.startswith(SHIMS)
        yield mod
    finally:
        sys.path.remove(SHIMS)
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v


def test_reference_wrappers_run_on_the_shims(reference_wrappers):
    import clusten
    b, h, n, m, c = 2, 4, 200, 48, 32
    idx = workloads.model_like_rows(b, n, m, 5).to(DEV)
    q, k, v, attn, g_attn, g_feat = (t.to(DEV) for t in workloads.attention_operands(b, h, n, m, c, torch.float32, 6))

    def run(qk_fn, av_fn):
        q_, k_, v_ = (t.clone().requires_grad_(True) for t in (q, k, v))
        a = qk_fn(q_, k_, idx)
        f = av_fn(a.softmax(-1), v_, idx)
        f.backward(g_feat)
        return a.detach(), f.detach(), q_.grad, k_.grad, v_.grad

    got = run(reference_wrappers.CLUSTENQKFunction.apply, reference_wrappers.CLUSTENAVFunction.apply)
    want = run(clusten.CLUSTENQKFunction.apply, clusten.CLUSTENAVFunction.apply)
    for g_, w_ in zip(got, want):
        assert torch.equal(g_, w_)

    n_out, ic, cw = 50, 4, 64
    idx_w = workloads.select_rows(idx, n_out, 7)
    w, f, g = (t.to(DEV) for t in workloads.merge_operands(b, n_out, n, m, ic, cw, torch.float32, 8))

    def run_wf(fn):
        w_, f_ = w.clone().requires_grad_(True), f.clone().requires_grad_(True)
        o = fn(w_, f_, idx_w)
        o.backward(g)
        return o.detach(), w_.grad, f_.grad

    for g_, w_ in zip(run_wf(reference_wrappers.CLUSTENWFFunction.apply), run_wf(clusten.CLUSTENWFFunction.apply)):
        assert torch.equal(g_, w_)
