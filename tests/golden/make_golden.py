#!/usr/bin/env python3
"""Record outputs of the reference's own CUDA extension as golden vectors.

Runs on a machine with a GPU and a built oracle/_ref/ (oracle/build_ref.py compiles the
reference's unmodified clusten/src there).  For each operator it draws seeded inputs,
calls the reference kernels the way clusten/clusten.py does, and stores inputs and
outputs (fp32) in tests/golden/ref_cuda_<op>.npz, or under --out.  The CPU test
tests/test_oracle.py::test_oracle_against_reference_cuda_outputs pins the oracle to them.

    python tests/golden/make_golden.py [--out DIR]
"""
import argparse
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "ml-autofocusformer_b200"))

import workloads  # noqa: E402
from oracle import ref_cuda  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    out_dir = ap.parse_args().out
    os.makedirs(out_dir, exist_ok=True)
    dev = "cuda"
    b, h, n, m, c = 2, 2, 136, 48, 32
    # batch element 0: clustered rows shared by the 8 tokens of a cluster; element 1: random rows with
    # repeats whose last three slots point at token 0 (the padded-stage pattern)
    idx = torch.cat([workloads.shared_cluster_rows(1, n, m, 1), workloads.random_rows(1, n, n, m, 3)], 0)
    idx[1, :, -3:] = 0
    q, k, v, attn, g_attn, g_feat = workloads.attention_operands(b, h, n, m, c, torch.float32, 4)
    cu = lambda *ts: [t.to(dev) for t in ts]
    cpu = lambda t: t.detach().cpu().numpy()

    qd, kd, idxd, gd = cu(q, k, idx, g_attn)
    a = ref_cuda.qk_forward(qd, kd, idxd)
    dq, dk = ref_cuda.qk_backward(gd, qd, kd, idxd)
    np.savez_compressed(os.path.join(out_dir, "ref_cuda_qk.npz"), op="qk", q=cpu(q), k=cpu(k), idx=cpu(idx),
                        g=cpu(g_attn), attn=cpu(a), dq=cpu(dq), dk=cpu(dk))

    ad, vd, gfd = cu(attn, v, g_feat)
    f = ref_cuda.av_forward(ad, vd, idxd)
    da, dv = ref_cuda.av_backward(gfd, ad, vd, idxd)
    np.savez_compressed(os.path.join(out_dir, "ref_cuda_av.npz"), op="av", attn=cpu(attn), v=cpu(v),
                        idx=cpu(idx), g=cpu(g_feat), feat=cpu(f), dattn=cpu(da), dv=cpu(dv))

    n_out, ic, cw = 40, 4, 24
    idx_w = workloads.select_rows(idx, n_out, 5)
    w, feat, g = workloads.merge_operands(b, n_out, n, m, ic, cw, torch.float32, 6)
    wd, fd, iwd, gwd = cu(w, feat, idx_w, g)
    o = ref_cuda.wf_forward(wd, fd, iwd)
    dw, df = ref_cuda.wf_backward(gwd, wd, fd, iwd)
    np.savez_compressed(os.path.join(out_dir, "ref_cuda_wf.npz"), op="wf", w=cpu(w), feat=cpu(feat),
                        idx=cpu(idx_w), g=cpu(g), out=cpu(o), dw=cpu(dw), dfeat=cpu(df))
    print("wrote golden vectors to", out_dir)


if __name__ == "__main__":
    main()
