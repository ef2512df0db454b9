#!/usr/bin/env python3
"""Benchmark of the CLUSTEN operators on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype fp32|bf16] [--impl b200|reference]
    python bench.py --ops            # per-operator table (fp32 and bf16, three index regimes)
    python bench.py --workload config2   # per-stage chain QK -> +bias -> softmax -> AV, WF between stages (b=256, bf16)
    python bench.py --no-model       # leave out the model-level (images/sec) legs

A step is one pass of the hot path over one batch of synthetic input at the stage-1 shapes
of AutoFocusFormer (224^2 image, batch 128 per GPU): CLUSTENAV forward + backward on
attn [128,2,3136,48] / v [128,2,3136,32], and CLUSTENWF forward + backward on weights
[128,784,48,4] / feat [128,3136,64], with clustered neighbour tables (8 tokens of a cluster
share one row of their 48 nearest tokens) and N(0,1) upstream gradients.  The inverse
neighbour index used by the backward kernels is rebuilt in every step.

The metric is GB/s of algorithmic bytes (each input read once, each output written once,
int64 indices, nothing for workspaces) summed over the step; one JSON line is printed by
rank 0.  With N > 1 every rank runs its own batch (weak scaling, no collective on the data
path) and the time is the maximum over ranks.

Beside the step the line carries sub-records: `bf16` (the same step in bf16), `config0` (QK forward
[2,2,3136,32], m=48: the PyTorch formulation on the host cores next to the kernel), `config2` (the
per-stage chain at batch 256 in bf16) and `model` (forward images/sec of the reference's
AutoFocusFormer, unmodified, on these operators: Tiny-like 224^2 at batch 256 in fp32 and bf16
autocast, Base-like 384^2 at batch 64 in bf16 autocast; 50 warm-up + 30 timed forwards as in
main.py:343-354 of the reference; summed over the ranks).

--impl reference times the pure-PyTorch gather formulation of the reference's kernel tests on
the host CPU cores (the reference ships no CPU implementation of these operators) on a
bounded slice of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "ml-autofocusformer_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

if "reference" in sys.argv:
    # torchrun pins OMP_NUM_THREADS=1; the CPU arm is meant to use every host core it may run on
    try:
        _cores = len(os.sched_getaffinity(0))
    except AttributeError:
        _cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(_cores)
    os.environ["MKL_NUM_THREADS"] = str(_cores)

import torch  # noqa: E402

import workloads  # noqa: E402

# stage-1 shapes of the benchmark configuration
CFG = dict(b=128, h=2, n=3136, m=48, c=32, n_out=784, cw=64, ic=4)
CPU_SAMPLE_BATCH = 4
# dram__bytes_read.sum + dram__bytes_write.sum of one launch from an ncu capture at b=32, scaled x4 to the
# benchmark's b=128 (traffic grows with the batch); see profiles/.  NCU_CAPTURE_BUILD names the commit whose
# kernels were captured: the figure describes that build, not necessarily the one being timed.
NCU_CAPTURE_BUILD = "c73042a"
NCU_DRAM_BYTES_PER_LAUNCH = {("av_d_value", "fp32"): 4 * (84390144 + 9697024),
                             ("av_forward", "fp32"): 4 * (103208448 + 11935744),
                             ("av_d_attn", "fp32"): 4 * (89984256 + 16303872),
                             ("wf_forward", "fp32"): 4 * (54714368 + 3070464),
                             ("wf_d_weights", "fp32"): 4 * (61138688 + 3995136),
                             ("wf_d_feat", "fp32"): 4 * (50619904 + 4648704)}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def step_bytes(cfg, esize):
    b, h, n, m, c = cfg["b"], cfg["h"], cfg["n"], cfg["m"], cfg["c"]
    av = dict(b=b, h=h, n=n, m=m, c=c, s=esize)
    wf = dict(b=b, n=n, m=m, c=cfg["cw"], s=esize, n_out=cfg["n_out"], ic=cfg["ic"])
    return {
        "av_fwd": workloads.algorithmic_bytes("av", "fwd", **av),
        "av_bwd": workloads.algorithmic_bytes("av", "bwd", **av),
        "wf_fwd": workloads.algorithmic_bytes("wf", "fwd", **wf),
        "wf_bwd": workloads.algorithmic_bytes("wf", "bwd", **wf),
    }


def kernel_bytes(cfg, esize):
    """Algorithmic bytes of each kernel launched in a step: what that launch must read and write."""
    b, h, n, m, c = cfg["b"], cfg["h"], cfg["n"], cfg["m"], cfg["c"]
    n_out, cw, ic = cfg["n_out"], cfg["cw"], cfg["ic"]
    s = esize
    bhnc, bhnm, idx = b * h * n * c * s, b * h * n * m * s, b * n * m * 8
    w, f, o, iw = b * n_out * m * ic * s, b * n * cw * s, b * n_out * ic * cw * s, b * n_out * m * 8
    return {
        "av_forward": bhnm + 2 * bhnc + idx,          # attn, v, idx -> feat
        "av_d_attn": 2 * bhnc + idx + bhnm,           # d_feat, v, idx -> d_attn
        "av_d_value": bhnm + 2 * bhnc,                # attn, d_feat -> d_value (via the inverse index)
        "wf_forward": w + f + iw + o,
        "wf_d_weights": f + o + iw + w,
        "wf_d_feat": w + o + f,
        "inverse_build": idx + iw,                    # both neighbour tables, once each
        "wf_order": b * n_out * (8 + 4),              # first neighbour of every row -> permutation
    }


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                smax = float(r[1])
            except ValueError:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "samples": len(sm), "reasons": sorted(reasons)}


def _physical_gpu(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v.strip() for v in vis.split(",") if v.strip()]
        if local_rank < len(ids):
            return ids[local_rank]
    return str(local_rank)


# --------------------------------------------------------------------------- workload
def make_workload(cfg, dtype, device, seed):
    b, h, n, m, c = cfg["b"], cfg["h"], cfg["n"], cfg["m"], cfg["c"]
    idx = workloads.shared_cluster_rows(b, n, m, seed, device)
    _, _, v, attn, _, g_feat = workloads.attention_operands(b, h, n, m, c, dtype, seed + 1, device)
    idx_w = workloads.select_rows(idx, cfg["n_out"], seed + 2)
    w, feat, g_new = workloads.merge_operands(b, cfg["n_out"], n, m, cfg["ic"], cfg["cw"], dtype, seed + 3, device)
    return dict(idx=idx, v=v, attn=attn, g_feat=g_feat, idx_w=idx_w, w=w, feat=feat, g_new=g_new)


def device_step(ops, wl, cached=None):
    """The hot path through the C ABI, operands resident in HBM.  cached = (inverse of the attention table,
    inverse of the merge table, row order) built beforehand: the step a model runs for every block of a stage
    but the first, whose index tensors it has seen already."""
    n = wl["v"].shape[2]
    feat = ops.av_forward(wl["attn"], wl["v"], wl["idx"])
    inv = cached[0] if cached else ops.build_inverse(wl["idx"], n)
    d_attn, d_v = ops.av_backward(wl["g_feat"], wl["attn"], wl["v"], wl["idx"], inv)
    order = cached[2] if cached else ops.build_row_order(wl["idx_w"])
    if order is None:
        order = False
    out = ops.wf_forward(wl["w"], wl["feat"], wl["idx_w"], order)
    inv_w = cached[1] if cached else ops.build_inverse(wl["idx_w"], n)
    d_w, d_f = ops.wf_backward(wl["g_new"], wl["w"], wl["feat"], wl["idx_w"], inv_w, order)
    return feat, d_attn, d_v, out, d_w, d_f


class EndToEnd:
    """The same step through the autograd operators with HOST buffers: every step copies its pinned
    inputs to the device, runs the operators forward and backward and copies all six results back to
    pinned host memory.  Copies run on their own streams (inputs of the merge operator travel while the
    attention operator computes, results travel while the next step's inputs arrive; device buffers are
    double-buffered), the timed region ends when the last result of the last step is on the host."""

    def __init__(self, wl):
        self.host = {k: v.cpu().pin_memory() for k, v in wl.items()}
        self.dev = [{k: torch.empty_like(v) for k, v in wl.items()} for _ in range(2)]
        self.out_host = None
        self.h2d = sum(v.numel() * v.element_size() for v in self.host.values())
        self.d2h = 0
        self.s_in = torch.cuda.Stream()
        self.s_out = torch.cuda.Stream()
        self.step_no = 0
        self.done = [None, None]          # compute-done event per device buffer set

    def step(self):
        from clusten import CLUSTENAVFunction, CLUSTENWFFunction, clear_inverse_cache
        main = torch.cuda.current_stream()
        slot = self.step_no & 1
        self.step_no += 1
        d = self.dev[slot]
        av_keys, wf_keys = ("idx", "v", "attn", "g_feat"), ("idx_w", "w", "feat", "g_new")
        with torch.cuda.stream(self.s_in):
            if self.done[slot] is not None:
                self.s_in.wait_event(self.done[slot])      # the kernels that read this buffer set are finished
            for k in av_keys:
                d[k].copy_(self.host[k], non_blocking=True)
            ev_av = torch.cuda.Event()
            ev_av.record(self.s_in)
            for k in wf_keys:
                d[k].copy_(self.host[k], non_blocking=True)
            ev_wf = torch.cuda.Event()
            ev_wf.record(self.s_in)
        clear_inverse_cache()
        main.wait_event(ev_av)
        attn = d["attn"].detach().requires_grad_(True)
        v = d["v"].detach().requires_grad_(True)
        feat = CLUSTENAVFunction.apply(attn, v, d["idx"])
        feat.backward(d["g_feat"])
        res_av = [feat.detach(), attn.grad, v.grad]
        ev_av_done = torch.cuda.Event()
        ev_av_done.record(main)
        main.wait_event(ev_wf)
        w = d["w"].detach().requires_grad_(True)
        f = d["feat"].detach().requires_grad_(True)
        out = CLUSTENWFFunction.apply(w, f, d["idx_w"])
        out.backward(d["g_new"])
        res_wf = [out.detach(), w.grad, f.grad]
        ev_done = torch.cuda.Event()
        ev_done.record(main)
        self.done[slot] = ev_done
        results = res_av + res_wf
        if self.out_host is None:
            self.out_host = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True) for r in results]
            self.d2h = sum(r.numel() * r.element_size() for r in results)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(ev_av_done)
            for hbuf, r in zip(self.out_host[:3], res_av):
                hbuf.copy_(r, non_blocking=True)
                r.record_stream(self.s_out)
            self.s_out.wait_event(ev_done)
            for hbuf, r in zip(self.out_host[3:], res_wf):
                hbuf.copy_(r, non_blocking=True)
                r.record_stream(self.s_out)

    def finish(self):
        """Make the current stream wait for all copies (call before the closing timing event)."""
        torch.cuda.current_stream().wait_stream(self.s_out)
        torch.cuda.current_stream().wait_stream(self.s_in)


# --------------------------------------------------------------------------- CPU baseline
def cpu_formula_step(sample):
    from oracle import formula
    formula.forward_backward("av", sample["attn"], sample["v"], sample["idx"], sample["g_feat"], chunk=1)
    formula.forward_backward("wf", sample["w"], sample["feat"], sample["idx_w"], sample["g_new"], chunk=1)


def cpu_sample(cfg, dtype, seed):
    small = dict(cfg, b=CPU_SAMPLE_BATCH)
    return small, make_workload(small, dtype, "cpu", seed)


def time_cpu(cfg, dtype, steps, warmup):
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    torch.set_num_threads(cores)
    small, sample = cpu_sample(cfg, dtype, 0)
    for _ in range(warmup):
        cpu_formula_step(sample)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_formula_step(sample)
    dt = (time.perf_counter() - t0) / steps
    nbytes = sum(step_bytes(small, 4 if dtype == torch.float32 else 2).values())
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "ms_per_step": dt * 1e3,
            "sample": f"{CPU_SAMPLE_BATCH} of {cfg['b']} batch elements, AV+WF forward+backward, "
                      f"PyTorch gather formulation (oracle/formula.py), {steps} repeats"}


def time_cpu_full_batch(cfg, dtype):
    """One repeat of the whole batch on the host cores, in chunks of CPU_SAMPLE_BATCH with the chunk times
    summed (the gathered [b,h,n,m,c] tensor of the formulation does not fit otherwise)."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    chunks = -(-cfg["b"] // CPU_SAMPLE_BATCH)
    total = 0.0
    for ci in range(chunks):
        small, sample = cpu_sample(cfg, dtype, 100 + ci)
        t0 = time.perf_counter()
        cpu_formula_step(sample)
        total += time.perf_counter() - t0
    nbytes = sum(step_bytes(cfg, 4 if dtype == torch.float32 else 2).values())
    return {"value": nbytes / total / 1e9, "unit": "GB/s", "s_per_step": total, "cores": cores,
            "sample": f"all {cfg['b']} batch elements once, {chunks} chunks of {CPU_SAMPLE_BATCH}, chunk times summed"}


# --------------------------------------------------------------------------- reference CUDA extension (speed bar)
def time_reference_cuda(wl, reps=5):
    from oracle import ref_cuda
    if wl is None or not ref_cuda.available() or wl["attn"].dtype != torch.float32:
        return None

    def run():
        ref_cuda.av_forward(wl["attn"], wl["v"], wl["idx"])
        ref_cuda.av_backward(wl["g_feat"], wl["attn"], wl["v"], wl["idx"])
        ref_cuda.wf_forward(wl["w"], wl["feat"], wl["idx_w"])
        ref_cuda.wf_backward(wl["g_new"], wl["w"], wl["feat"], wl["idx_w"])

    run()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for _ in range(reps):
        run()
    ev[1].record()
    torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[1]) / reps


# --------------------------------------------------------------------------- per-operator table
def _time(fn, reps=15, warmup=3):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(reps):
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b_.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b_))
    return statistics.median(times)


def per_operator_table():
    """Median time, algorithmic GB/s and fraction of the HBM peak of every operator and direction at
    the stage-1 shapes, fp32 and bf16, for the three index regimes; the reference's own CUDA
    extension (fp32) and the inverse-index build beside them.  One JSON line per row."""
    from clusten import ops
    from oracle import ref_cuda
    peak, kind = _peaks()
    cfg = dict(CFG)
    b, h, n, m, c = cfg["b"], cfg["h"], cfg["n"], cfg["m"], cfg["c"]
    dev = torch.device("cuda", 0)
    have_ref = ref_cuda.available()
    for regime in ("shared", "model", "random"):
        idx = workloads.make_index(regime, b, n, m, 7, dev)
        idx_w = workloads.select_rows(idx, cfg["n_out"], 8)
        for dtype in (torch.float32, torch.bfloat16):
            s = 4 if dtype == torch.float32 else 2
            q, k, v, attn, g_attn, g_feat = workloads.attention_operands(b, h, n, m, c, dtype, 9, dev)
            inv = ops.build_inverse(idx, n)
            inv_w = ops.build_inverse(idx_w, n)
            rows = [
                ("qk_fwd", lambda: ops.qk_forward(q, k, idx), ("qk", "fwd", {}),
                 lambda: ref_cuda.qk_forward(q, k, idx)),
                ("qk_bwd", lambda: ops.qk_backward(g_attn, q, k, idx, inv), ("qk", "bwd", {}),
                 lambda: ref_cuda.qk_backward(g_attn, q, k, idx)),
                ("av_fwd", lambda: ops.av_forward(attn, v, idx), ("av", "fwd", {}),
                 lambda: ref_cuda.av_forward(attn, v, idx)),
                ("av_bwd", lambda: ops.av_backward(g_feat, attn, v, idx, inv), ("av", "bwd", {}),
                 lambda: ref_cuda.av_backward(g_feat, attn, v, idx)),
            ]
            for ic in (1, 4):
                w, feat, g_new = workloads.merge_operands(b, cfg["n_out"], n, m, ic, cfg["cw"], dtype, 10, dev)
                kw = dict(n_out=cfg["n_out"], ic=ic)
                rows.append((f"wf_fwd_ic{ic}", (lambda w=w, feat=feat: ops.wf_forward(w, feat, idx_w)),
                             ("wf", "fwd", kw), (lambda w=w, feat=feat: ref_cuda.wf_forward(w, feat, idx_w))))
                rows.append((f"wf_bwd_ic{ic}",
                             (lambda w=w, feat=feat, g_new=g_new: ops.wf_backward(g_new, w, feat, idx_w, inv_w)),
                             ("wf", "bwd", kw),
                             (lambda w=w, feat=feat, g_new=g_new: ref_cuda.wf_backward(g_new, w, feat, idx_w))))
            for name, fn, (op, direction, kw), ref_fn in rows:
                cc = cfg["cw"] if op == "wf" else c
                nbytes = workloads.algorithmic_bytes(op, direction, b=b, h=h, n=n, m=m, c=cc, s=s, **kw)
                ms = _time(fn)
                row = {"op": name, "regime": regime, "dtype": str(dtype).split(".")[-1], "ms": round(ms, 4),
                       "GBps": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / peak, 3),
                       "MB": round(nbytes / 1e6, 1)}
                if have_ref and dtype == torch.float32:
                    row["reference_ext_ms"] = round(_time(ref_fn, reps=5, warmup=1), 4)
                print(json.dumps(row), flush=True)
            if dtype == torch.float32:
                for name, ix in (("inverse_build_attn", idx), ("inverse_build_wf", idx_w)):
                    ms = _time(lambda ix=ix: ops.build_inverse(ix, n))
                    nb = ix.numel() * 8
                    print(json.dumps({"op": name, "regime": regime, "ms": round(ms, 4),
                                      "GBps": round(nb / ms / 1e6, 1), "MB": round(nb / 1e6, 1),
                                      "peak": f"{peak} GB/s {kind}"}), flush=True)


# --------------------------------------------------------------------------- main arms
def run_reference_arm(args, dtype, rank):
    if rank != 0:
        return
    cfg = dict(CFG)
    res = time_cpu(cfg, dtype, max(1, args.steps), max(0, args.warmup))
    line = {
        "impl": "reference", "metric": "clusten_av_wf_fwd_bwd_algorithmic_bandwidth", "value": res["value"],
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if dtype == torch.float32 else "bf16", "data": "synthetic",
        "config": {"workload": "config1: CLUSTENAV + CLUSTENWF forward+backward, stage-1 shapes "
                               f"(sample of {CPU_SAMPLE_BATCH} batch elements per step)", **cfg},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- sub-records
def time_step_series(ops, wl, steps, reps, barrier, reduce_max, cached=None):
    """`reps` back-to-back repetitions of a timed loop of exactly `steps` device steps, each bracketed by a
    barrier + synchronize; per repetition the time is the maximum over the ranks.  -> ms per step, per rep."""
    series = []
    for _ in range(reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            device_step(ops, wl, cached)
        stop.record()
        barrier()
        series.append(reduce_max(start.elapsed_time(stop) / steps))
    return series


def config0_record(device):
    """BASELINE config 0: CLUSTENQK forward, fp32, q,k [2,2,3136,32], nbhd_idx [2,3136,48] (clustered,
    shared rows).  The PyTorch gather formulation on the host cores next to the kernel on the GPU, and
    their agreement."""
    from clusten import ops
    from oracle import formula
    b, h, n, m, c = 2, 2, 3136, 48, 32
    idx = workloads.shared_cluster_rows(b, n, m, 0)
    q, k, _, _, _, _ = workloads.attention_operands(b, h, n, m, c, torch.float32, 1)
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    formula.qk(q, k, idx)
    times = []
    for _ in range(5):
        t0 = time.perf_counter()
        ref = formula.qk(q, k, idx)
        times.append(time.perf_counter() - t0)
    cpu_ms = statistics.median(times) * 1e3
    qd, kd, idxd = q.to(device), k.to(device), idx.to(device)
    gpu_ms = _time(lambda: ops.qk_forward(qd, kd, idxd), reps=30, warmup=5)
    out = ops.qk_forward(qd, kd, idxd).cpu()
    err = ((out.double() - ref.double()).abs().max() / ref.double().abs().max()).item()
    nbytes = workloads.algorithmic_bytes("qk", "fwd", b=b, h=h, n=n, m=m, c=c, s=4)
    return {"workload": "config0: CLUSTENQK forward fp32 [2,2,3136,32], m=48", "MB": round(nbytes / 1e6, 2),
            "cpu_formula_ms": round(cpu_ms, 3), "cpu_cores": cores, "cpu_GBps": round(nbytes / cpu_ms / 1e6, 2),
            "gpu_ms": round(gpu_ms, 4), "gpu_GBps": round(nbytes / gpu_ms / 1e6, 1),
            "note": "8 MB: fits in L2, launch-latency bound on the GPU", "rel_err_vs_cpu_formula": err}


CONFIG2_STAGES = [  # tokens, heads, channels, neighbours
    dict(n=3136, h=2, C=64, m=48), dict(n=784, h=4, C=128, m=48),
    dict(n=196, h=8, C=256, m=48), dict(n=49, h=16, C=512, m=49)]


def config2_records(device, batch=256, dtype=torch.bfloat16, reps=12):
    """BASELINE config 2: per stage the chain QK -> + position bias -> softmax -> AV (the local-attention
    operators as models/aff_transformer.py:117-155 of the reference strings them together; bias add and
    softmax are torch kernels) and the WF merge to the next stage (:361), batch 256, bf16, clustered shared
    rows; stage 4 has m = 49 = every token.  Stages whose operands fit in L2 rotate over several buffer
    sets.  -> one record per stage."""
    from clusten import ops
    peak, _ = _peaks()
    out = []
    s = 2
    for si, st in enumerate(CONFIG2_STAGES):
        n, h, m, C = st["n"], st["h"], st["m"], st["C"]
        per_set = batch * (3 * h * n * 32 * s + 2 * h * n * m * s + n * m * 8)
        sets = max(1, min(8, -(-4 * 126_000_000 // per_set))) if per_set < 4 * 126_000_000 else 1
        bufs = []
        for k_ in range(sets):
            idx = workloads.shared_cluster_rows(batch, n, m, 40 + 10 * si + k_, device)
            q, k, v, _, _, _ = workloads.attention_operands(batch, h, n, m, 32, dtype, 41 + 10 * si + k_, device)
            bias = torch.randn(batch, h, n, m, device=device, dtype=dtype)
            bufs.append((idx, q, k, v, bias))
        rec = {"stage": si + 1, "tokens": n, "heads": h, "m": m, "buffer_sets": sets}
        timers = {}

        def timed(name, fn, i):
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            r = fn()
            b_.record()
            timers.setdefault(name, []).append((a, b_))
            return r

        def chain(i):
            idx, q, k, v, bias = bufs[i % sets]
            attn = timed("qk_ms", lambda: ops.qk_forward(q, k, idx), i)
            attn = timed("bias_softmax_ms", lambda: torch.softmax(attn + bias, -1), i)
            return timed("av_ms", lambda: ops.av_forward(attn, v, idx), i)

        for i in range(3):
            chain(i)
        timers.clear()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        for i in range(reps):
            chain(i)
        t1.record()
        torch.cuda.synchronize()
        rec["chain_ms"] = round(t0.elapsed_time(t1) / reps, 4)
        if m <= 48:
            # the same chain in the fused kernel (scores + bias + softmax + output, attn never written)
            def fused(i):
                idx, q, k, v, bias = bufs[i % sets]
                return ops.local_attention_forward(q, k, v, idx, pos_bias=bias)
            for i in range(3):
                fused(i)
            torch.cuda.synchronize()
            t0.record()
            for i in range(reps):
                fused(i)
            t1.record()
            torch.cuda.synchronize()
            rec["fused_chain_ms"] = round(t0.elapsed_time(t1) / reps, 4)
            chain_bytes = batch * (3 * h * n * 32 * s + h * n * m * s + n * m * 8 + h * n * 32 * s)
            rec["fused_chain_MB"] = round(chain_bytes / 1e6, 1)
            rec["fused_frac_of_hbm_peak"] = round(chain_bytes / rec["fused_chain_ms"] / 1e6 / peak, 3)
        for name, evs in timers.items():
            rec[name] = round(statistics.median(a.elapsed_time(b_) for a, b_ in evs), 4)
        ab = workloads.algorithmic_bytes("qk", "fwd", b=batch, h=h, n=n, m=m, c=32, s=s)
        rec["qk_av_MB"] = round(ab / 1e6, 1)
        rec["qk_frac_of_hbm_peak"] = round(ab / rec["qk_ms"] / 1e6 / peak, 3)
        rec["av_frac_of_hbm_peak"] = round(ab / rec["av_ms"] / 1e6 / peak, 3)
        del bufs
        if si < 3:
            n_out, ic = CONFIG2_STAGES[si + 1]["n"], 4
            wsets = []
            for k_ in range(sets):
                idx = workloads.shared_cluster_rows(batch, n, 48, 45 + 10 * si + k_, device)
                idx_w = workloads.select_rows(idx, n_out, 46 + 10 * si + k_)
                w, feat, _ = workloads.merge_operands(batch, n_out, n, 48, ic, C, dtype, 47 + 10 * si + k_, device)
                wsets.append((w, feat, idx_w))
            del idx
            for i in range(3):
                ops.wf_forward(*wsets[i % sets])
            torch.cuda.synchronize()
            t0.record()
            for i in range(reps):
                ops.wf_forward(*wsets[i % sets])
            t1.record()
            torch.cuda.synchronize()
            wf_ms = t0.elapsed_time(t1) / reps
            wb = workloads.algorithmic_bytes("wf", "fwd", b=batch, n=n, m=48, c=C, s=s, n_out=n_out, ic=ic)
            rec.update({"wf_ms": round(wf_ms, 4), "wf_MB": round(wb / 1e6, 1),
                        "wf_frac_of_hbm_peak": round(wb / wf_ms / 1e6 / peak, 3),
                        "wf_note": "row order built once per index tensor (cached), as the operator does"})
            del wsets
        torch.cuda.empty_cache()
        out.append(rec)
    return out


MODEL_LEGS = [("tiny224", 256, "fp32"), ("tiny224", 256, "bf16"), ("base384", 64, "bf16")]


def model_records(device, world, barrier, reduce_max, warmup=50, steps=30, legs=MODEL_LEGS, with_reference=True):
    """Forward images/sec of the reference's AutoFocusFormer (unmodified; bytecode in oracle/_ref/aff_model)
    on this package's operators, by the protocol of main.py:343-354 of the reference: `warmup` untimed
    forwards, then `steps` timed ones on one resident batch, images/sec = steps * batch / time; here with
    CUDA events, the maximum time over the ranks, and the batch per rank fixed (weak scaling), so the value
    is world * steps * batch / time.  16-bit legs run under autocast as the reference does (main.py:344).
    Also per leg: an end-to-end figure whose timed region copies the images from pinned host memory and
    the logits back every step, and the logits' agreement with the same model on the PyTorch gather
    formulation at a small batch."""
    import aff_harness
    if not aff_harness.available():
        return {"unavailable": "oracle/_ref/aff_model (bytecode of the reference's model) is not built"}
    records = []
    for config, batch, dname in legs:
        dtype = torch.float32 if dname == "fp32" else torch.bfloat16
        rec = {"config": config, "batch_per_gpu": batch, "dtype": dname,
               "precision": "fp32" if dname == "fp32" else "torch.autocast(bfloat16)"}
        try:
            aff_harness.use_implementation("b200")
            model = aff_harness.build_model(config, device, seed=0)
            # parity at a small batch (the formulation materialises [b,h,n,m,c])
            xs = aff_harness.synthetic_images(config, 2, device, seed=1)
            got = aff_harness.forward(model, xs, dtype)
            aff_harness.use_implementation("formula", formula_chunk=1)
            want = aff_harness.forward(model, xs, dtype)
            aff_harness.use_implementation("b200")
            rec["logits_rel_err_vs_formula"] = ((got.double() - want.double()).abs().max()
                                                / want.double().abs().max()).item()
            rec["top1_agreement"] = (got.argmax(1) == want.argmax(1)).float().mean().item()
            del model, xs, got, want
            model = aff_harness.build_model(config, device, seed=0)      # fresh stage-1 clustering cache for this batch
            images = aff_harness.synthetic_images(config, batch, device, seed=2)
            from clusten import _lib
            for _ in range(warmup):
                aff_harness.forward(model, images, dtype)
            l0 = _lib.launch_count()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            t0.record()
            for _ in range(steps):
                aff_harness.forward(model, images, dtype)
            t1.record()
            barrier()
            ms = reduce_max(t0.elapsed_time(t1))
            rec["images_per_sec"] = world * steps * batch / (ms * 1e-3)
            rec["ms_per_forward"] = ms / steps
            rec["library_launches_per_forward"] = (_lib.launch_count() - l0) / steps
            # end to end: images from pinned host memory in, logits out, every step
            host = images.cpu().pin_memory()
            out_host = torch.empty(batch, 1000, dtype=torch.float32).pin_memory()
            e_steps = max(3, steps // 3)
            barrier()
            t0.record()
            for _ in range(e_steps):
                images.copy_(host, non_blocking=True)
                out_host.copy_(aff_harness.forward(model, images, dtype).float(), non_blocking=True)
            t1.record()
            barrier()
            ms = reduce_max(t0.elapsed_time(t1))
            rec["e2e_images_per_sec"] = world * e_steps * batch / (ms * 1e-3)
            rec["e2e_h2d_bytes_per_step"] = host.numel() * 4
            rec["e2e_d2h_bytes_per_step"] = out_host.numel() * 4
            # the same model with ClusterAttention's local-attention chain done by the fused kernel (one method of
            # the model replaced: reported beside the unmodified model's figure)
            try:
                aff_harness.use_fused_attention(True)
                fused = aff_harness.forward(model, images[:2], dtype)
                aff_harness.use_fused_attention(False)
                plain = aff_harness.forward(model, images[:2], dtype)
                rec["fused_logits_rel_err_vs_separate"] = ((fused.double() - plain.double()).abs().max()
                                                           / plain.double().abs().max()).item()
                aff_harness.use_fused_attention(True)
                for _ in range(5):
                    aff_harness.forward(model, images, dtype)
                barrier()
                t0.record()
                for _ in range(steps):
                    aff_harness.forward(model, images, dtype)
                t1.record()
                barrier()
                rec["fused_attention_images_per_sec"] = world * steps * batch / (reduce_max(t0.elapsed_time(t1)) * 1e-3)
                # ... and every stage's neighbourhood tables and merge weights built by one kernel each (two more
                # methods replaced)
                aff_harness.use_fused_neighbourhood(True)
                aff_harness.use_fused_merging(True)
                both = aff_harness.forward(model, images[:2], dtype)
                rec["fused_tables_logits_rel_err_vs_separate"] = ((both.double() - plain.double()).abs().max()
                                                                  / plain.double().abs().max()).item()
                for _ in range(5):
                    aff_harness.forward(model, images, dtype)
                barrier()
                t0.record()
                for _ in range(steps):
                    aff_harness.forward(model, images, dtype)
                t1.record()
                barrier()
                rec["fused_attention_tables_merging_images_per_sec"] = (world * steps * batch
                                                                        / (reduce_max(t0.elapsed_time(t1)) * 1e-3))
            finally:
                aff_harness.use_fused(False)
            if with_reference and world == 1 and dname == "fp32" and aff_harness.reference_kernels_available():
                # the same model on the reference's own kernels (compiled unmodified into oracle/_ref), same GPU
                aff_harness.use_implementation("reference")
                for _ in range(5):
                    aff_harness.forward(model, images, dtype)
                torch.cuda.synchronize()
                t0.record()
                for _ in range(10):
                    aff_harness.forward(model, images, dtype)
                t1.record()
                torch.cuda.synchronize()
                rec["reference_kernels_images_per_sec"] = 10 * batch / (t0.elapsed_time(t1) * 1e-3)
                aff_harness.use_implementation("b200")
            del model, images
        except Exception as e:  # a leg that cannot run is reported, not hidden
            rec["error"] = f"{type(e).__name__}: {e}"[:300]
        torch.cuda.empty_cache()
        records.append(rec)
    return {"protocol": f"{warmup} warm-up + {steps} timed forwards, eval, no_grad; seeded random weights, N(0,1) "
                        "images of ImageNet's shape (dataset and checkpoints are not available)",
            "standins": "timm DropPath/trunc_normal_, cdist+topk for pykeops KNN (aff_harness.py)",
            "legs": records}


def run_b200_arm(args, dtype, rank, local_rank, world):
    from clusten import _lib, ops
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    cfg = dict(CFG)
    esize = 4 if dtype == torch.float32 else 2
    wl = make_workload(cfg, dtype, device, 1234 + rank)
    sbytes = step_bytes(cfg, esize)
    total_bytes = sum(sbytes.values())

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return t.item()

    # ---- device-resident timing: `reps` repetitions of exactly `steps` steps; the first repetition also
    #      carries the per-kernel CUDA events of the library
    for _ in range(args.warmup):
        device_step(ops, wl)
    barrier()
    sampler = ClockSampler(_physical_gpu(local_rank))
    sampler.start()
    _lib.timing_enable(True)
    _lib.timing_collect()
    launches0 = _lib.launch_count()
    first = time_step_series(ops, wl, args.steps, 1, barrier, reduce_max)
    launches = _lib.launch_count() - launches0
    kernel_ms = _lib.timing_collect()
    _lib.timing_enable(False)
    series = first + time_step_series(ops, wl, args.steps, max(0, args.reps - 1), barrier, reduce_max)
    ms = statistics.median(series)
    # the same step with the index-derived buffers built once beforehand (what every block of a stage but the
    # first runs: the operators cache them per index tensor)
    n_tok = wl["v"].shape[2]
    order0 = ops.build_row_order(wl["idx_w"])
    cached = (ops.build_inverse(wl["idx"], n_tok), ops.build_inverse(wl["idx_w"], n_tok),
              False if order0 is None else order0)
    cached_ms = statistics.median(time_step_series(ops, wl, args.steps, 3, barrier, reduce_max, cached))
    del cached

    # ---- end to end with host buffers
    e2e = EndToEnd(wl)
    for _ in range(min(args.warmup, 3)):
        e2e.step()
    e2e.finish()
    barrier()
    e_steps = max(1, min(args.steps, 10))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(e_steps):
        e2e.step()
    e2e.finish()
    stop.record()
    barrier()
    clocks = sampler.stop()
    e2e_ms = reduce_max(start.elapsed_time(stop) / e_steps)
    e2e_h2d, e2e_d2h = e2e.h2d, e2e.d2h
    del e2e
    torch.cuda.empty_cache()

    # ---- the same step in the other 16/32-bit type
    other = torch.bfloat16 if dtype == torch.float32 else torch.float32
    other_name = "bf16" if dtype == torch.float32 else "f32"
    del wl
    torch.cuda.empty_cache()
    wl2 = make_workload(cfg, other, device, 1234 + rank)
    for _ in range(max(3, args.warmup)):
        device_step(ops, wl2)
    _lib.timing_enable(True)
    _lib.timing_collect()
    o_first = time_step_series(ops, wl2, args.steps, 1, barrier, reduce_max)
    o_kernel_ms = _lib.timing_collect()
    _lib.timing_enable(False)
    o_series = o_first + time_step_series(ops, wl2, args.steps, max(0, min(args.reps, 5) - 1), barrier, reduce_max)
    o_esize = 6 - esize
    o_total = sum(step_bytes(cfg, o_esize).values())
    ref_ms = time_reference_cuda(wl2 if other == torch.float32 else None) if world == 1 else None
    del wl2
    torch.cuda.empty_cache()
    if world == 1 and ref_ms is None and dtype == torch.float32:
        wl = make_workload(cfg, dtype, device, 1234 + rank)
        ref_ms = time_reference_cuda(wl)
        del wl
        torch.cuda.empty_cache()

    model = None
    if not args.no_model:
        model = model_records(device, world, barrier, reduce_max, args.model_warmup, args.model_steps)
    config2 = config0 = None
    if world == 1 and rank == 0:
        config2 = config2_records(device)
        config0 = config0_record(device)

    if rank != 0:
        return
    peak, peak_kind = _peaks()

    def kernel_table(kms, es):
        kb = kernel_bytes(cfg, es)
        t = {}
        for name, (cnt, tot) in kms.items():
            t[name] = {"launches": cnt, "ms_per_step": tot / args.steps}
            if name in kb:
                t[name]["frac_of_hbm_peak"] = kb[name] / (tot / args.steps * 1e-3) / 1e9 / peak
        return t, kb

    per_kernel, kb = kernel_table(kernel_ms, esize)
    known = [k_ for k_ in per_kernel if k_ in kb]
    dominant = max(known, key=lambda k_: per_kernel[k_]["ms_per_step"]) if known else None
    roof = None
    if dominant is not None:
        dom_bytes = kb[dominant]
        dom_ms = per_kernel[dominant]["ms_per_step"]
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        traffic = NCU_DRAM_BYTES_PER_LAUNCH.get((dominant, args.dtype))
        roof = {"kernel": dominant, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                "traffic": traffic,
                "traffic_source": (f"ncu capture at b=32 scaled x4, kernels of build {NCU_CAPTURE_BUILD}"
                                   if traffic else None),
                "limiter": "by the roofline model the kernel is HBM-bound; the ncu summaries in profiles/ name what "
                           "actually limits it (instruction issue on index work where frac is low)",
                "ms_per_step": dom_ms, "bytes_per_step": dom_bytes}
    o_table, o_kb = kernel_table(o_kernel_ms, o_esize)
    o_ms = statistics.median(o_series)
    o_known = [k_ for k_ in o_table if k_ in o_kb]
    o_dom = max(o_known, key=lambda k_: o_table[k_]["ms_per_step"]) if o_known else None
    line = {
        "metric": "clusten_av_wf_fwd_bwd_algorithmic_bandwidth",
        "value": world * total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32" if dtype == torch.float32 else "bf16",
        "data": "synthetic",
        "config": {"workload": "config1: CLUSTENAV + CLUSTENWF(ic=4) forward+backward at stage-1 shapes, "
                               "inverse index rebuilt every step", **cfg,
                   "l2": "inputs larger than L2 (step touches > 1.5 GB)", "index_regime": "shared cluster rows"},
        "repetitions": {"count": len(series), "steps_each": args.steps, "ms_per_step_median": ms,
                        "ms_per_step_min": min(series), "ms_per_step_max": max(series)},
        "bytes_per_step": sbytes,
        "hbm_frac_of_step": total_bytes / (ms * 1e-3) / 1e9 / peak,
        "cached_index_buffers": {"ms_per_step": cached_ms, "value": world * total_bytes / (cached_ms * 1e-3) / 1e9,
                                 "unit": "GB/s", "hbm_frac_of_step": total_bytes / (cached_ms * 1e-3) / 1e9 / peak,
                                 "note": "same step with the inverse indices and the row order built beforehand "
                                         "(reported beside the headline, which rebuilds them every step)"},
        "roofline": roof,
        "kernels": per_kernel,
        "e2e": {"value": world * total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "ms_per_step": e2e_ms, "h2d_bytes_per_step": e2e_h2d, "d2h_bytes_per_step": e2e_d2h,
                "pcie_GBps_per_rank": (e2e_h2d + e2e_d2h) / (e2e_ms * 1e-3) / 1e9},
        "gpu_launches": launches * world,          # every rank launches the same kernels
        "clocks": clocks,
        other_name: {"ms_per_step": o_ms, "value": world * o_total / (o_ms * 1e-3) / 1e9, "unit": "GB/s",
                     "hbm_frac_of_step": o_total / (o_ms * 1e-3) / 1e9 / peak,
                     "repetitions": len(o_series), "dominant_kernel": o_dom,
                     "dominant_frac_of_hbm_peak": o_table[o_dom].get("frac_of_hbm_peak") if o_dom else None,
                     "kernels": o_table},
    }
    if model is not None:
        line["model"] = model
    if config2 is not None:
        line["config2"] = config2
    if config0 is not None:
        line["config0"] = config0
    if world == 1:
        cpu = time_cpu(cfg, dtype, 3, 1)
        line["cpu_baseline"] = {k: v for k, v in cpu.items() if k != "ms_per_step"}
        line["cpu_baseline"]["full_batch"] = time_cpu_full_batch(cfg, dtype)
        if ref_ms is not None:
            line["reference_cuda_ext"] = {"ms_per_step": ref_ms,
                                          "value": total_bytes / (ref_ms * 1e-3) / 1e9, "unit": "GB/s",
                                          "note": "the reference's own kernels (oracle/_ref), same step "
                                                  "without an inverse index, fp32"}
    print(json.dumps(line), flush=True)


def run_config2(args):
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peak, kind = _peaks()
    print(json.dumps({"workload": "config2: per-stage chain QK -> +bias -> softmax -> AV, WF between stages",
                      "batch": 256, "dtype": "bf16", "index_regime": "shared cluster rows",
                      "peak": f"{peak} GB/s {kind}", "stages": config2_records(device)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--dtype", choices=["fp32", "bf16"], default="fp32")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--ops", action="store_true", help="print the per-operator table instead")
    ap.add_argument("--workload", choices=["config1", "config2"], default="config1")
    ap.add_argument("--reps", type=int, default=9, help="repetitions of the timed loop (median reported)")
    ap.add_argument("--no-model", action="store_true", help="skip the model-level images/sec legs")
    ap.add_argument("--model-warmup", type=int, default=50)
    ap.add_argument("--model-steps", type=int, default=30)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    dtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, dtype, rank)
        return
    if args.ops:
        per_operator_table()
        return
    if args.workload == "config2":
        run_config2(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the operators have no CPU path)")
    if world > 1:
        torch.cuda.set_device(local_rank)
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_b200_arm(args, dtype, rank, local_rank, world)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
