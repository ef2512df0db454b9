#!/usr/bin/env python3
"""Benchmark of the CLUSTEN operators on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype fp32|bf16] [--impl b200|reference]
    python bench.py --ops            # per-operator table (fp32 and bf16, three index regimes)

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
# benchmark's b=128 (traffic grows with the batch); see profiles/
NCU_DRAM_BYTES_PER_LAUNCH = {("av_d_value", "fp32"): 4 * (84358656 + 10250240),
                             ("av_forward", "fp32"): 4 * (103323904 + 10757888),
                             ("wf_forward", "fp32"): 4 * (54756864 + 2429440),
                             ("wf_d_weights", "fp32"): 4 * (61346816 + 2926080),
                             ("wf_d_feat", "fp32"): 4 * (50620928 + 4114688)}


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


def device_step(ops, wl):
    """The hot path through the C ABI, operands resident in HBM."""
    n = wl["v"].shape[2]
    feat = ops.av_forward(wl["attn"], wl["v"], wl["idx"])
    inv = ops.build_inverse(wl["idx"], n)
    d_attn, d_v = ops.av_backward(wl["g_feat"], wl["attn"], wl["v"], wl["idx"], inv)
    order = ops.build_row_order(wl["idx_w"])
    if order is None:
        order = False
    out = ops.wf_forward(wl["w"], wl["feat"], wl["idx_w"], order)
    inv_w = ops.build_inverse(wl["idx_w"], n)
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


# --------------------------------------------------------------------------- reference CUDA extension (speed bar)
def time_reference_cuda(wl, reps=5):
    from oracle import ref_cuda
    if not ref_cuda.available() or wl["attn"].dtype != torch.float32:
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

    # ---- device-resident timing
    for _ in range(args.warmup):
        device_step(ops, wl)
    barrier()
    sampler = ClockSampler(_physical_gpu(local_rank))
    sampler.start()
    _lib.timing_enable(True)
    _lib.timing_collect()
    launches0 = _lib.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        device_step(ops, wl)
    stop.record()
    barrier()
    launches = _lib.launch_count() - launches0
    kernel_ms = _lib.timing_collect()
    _lib.timing_enable(False)
    ms = reduce_max(start.elapsed_time(stop) / args.steps)

    # ---- end to end with host buffers
    e2e = EndToEnd(wl)
    for _ in range(min(args.warmup, 3)):
        e2e.step()
    e2e.finish()
    barrier()
    e_steps = max(1, min(args.steps, 10))
    start.record()
    for _ in range(e_steps):
        e2e.step()
    e2e.finish()
    stop.record()
    barrier()
    clocks = sampler.stop()
    e2e_ms = reduce_max(start.elapsed_time(stop) / e_steps)

    if rank != 0:
        return
    peak, peak_kind = _peaks()
    kb = kernel_bytes(cfg, esize)
    # the library reports times per kernel name; split the names that serve several operators
    per_kernel = {}
    for name, (cnt, tot) in kernel_ms.items():
        per_kernel[name] = {"launches": cnt, "ms_per_step": tot / args.steps}
    dominant = max(per_kernel, key=lambda k_: per_kernel[k_]["ms_per_step"]) if per_kernel else None
    roof = None
    if dominant is not None:
        dom_bytes = kb[dominant]
        dom_ms = per_kernel[dominant]["ms_per_step"]
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        roof = {"kernel": dominant, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((dominant, args.dtype)),
                "ms_per_step": dom_ms, "bytes_per_step": dom_bytes}
    line = {
        "metric": "clusten_av_wf_fwd_bwd_algorithmic_bandwidth",
        "value": world * total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32" if dtype == torch.float32 else "bf16",
        "data": "synthetic",
        "config": {"workload": "config1: CLUSTENAV + CLUSTENWF(ic=4) forward+backward at stage-1 shapes, "
                               "inverse index rebuilt every step", **cfg,
                   "l2": "inputs larger than L2 (step touches > 1.5 GB)", "index_regime": "shared cluster rows"},
        "bytes_per_step": sbytes,
        "hbm_frac_of_step": total_bytes / (ms * 1e-3) / 1e9 / peak,
        "roofline": roof,
        "kernels": per_kernel,
        "e2e": {"value": world * total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "ms_per_step": e2e_ms, "h2d_bytes_per_step": e2e.h2d, "d2h_bytes_per_step": e2e.d2h},
        "gpu_launches": launches * world,          # every rank launches the same kernels
        "clocks": clocks,
    }
    if world == 1:
        line["cpu_baseline"] = {k: v for k, v in time_cpu(cfg, dtype, 3, 1).items() if k != "ms_per_step"}
        ref_ms = time_reference_cuda(wl)
        if ref_ms is not None:
            line["reference_cuda_ext"] = {"ms_per_step": ref_ms,
                                          "value": total_bytes / (ref_ms * 1e-3) / 1e9, "unit": "GB/s",
                                          "note": "the reference's own kernels (oracle/_ref), same step "
                                                  "without an inverse index, fp32"}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--dtype", choices=["fp32", "bf16"], default="fp32")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--ops", action="store_true", help="print the per-operator table instead")
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
