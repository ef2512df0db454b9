"""Batch sharding across ranks (no collective on the data path): world-size-2 gloo run on CPU of the
bookkeeping bench.py uses -- every rank takes its own batch, the step time is the maximum over ranks
and the job throughput is N times the per-rank bytes over that time."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join({root!r}, "ml-autofocusformer_b200"))
    import workloads
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # each rank generates ITS OWN batch (weak scaling): different seeds give different tables
    idx = workloads.shared_cluster_rows(2, 136, 16, 1234 + rank)
    sig = torch.tensor([float(idx.sum())], dtype=torch.float64)
    sigs = [torch.zeros_like(sig) for _ in range(world)]
    dist.all_gather(sigs, sig)
    # the step time is the slowest rank's
    t = torch.tensor([1.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    nbytes = workloads.algorithmic_bytes("av", "fwd", b=2, h=2, n=136, m=16, c=32, s=4)
    if rank == 0:
        print(json.dumps({{"world": world, "max_ms": t.item(), "distinct": len({{s.item() for s in sigs}}),
                          "job_bytes": world * nbytes}}))
    dist.destroy_process_group()
""")


def test_two_ranks_shard_the_batch_without_a_data_collective(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    r = json.loads(line)
    assert r["world"] == 2 and r["max_ms"] == 2.0 and r["distinct"] == 2
    assert r["job_bytes"] == 2 * (2 * 2 * 2 * 136 * 32 * 4 + 2 * 136 * 16 * 8 + 2 * 2 * 136 * 16 * 4)


def test_inverse_cache_pins_and_invalidates():
    """Host logic of the inverse-index cache (no GPU needed: it only looks at tensor identity)."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "ml-autofocusformer_b200"))
    from clusten.ops import _InverseCache
    cache = _InverseCache(2)
    a = torch.zeros(2, 4, 3, dtype=torch.long)
    cache.put(a, 4, "inv-a")
    assert cache.get(a, 4) == "inv-a"
    assert cache.get(a, 5) is None                       # other target count
    a.add_(1)                                            # in-place change bumps the version
    assert cache.get(a, 4) is None
    b_, c_ = torch.zeros(2, 4, 3, dtype=torch.long), torch.zeros(2, 4, 3, dtype=torch.long)
    cache.put(b_, 4, "inv-b")
    cache.put(c_, 4, "inv-c")
    assert len(cache.entries) == 2 and cache.get(b_, 4) == "inv-b" and cache.get(c_, 4) == "inv-c"
