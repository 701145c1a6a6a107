"""Host-side multi-rank logic on CPU (gloo, world size 2): shard plans are disjoint and
cover the global batch, timings reduce with max over ranks, and the reference arm of
bench.py runs on rank 0 only when launched under torchrun."""
import json
import os
import socket
import subprocess
import sys

import helpers

ROOT = helpers.ROOT

_WORKER = r"""
import os, sys, json
sys.path.insert(0, %r)
import torch.distributed as dist
import bench
dist.init_process_group("gloo")
r, w = dist.get_rank(), dist.get_world_size()
plan = bench.shard_plan(r, w, 256)
plans = [None] * w
dist.all_gather_object(plans, plan)
mx = bench.max_over_ranks([1.0 + r, 10.0 - r])
if r == 0:
    print(json.dumps({"plans": plans, "max": mx}))
dist.destroy_process_group()
"""


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _torchrun(args, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port())] + args
    env = dict(os.environ, OMP_NUM_THREADS="4")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def test_shard_plans_and_max_reduction_with_two_gloo_ranks(tmp_path):
    w = tmp_path / "worker.py"
    w.write_text(_WORKER % ROOT)
    r = _torchrun([str(w)])
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    plans = out["plans"]
    assert [p["row_offset"] for p in plans] == [0, 256]
    assert all(p["rows"] == 256 and p["global_rows"] == 512 for p in plans)
    assert len({p["prefix_seed"] for p in plans}) == 2
    # every rank draws from the counter-based stream keyed by the global row, so sharding does not change a row's codes
    assert all(p["rng_mode"] == 1 for p in plans)
    import numpy as np
    import bench
    a = np.arange(12, dtype=np.int32).reshape(3, 4)
    assert bench.token_checksum(a) == bench.token_checksum(a.copy()) != bench.token_checksum(a[::-1])
    assert out["max"] == [2.0, 10.0]


def test_reference_arm_runs_on_rank_zero_only_under_torchrun():
    r = _torchrun([os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--workload", "c2s",
                   "--steps", "1", "--warmup", "0"])
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port")
    assert d["e2e"]["h2d_bytes_per_step"] == 0
