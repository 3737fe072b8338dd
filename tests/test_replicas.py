"""CPU tests of the multi-GPU (replicas-only) plumbing of bench.py: world_size-2 gloo ranks agree on the
max-over-ranks time and the whole-job throughput, and rank 0 alone prints the reference arm."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, json
sys.path.insert(0, {root!r})
import torch, torch.distributed as dist
import bench
rank, world, local = bench.dist_env()
dist.init_process_group("gloo", rank=rank, world_size=world)
# each replica "took" a different time for the same number of tokens
mine = 0.5 + 0.25 * rank
slowest = bench.max_over_ranks(mine, world, torch.device("cpu"))
value = bench.aggregate(tokens_per_rank=1000, seconds_max=slowest, world=world)
dist.barrier()
print(json.dumps({{"rank": rank, "slowest": slowest, "value": value}}))
dist.destroy_process_group()
"""


def _spawn(rank, world, port, script):
    env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
               MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    return subprocess.Popen([sys.executable, "-c", script], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                            text=True)


def test_two_replicas_aggregate_over_gloo():
    script = WORKER.format(root=ROOT)
    port = 29000 + os.getpid() % 2000
    procs = [_spawn(r, 2, port, script) for r in range(2)]
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err[-2000:]
        outs.append(json.loads(out.strip().splitlines()[-1]))
    for o in outs:
        assert o["slowest"] == pytest.approx(0.75)          # max over ranks, same on every rank
        assert o["value"] == pytest.approx(2 * 1000 / 0.75)  # all ranks' tokens / slowest rank's time


def test_step_bytes_matches_roofline_figures():
    sys.path.insert(0, ROOT)
    import bench
    import synthetic as S
    assert bench.step_bytes(4096, 256) == sum(S.decode_step_bytes(4096 + i) for i in range(256))
    assert bench.step_bytes(4096, 1) == 1_192_101_888 + 114_688 * 4096 + 114_688


def test_reference_arm_runs_on_rank0_only():
    """Under torchrun-style env with RANK=1 the reference arm does no work and prints nothing."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--gpus", "2"], env=env, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and p.stdout.strip() == ""
