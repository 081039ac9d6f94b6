"""Multi-process tests on CPU (gloo, world size 2-3): DDP equivalence of the module path and
host-side failure detection. No GPU is involved and nothing is ever hung on a device."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

from zero_to_hero_b200.parallel.fused_ddp import shard_bounds

WORKER = str(Path(__file__).resolve().parent / "dist_worker.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(mode: str, world: int, timeout: float = 120, env_extra=None):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="",
                   OMP_NUM_THREADS="1")
        env.update(env_extra or {})
        procs.append(subprocess.Popen([sys.executable, WORKER, mode], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<<killed by test timeout>>"
        outs.append(out)
    return outs


def _assert_all_ok(outs):
    for r, o in enumerate(outs):
        assert f"OK rank {r}" in o and "FAIL" not in o, f"rank {r} output:\n{o}"


def test_shard_bounds_cover_buffer_exactly():
    for total in (8, 1000, 124_475_904, 64):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(total, world, r) for r in range(world)]
            pos = 0
            for off, n in spans:
                assert off % 8 == 0 and off == min(pos, total)
                pos = off + n
            assert pos == total


def test_ddp_module_path_two_ranks():
    _assert_all_ok(run_ranks("ddp_modules", 2))


def test_heartbeat_all_alive():
    _assert_all_ok(run_ranks("heartbeat_ok", 3))


def test_heartbeat_detects_silent_rank():
    _assert_all_ok(run_ranks("heartbeat_dead_rank", 3))


def test_heartbeat_detects_orderly_leave():
    _assert_all_ok(run_ranks("heartbeat_leave", 2))


def test_collective_times_out_cleanly_when_a_rank_never_joins():
    _assert_all_ok(run_ranks("collective_timeout", 2, env_extra={"PG_TIMEOUT": "3"}))


def test_launcher_runs_cpu_ranks_and_reports_failure():
    """The job launcher starts one trainer per rank (gloo on CPU here), returns 0 when all ranks
    finish and a non-zero code when a rank fails."""
    from zero_to_hero_b200.launch import launch

    ok = launch(["--preset", "gpt2-tiny", "train.dtype=fp32", "train.steps=2", "train.total_batch_tokens=1024",
                 "train.eval_interval=0"], ranks=2, cpu=True, timeout_s=300)
    assert ok == 0
    bad = launch(["--preset", "no-such-preset"], ranks=2, cpu=True, timeout_s=120)
    assert bad != 0
