"""Multi-GPU tests of the peer-memory collectives and the fused DDP step. They run as child
processes (one per GPU) with NVLS disabled in NCCL; the library's own kernels use plain peer
loads/stores. Skipped when fewer than two GPUs are visible."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
WORKER = str(Path(__file__).resolve().parent / "ddp_gpu_worker.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world, extra_env):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        env.update(extra_env)
        procs.append(subprocess.Popen([sys.executable, WORKER], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<<killed by test timeout>>"
        outs.append(out)
    for r, o in enumerate(outs):
        assert f"OK rank {r}" in o, f"rank {r} output:\n{o[-3000:]}"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_ddp_matches_nccl_baseline(world):
    """Standalone all-reduces vs NCCL; bucketed (overlapped) and single-bucket fused steps vs the
    NCCL + local AdamW baseline; a late rank inside and beyond the device wait budget."""
    _run(world, {})


@pytest.mark.parametrize("world", [2, 8])
def test_fused_ddp_multimem_flavour(world):
    """The same with the in-switch (multimem) reduction and broadcast; no rank is late here."""
    _run(world, {"Z2H_TEST_NVLS": "1", "Z2H_TEST_SLOW_RANK": "0"})
