"""Child-process bodies of the multi-rank CPU tests (gloo); launched by test_distributed_cpu.py."""
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    from datetime import timedelta
    dist.init_process_group("gloo", timeout=timedelta(seconds=float(os.environ.get("PG_TIMEOUT", "20"))))
    from zero_to_hero_b200.parallel.health import HeartbeatMonitor, RankFailure, default_store

    if mode == "ddp_modules":
        # module path + torch DDP over gloo: replicas stay identical, loss matches a 1-rank run
        from zero_to_hero_b200.config import get_preset
        from zero_to_hero_b200.train import train
        cfg = get_preset("gpt2-tiny")
        cfg.train.dtype, cfg.train.steps, cfg.train.eval_interval = "fp32", 3, 0
        cfg.train.total_batch_tokens = cfg.train.micro_batch * cfg.model.block_size * world * 2
        out = train(cfg)
        sd = out["model"].state_dict()
        flat = torch.cat([v.reshape(-1).float() for v in sd.values()])
        gathered = [torch.zeros_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        assert all(torch.equal(gathered[0], g) for g in gathered), "replicas diverged"
        print(f"OK rank {rank} loss {out['history'][-1]['train']:.4f}")
    elif mode == "heartbeat_ok":
        mon = HeartbeatMonitor(default_store(), rank, world, timeout_s=10)
        for step in range(3):
            mon.beat(step)
            mon.wait_all(step)
        print(f"OK rank {rank}")
    elif mode == "heartbeat_dead_rank":
        # the last rank stops after step 0 without a word; the others must notice on the host
        mon = HeartbeatMonitor(default_store(), rank, world, timeout_s=2)
        mon.beat(0)
        mon.wait_all(0)
        if rank == world - 1:
            time.sleep(6)  # plays dead: no heartbeat, no collective
            print(f"OK rank {rank} (played dead)")
            os._exit(0)
        mon.beat(1)
        try:
            mon.wait_all(1)
            print(f"FAIL rank {rank}: no failure detected")
        except RankFailure as e:
            assert e.rank == world - 1
            print(f"OK rank {rank} detected: {e}")
        os._exit(0)
    elif mode == "heartbeat_leave":
        mon = HeartbeatMonitor(default_store(), rank, world, timeout_s=5)
        mon.beat(0)
        mon.wait_all(0)
        if rank == world - 1:
            # leaves between steps: only once every peer has started step 1 (a "left" written
            # while a slow peer still waits for step 0 would replace the beat that peer needs)
            mon.wait_all(1)
            mon.leave()
            print(f"OK rank {rank} left")
            os._exit(0)
        mon.beat(1)
        try:
            mon.wait_all(1)
            print(f"FAIL rank {rank}")
        except RankFailure as e:
            assert "left" in str(e)
            print(f"OK rank {rank} detected: {e}")
        os._exit(0)
    elif mode == "collective_timeout":
        # a rank that never joins a collective: the short process-group timeout ends it with an error
        if rank == world - 1:
            time.sleep(8)
            print(f"OK rank {rank} (never joined)")
            os._exit(0)
        t = torch.ones(4)
        try:
            dist.all_reduce(t)
            print(f"FAIL rank {rank}: all_reduce returned")
        except Exception as e:
            print(f"OK rank {rank} collective failed cleanly: {type(e).__name__}")
        os._exit(0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
