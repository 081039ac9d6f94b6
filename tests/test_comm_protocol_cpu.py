"""Signalling protocol and bucket planning of the fused data-parallel step, on the CPU.

The protocol functions are the ones the CUDA kernels use (csrc/comm/signal_protocol.h), compiled
for the host with std::atomic and driven with one thread per rank (csrc/cpu/protocol_sim.cpp), so
a peer that never signals is a thread that stays quiet: no GPU ever waits for anything here."""
import ctypes

import pytest

from zero_to_hero_b200.ops import _lib
from zero_to_hero_b200.parallel.fused_ddp import (MAX_BUCKETS, PAD_SLOTS, RANGE_ONE_SHOT, RANGE_TWO_SHOT,
                                                  RANGE_ZERO, plan_buckets, plan_ranges, shard_bounds)


@pytest.fixture(scope="module")
def host():
    lib = _lib.host_lib()
    lib.z2h_protocol_sim_steps.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint]
    lib.z2h_protocol_sim_silent_peer.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
    lib.z2h_protocol_sim_last_one_out.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.z2h_protocol_epoch_reached.argtypes = [ctypes.c_uint, ctypes.c_uint]
    return lib


def test_pad_layout_matches_python_constants(host):
    assert host.z2h_protocol_pad_slots() == PAD_SLOTS


def test_epoch_comparison_is_wrap_safe(host):
    r = host.z2h_protocol_epoch_reached
    assert r(5, 5) == 1 and r(6, 5) == 1 and r(4, 5) == 0
    assert r(2, 0xFFFFFFFE) == 1          # 2 is four steps after 0xFFFFFFFE
    assert r(0xFFFFFFFE, 2) == 0          # and the old epoch does not satisfy the new one
    assert r(0, 0xFFFFFFFF) == 1


@pytest.mark.parametrize("world", [2, 3, 8])
def test_clean_steps_with_buckets_and_norm_exchange(host, world):
    assert host.z2h_protocol_sim_steps(world, 25, 5, 0) == 0


def test_steps_across_the_epoch_wrap(host):
    assert host.z2h_protocol_sim_steps(4, 40, 3, 0xFFFFFFF0) == 0


def test_silent_peer_times_out_and_late_signal_is_not_mistaken(host):
    world, budget_ms = 4, 150
    out = (ctypes.c_int * (4 * world))()
    assert host.z2h_protocol_sim_silent_peer(world, budget_ms, out) == 0
    rows = [list(out[4 * r:4 * r + 4]) for r in range(world)]
    for r in range(world - 1):
        timed_out, status, step2, waited_ms = rows[r]
        assert timed_out == 0, rows            # the wait gave up ...
        assert status == 5, rows               # ... and said why (peer timeout)
        assert budget_ms <= waited_ms < budget_ms + 2000, rows   # ... inside its budget
        assert step2 == 1, rows                # the next step completes, and not on the stale signal
    assert rows[world - 1][2] == 1


def test_last_one_out_elects_exactly_one(host):
    assert host.z2h_protocol_sim_last_one_out(16, 50) == 50


# ---------------------------------------------------------------------------------------------
def _gpt2_like_groups(L=4, per_layer=12 * 64 * 64, emb=1024 * 64, small=640):
    off = emb
    layer_off = []
    for _ in range(L):
        layer_off.append(off)
        off += per_layer
    groups = [(layer_off[l], per_layer, l) for l in reversed(range(L))]
    groups.append((0, emb, -1))
    groups.append((off, small, -1))
    return groups, off + small


def test_bucket_plan_tiles_buffer_in_backward_order():
    groups, total = _gpt2_like_groups()
    per_layer_bytes = 12 * 64 * 64 * 4
    buckets = plan_buckets(total, groups, per_layer_bytes, one_shot_bytes=4096)
    # one bucket per layer, last layer first, then the embeddings and the small-parameter block
    assert [b.ready_key for b in buckets] == [3, 2, 1, 0, -1, -1]
    assert sorted((b.off, b.n) for b in buckets)[0][0] == 0
    assert sum(b.n for b in buckets) == total
    assert [b.one_shot for b in buckets] == [False] * 5 + [True]   # only the 2.5 KB block is one-shot
    # a larger bucket size merges neighbouring layers; the merged bucket is ready with its LAST layer
    merged = plan_buckets(total, groups, 2 * per_layer_bytes + 1, one_shot_bytes=0)
    assert [b.ready_key for b in merged][:2] == [1, 0] or [b.ready_key for b in merged][:2] == [2, 0]
    assert sum(b.n for b in merged) == total
    for b in merged:
        assert b.off % 8 == 0 and b.n % 8 == 0
    # bucket size 0: one bucket, reduced after backward
    single = plan_buckets(total, groups, 0, one_shot_bytes=0)
    assert len(single) == 1 and (single[0].off, single[0].n, single[0].ready_key) == (0, total, -1)
    with pytest.raises(ValueError):
        plan_buckets(total, groups[:-1], per_layer_bytes, 0)   # a hole in the cover
    with pytest.raises(ValueError):
        plan_buckets(total, groups, 1, 0, max_buckets=3)


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_ranges_of_all_ranks_partition_every_two_shot_bucket(world):
    groups, total = _gpt2_like_groups()
    buckets = plan_buckets(total, groups, 12 * 64 * 64 * 4, one_shot_bytes=4096)
    owners = [0] * total
    for rank in range(world):
        ranges, n_state, n_red = plan_ranges(buckets, total, world, rank)
        pos = 0
        state = 0
        for r in ranges:                      # sorted, gap-free cover of the flat buffer
            assert r.goff == pos and r.n > 0 and r.n % 8 == 0 and r.goff % 8 == 0
            pos += r.n
            if r.kind != RANGE_ZERO:
                state += r.n
            if r.kind == RANGE_TWO_SHOT:
                for i in range(r.goff, r.goff + r.n, 8):
                    owners[i] += 1
            if r.kind == RANGE_ONE_SHOT:
                assert r.roff + r.n <= n_red
        assert pos == total and state == n_state
        assert n_red == sum(b.n for b in buckets if b.one_shot)
    for b in buckets:
        want = 0 if b.one_shot else 1
        assert all(owners[i] == want for i in range(b.off, b.off + b.n, 8)), b
    assert len(buckets) <= MAX_BUCKETS
    # the slices of one bucket are what shard_bounds says
    b0 = buckets[0]
    assert sum(shard_bounds(b0.n, world, r)[1] for r in range(world)) == b0.n


def test_bucket_size_grows_until_the_plan_fits_the_signal_pad():
    """100 layers at one bucket per layer would need more signal slots than a pad has; the
    communicator doubles the bucket size until the plan fits (same loop as FusedDDP.setup)."""
    groups, total = _gpt2_like_groups(L=100, per_layer=12 * 64 * 64)
    size = 12 * 64 * 64 * 4
    with pytest.raises(ValueError):
        plan_buckets(total, groups, size, 0)
    while True:
        try:
            buckets = plan_buckets(total, groups, size, 0)
            break
        except ValueError:
            size *= 2
    assert len(buckets) <= MAX_BUCKETS and sum(b.n for b in buckets) == total
    assert buckets[0].ready_key < 99     # several layers share the first bucket


@pytest.mark.parametrize("preset", ["gpt2-124m", "gpt2-350m", "gpt2-1.5b"])
def test_bucket_and_range_plan_covers_every_preset_at_every_world(preset):
    """For the real parameter layouts: at 2, 4 and 8 ranks every rank's ranges tile the flat buffer in
    units of 8 elements, every element of a two-shot bucket has exactly one owner and every element of
    a one-shot bucket is kept by all ranks."""
    import torch
    from zero_to_hero_b200.config import get_preset
    from zero_to_hero_b200.engine import ParamLayout
    cfg = get_preset(preset)
    lay = ParamLayout(cfg.model)
    groups = lay.backward_groups(cfg.model.num_layers)
    bucket_bytes = 32 << 20
    while True:  # what FusedDDP.setup does: grow the bucket size until the count fits
        try:
            buckets = plan_buckets(lay.total, groups, bucket_bytes, 512 << 10)
            break
        except ValueError:
            bucket_bytes *= 2
    one_shot = torch.zeros(lay.total, dtype=torch.bool)
    for b in buckets:
        if b.one_shot:
            one_shot[b.off:b.off + b.n] = True
    for world in (2, 4, 8):
        owners = torch.zeros(lay.total, dtype=torch.int16)
        for rank in range(world):
            ranges, _, _ = plan_ranges(buckets, lay.total, world, rank)
            pos = 0
            for rg in sorted(ranges, key=lambda x: x.goff):
                assert rg.goff == pos and rg.n % 8 == 0 and rg.goff % 8 == 0, (world, rank, rg)
                pos += rg.n
                if rg.kind != RANGE_ZERO:
                    owners[rg.goff:rg.goff + rg.n] += 1
            assert pos == lay.total
        assert bool((owners[~one_shot] == 1).all()) and bool((owners[one_shot] == world).all())
