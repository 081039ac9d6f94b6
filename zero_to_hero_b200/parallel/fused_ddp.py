"""Data-parallel communicators for the fused engine.

`FusedDDP` is the product path: gradients and the bf16 parameter copy live in symmetric
(peer-mapped) memory and one optimizer step is the bucketed reduce + global-norm clip + AdamW +
all-gather kernel family of csrc/comm/ar_adamw.cu, with P2P loads/stores (or multimem) over
NVLink issued from inside the kernels and no NCCL call; the buckets are reduced while the
backward pass of the last micro-step still runs. fp32 master weights and AdamW moments exist
only for what a rank owns (1/world of every large bucket).

`TorchDDPComm` is the baseline with the same interface: NCCL (or gloo) all-reduce of the flat
gradient buffer followed by this library's single-GPU grad-norm + AdamW kernels on a
replicated state; it is what the fused path is validated against and what runs when
symmetric memory cannot be set up.

Both replace `DistributedDataParallel(model)` + `clip_grad_norm_` + `optimizer.step()` of the
reference trainer (nn/gpt2/train_ddp.py:89,141-143). torch.distributed is used for rendezvous
and handle exchange only.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_ulonglong, c_void_p
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _lib, native as N

MAX_RANKS = 8
MAX_BUCKETS = 64
PAD_SLOTS = (8 + MAX_BUCKETS) * MAX_RANKS  # csrc/comm/signal_protocol.h: kPadSlots
ONE_SHOT, TWO_SHOT, NVLS = 0, 1, 2
F32, BF16 = 0, 1
RANGE_TWO_SHOT, RANGE_ONE_SHOT, RANGE_ZERO = 0, 1, 2


def shard_bounds(total: int, world: int, rank: int, align: int = 8) -> tuple[int, int]:
    """[offset, length) of `rank`'s shard of a flat buffer of `total` elements; every shard
    starts on an `align`-element boundary and the last one takes the remainder."""
    per = ((total + world - 1) // world + align - 1) // align * align
    off = min(rank * per, total)
    return off, max(0, min(per, total - off))


@dataclass
class Bucket:
    """A contiguous piece [off, off+n) of the flat gradient buffer that is reduced as one unit.
    `ready_key` names the point of the backward pass after which it is final (the engine uses the
    layer index; -1 = only at the very end)."""
    index: int
    off: int
    n: int
    ready_key: int
    one_shot: bool


def plan_buckets(total: int, groups: list[tuple[int, int, int]] | None, bucket_bytes: int,
                 one_shot_bytes: int, max_buckets: int = MAX_BUCKETS) -> list[Bucket]:
    """Cut the flat fp32 gradient buffer into buckets.

    `groups` lists (offset, elements, ready_key) pieces in the order in which the backward pass
    completes them (the reference's DDP builds its buckets in reverse registration order for the
    same reason, nn/gpt2/train_ddp.py:89); together they must tile [0, total). Consecutive groups
    are merged while they are adjacent in memory, final at comparable times (both keyed, or both
    end-of-backward) and the bucket is still under `bucket_bytes`; the merged bucket is ready when
    its last group is. `bucket_bytes` <= 0 or no groups: one bucket, reduced after the backward
    pass. Buckets of at most `one_shot_bytes` take the one-shot route (every rank reduces the
    whole bucket and keeps its optimizer state replicated)."""
    if not groups or bucket_bytes <= 0:
        return [Bucket(0, 0, total, -1, total * 4 <= one_shot_bytes)]
    covered = sorted((o, n) for o, n, _ in groups)
    pos = 0
    for o, n in covered:
        if o != pos or n <= 0 or o % 8 or n % 8:
            raise ValueError("gradient groups must tile the flat buffer in multiples of 8 elements")
        pos = o + n
    if pos != total:
        raise ValueError("gradient groups do not cover the flat buffer")
    merged: list[list[int]] = []  # [off, n, key]
    for off, n, key in groups:
        if merged:
            moff, mn, mkey = merged[-1]
            adjacent = off + n == moff or moff + mn == off
            if adjacent and (mkey < 0) == (key < 0) and mn * 4 < bucket_bytes:
                merged[-1] = [min(off, moff), mn + n, key]
                continue
        merged.append([off, n, key])
    if len(merged) > max_buckets:
        raise ValueError(f"{len(merged)} buckets exceed the limit of {max_buckets}; raise bucket_mb")
    return [Bucket(i, off, n, key, n * 4 <= one_shot_bytes) for i, (off, n, key) in enumerate(merged)]


@dataclass
class OwnedRange:
    goff: int   # offset in the flat buffers
    n: int
    loff: int   # offset in this rank's optimizer state
    roff: int   # offset in the one-shot result buffer (one-shot buckets only)
    kind: int


def plan_ranges(buckets: list[Bucket], total: int, world: int, rank: int):
    """What `rank` owns: its slice of every two-shot bucket and the whole of every one-shot bucket
    (replicated), laid out back to back in its optimizer state; plus the gaps, which the optimizer
    phase only clears. Returns (ranges sorted by goff incl. gaps, state elements, red elements)."""
    owned: list[OwnedRange] = []
    loff = roff = 0
    for b in buckets:
        if b.one_shot:
            continue
        so, sn = shard_bounds(b.n, world, rank)
        if sn > 0:
            owned.append(OwnedRange(b.off + so, sn, loff, 0, RANGE_TWO_SHOT))
            loff += sn
    for b in buckets:
        if b.one_shot:
            owned.append(OwnedRange(b.off, b.n, loff, roff, RANGE_ONE_SHOT))
            loff += b.n
            roff += b.n
    owned.sort(key=lambda r: r.goff)
    out: list[OwnedRange] = []
    pos = 0
    for r in owned:
        if r.goff > pos:
            out.append(OwnedRange(pos, r.goff - pos, 0, 0, RANGE_ZERO))
        out.append(r)
        pos = r.goff + r.n
    if pos < total:
        out.append(OwnedRange(pos, total - pos, 0, 0, RANGE_ZERO))
    return out, loff, roff


def _ptr_array(ptrs: list[int]):
    arr = (c_void_p * MAX_RANKS)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


def _lib_fn(name, argtypes):
    fn = getattr(_lib.cuda_lib(), name)
    fn.restype = c_int
    fn.argtypes = argtypes
    return fn


class SymmetricBuffer:
    """One tensor allocated in symmetric memory and mapped on every rank of the group."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group.group_name)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)


class PeerComm:
    """Signal pad, epoch counter and status word shared by the peer-memory collectives."""

    def __init__(self, device: torch.device, group=None, budget_s: float = 2.0):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised before building a PeerComm")
        self.device = device
        self.group = group or dist.group.WORLD
        self.rank, self.world_size = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world_size > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks (one NVSwitch domain) are supported")
        lib = _lib.cuda_lib()
        if int(lib.z2h_comm_pad_slots()) != PAD_SLOTS or int(lib.z2h_comm_max_buckets()) != MAX_BUCKETS:
            raise RuntimeError("signal pad layout of the native library differs from this module")
        self.pad = SymmetricBuffer(PAD_SLOTS, torch.int64, device, self.group)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.budget_ns = int(budget_s * 1e9)
        self._ar = _lib_fn("z2h_allreduce", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_longlong, c_int, c_int, c_void_p, c_void_p, c_ulonglong,
                                             c_void_p, c_int, c_void_p])
        torch.cuda.synchronize(device)
        dist.barrier(self.group)

    def allreduce_(self, buf: SymmetricBuffer, out: torch.Tensor | None = None, algo: int | None = None,
                   max_ctas: int = 0) -> torch.Tensor:
        """Sum all-reduce of a symmetric buffer. One-shot returns `out` (a local tensor); two-shot
        and NVLS (one kernel of multimem.ld_reduce + multimem.st, needs a multicast address)
        reduce in place. Default: one-shot up to 512 KiB, two-shot above."""
        t = buf.tensor
        nbytes = t.numel() * t.element_size()
        if algo is None:
            algo = ONE_SHOT if nbytes <= (512 << 10) else TWO_SHOT
        if algo == NVLS and not buf.multicast_ptr:
            raise RuntimeError("this symmetric buffer has no multicast address (NVLS unavailable)")
        dtype = F32 if t.dtype == torch.float32 else BF16
        if algo == ONE_SHOT and out is None:
            out = torch.empty_like(t)
        rc = self._ar(_ptr_array(buf.ptrs), _ptr_array(self.pad.ptrs), _lib.ptr(out),
                      c_void_p(buf.multicast_ptr if algo == NVLS else 0), self.rank,
                      self.world_size, t.numel(), dtype, algo, _lib.ptr(self.epoch),
                      _lib.ptr(self.done_counter), self.budget_ns,
                      _lib.ptr(_lib.status_word(self.device)), max_ctas, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"z2h_allreduce failed with code {rc}")
        return out if algo == ONE_SHOT else t


class FusedDDP(PeerComm):
    """Sharded-state data parallelism driven by the fused peer-memory kernels.

    The flat gradient buffer is cut into buckets (`plan_buckets`). `reduce_bucket(b)` launches the
    reduction of one bucket on the current stream: the engine calls it on a communication stream
    as soon as the last micro-step's backward has completed that bucket, so the reduction
    overlaps the rest of the backward pass. `optimizer_phase` then clips by the global norm, runs
    AdamW on what this rank owns and distributes the updated bf16 parameters. Large buckets are
    two-shot (each rank reduces and owns 1/world of the bucket), small ones one-shot (replicated
    state, no all-gather)."""

    supports_overlap = True

    def __init__(self, device: torch.device, group=None, budget_s: float = 2.0, nvls: bool = False,
                 bucket_mb: float = 0, one_shot_kb: int = 512, overlap_ctas: int = 24):
        """`nvls=True` asks for the multimem flavour (in-switch reduction and broadcast); it is
        used when the symmetric allocations come with a multicast address, otherwise the plain
        peer load / store kernels run (`self.nvls` tells which). `bucket_mb` = 0: one bucket
        reduced after backward. `overlap_ctas` caps the grid of a reduction that runs beside the
        backward pass (its CTAs are small enough to share an SM with a GEMM CTA)."""
        super().__init__(device, group, budget_s)
        self._bucket = _lib_fn("z2h_reduce_bucket", [
            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p, c_int,
            c_void_p, c_int, c_void_p, c_ulonglong, c_void_p, c_int, c_void_p])
        self._phase = _lib_fn("z2h_optimizer_phase", [
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
            c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
            c_void_p, c_ulonglong, c_void_p, c_int, c_void_p])
        self._grid = _lib_fn("z2h_reduce_bucket_grid", [c_longlong, c_int])
        self._want_nvls = nvls
        self.nvls = False
        self.bucket_bytes = int(float(bucket_mb) * (1 << 20))
        self.one_shot_bytes = int(one_shot_kb) << 10
        self.overlap_ctas = int(overlap_ctas)
        self._first = True
        if _lib.cuda_lib().z2h_comm_preload() != 0:
            raise RuntimeError("could not load the communication kernels")

    # ------------------------------------------------------------------ layout
    def setup(self, total: int, n_decay: int, groups: list[tuple[int, int, int]] | None = None) -> None:
        dev = self.device
        self.total, self.n_decay = total, n_decay
        self.g_buf = SymmetricBuffer(total, torch.float32, dev, self.group)
        self.p16_buf = SymmetricBuffer(total, torch.bfloat16, dev, self.group)
        self.g, self.p16 = self.g_buf.tensor, self.p16_buf.tensor
        self.nvls = bool(self._want_nvls and self.g_buf.multicast_ptr and self.p16_buf.multicast_ptr)
        bucket_bytes = self.bucket_bytes
        while True:  # a very deep model: merge more layers per bucket until the signal pad has a slot for each
            try:
                self.buckets = plan_buckets(total, groups, bucket_bytes, self.one_shot_bytes)
                break
            except ValueError as err:
                if "exceed the limit" not in str(err):
                    raise
                bucket_bytes *= 2
        self.ranges, n_state, n_red = plan_ranges(self.buckets, total, self.world_size, self.rank)
        n = max(n_state, 8)
        self.p32_shard = torch.zeros(n, device=dev)
        self.m_shard = torch.zeros(n, device=dev)
        self.v_shard = torch.zeros(n, device=dev)
        self.red = torch.zeros(max(n_red, 8), device=dev)
        # per-bucket launch geometry: slice to reduce, destination, grid, partial-sum slots
        self._launch: list[dict] = []
        red_off = 0
        n_partials = 0
        for b in self.buckets:
            if b.one_shot:
                goff, n_el, dst = b.off, b.n, self.red[red_off:red_off + b.n]
                red_off += b.n
            else:
                so, sn = shard_bounds(b.n, self.world_size, self.rank)
                goff, n_el, dst = b.off + so, sn, self.g[b.off + so:b.off + so + sn]
            cap = self.overlap_ctas if b.ready_key >= 0 else 0
            grid = int(self._grid(max(n_el, 4), cap))
            self._launch.append(dict(goff=goff, n=n_el, dst=dst, cap=cap, poff=n_partials, grid=grid,
                                     count=int((not b.one_shot) or b.index % self.world_size == self.rank)))
            n_partials += grid
        self.num_partials = n_partials
        self.partials = torch.zeros(max(n_partials, 8), device=dev)
        desc = torch.zeros(len(self.ranges), 5, dtype=torch.int64)
        for i, r in enumerate(self.ranges):
            desc[i] = torch.tensor([r.goff, r.n, r.loff, r.roff, r.kind])  # kind in the low 32 bits
        self.range_desc = desc.to(dev)
        self.total_units = sum(r.n // 8 for r in self.ranges)
        self.launches_per_step = len(self.buckets) + 2

    def buckets_for(self, ready_key: int) -> list[int]:
        return [b.index for b in self.buckets if b.ready_key == ready_key]

    def _owned(self):
        return [r for r in self.ranges if r.kind != RANGE_ZERO]

    def load_master(self, full: torch.Tensor) -> None:
        self.scatter_shards(full, self.p32_shard)

    def gather_shards(self, shard: torch.Tensor) -> torch.Tensor:
        """The full flat vector rebuilt from every rank's owned ranges (NCCL; off the hot path).
        Replicated (one-shot) ranges are contributed by rank 0."""
        full = torch.zeros(self.total, device=self.device)
        for r in self._owned():
            if r.kind == RANGE_TWO_SHOT or self.rank == 0:
                full[r.goff:r.goff + r.n].copy_(shard[r.loff:r.loff + r.n])
        dist.all_reduce(full, group=self.group)
        return full

    def scatter_shards(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        for r in self._owned():
            shard[r.loff:r.loff + r.n].copy_(full[r.goff:r.goff + r.n])

    def gather_master(self) -> torch.Tensor:
        return self.gather_shards(self.p32_shard)

    # ------------------------------------------------------------------ step
    def align_first(self) -> None:
        """Ranks reach their first reduction seconds apart (graph capture, lazy module loading);
        line them up once on the host so the in-kernel waits only ever see step skew."""
        if self._first:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            self._first = False

    def reduce_bucket(self, b: int) -> None:
        """Launch the reduction of bucket `b` on the current stream."""
        L, bk = self._launch[b], self.buckets[b]
        rc = self._bucket(_ptr_array(self.g_buf.ptrs), _ptr_array(self.pad.ptrs),
                          c_void_p(self.g_buf.multicast_ptr if self.nvls else 0), self.rank,
                          self.world_size, b, L["goff"], L["n"], _lib.ptr(L["dst"]), int(bk.one_shot),
                          c_void_p(self.partials.data_ptr() + 4 * L["poff"]), L["count"],
                          _lib.ptr(self.epoch), self.budget_ns,
                          _lib.ptr(_lib.status_word(self.device)), L["cap"], _lib.stream_ptr())
        if rc != L["grid"]:
            raise RuntimeError(f"z2h_reduce_bucket returned {rc} for bucket {b} (expected grid {L['grid']})")

    def optimizer_phase(self, hyper: torch.Tensor, norm_out: torch.Tensor) -> None:
        rc = self._phase(_ptr_array(self.g_buf.ptrs), _ptr_array(self.p16_buf.ptrs),
                         _ptr_array(self.pad.ptrs),
                         c_void_p(self.p16_buf.multicast_ptr if self.nvls else 0), _lib.ptr(self.red),
                         _lib.ptr(self.p32_shard), _lib.ptr(self.m_shard), _lib.ptr(self.v_shard),
                         self.rank, self.world_size, _lib.ptr(self.range_desc), len(self.ranges),
                         self.total_units, self.n_decay, _lib.ptr(hyper), _lib.ptr(self.partials),
                         self.num_partials, _lib.ptr(norm_out), _lib.ptr(self.epoch),
                         _lib.ptr(self.done_counter), self.budget_ns,
                         _lib.ptr(_lib.status_word(self.device)), 0, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"z2h_optimizer_phase failed with code {rc}")

    def fused_step(self, hyper: torch.Tensor, norm_out: torch.Tensor, reduced: bool = False) -> None:
        """One optimizer step. `reduced`: the engine already launched every bucket's reduction
        (overlapped with backward); otherwise all buckets are reduced here, back to back."""
        if not reduced:
            self.align_first()
            for b in range(len(self.buckets)):
                self.reduce_bucket(b)
        self.optimizer_phase(hyper, norm_out)


class TorchDDPComm:
    """Baseline communicator: library all-reduce + this package's AdamW kernels, replicated
    optimizer state. Works with NCCL on GPUs; `allreduce_flat` alone also works with gloo."""

    launches_per_step = 2
    supports_overlap = False

    def __init__(self, device: torch.device, group=None):
        self.device = device
        self.group = group or dist.group.WORLD
        self.rank, self.world_size = dist.get_rank(self.group), dist.get_world_size(self.group)

    def setup(self, total: int, n_decay: int, groups=None) -> None:
        dev = self.device
        self.total, self.n_decay = total, n_decay
        self.g = torch.zeros(total, device=dev)
        self.p16 = torch.zeros(total, device=dev, dtype=torch.bfloat16)
        self.p32_shard = torch.zeros(total, device=dev)
        self.m_shard = torch.zeros(total, device=dev)
        self.v_shard = torch.zeros(total, device=dev)
        self.partials = torch.zeros(1024, device=dev)

    def load_master(self, full: torch.Tensor) -> None:
        self.p32_shard.copy_(full)

    def gather_master(self) -> torch.Tensor:
        return self.p32_shard.clone()

    def gather_shards(self, shard: torch.Tensor) -> torch.Tensor:
        return shard.clone()

    def scatter_shards(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        shard.copy_(full)

    def fused_step(self, hyper: torch.Tensor, norm_out: torch.Tensor, reduced: bool = False) -> None:
        dist.all_reduce(self.g, group=self.group)  # gradients are pre-scaled by 1/world
        n = N.gradnorm_partials(self.g, self.partials)
        N.adamw_step(self.p32_shard, self.g, self.m_shard, self.v_shard, self.p16, self.n_decay, hyper,
                     self.partials, n, norm_out, zero_grad=True)
