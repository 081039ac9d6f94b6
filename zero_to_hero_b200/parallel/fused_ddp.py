"""Data-parallel communicators for the fused engine.

`FusedDDP` is the product path: gradients and the bf16 parameter copy live in symmetric
(peer-mapped) memory and one optimizer step is the three-launch reduce-scatter + global-norm
clip + AdamW + all-gather kernel family of csrc/comm/ar_adamw.cu, with P2P loads/stores over
NVLink issued from inside the kernels and no NCCL call. fp32 master weights and AdamW moments
exist only for the shard a rank owns (1/world of the model).

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

import torch
import torch.distributed as dist

from ..ops import _lib, native as N

MAX_RANKS = 8
PAD_SLOTS = 8 * MAX_RANKS
ONE_SHOT, TWO_SHOT = 0, 1
F32, BF16 = 0, 1


def shard_bounds(total: int, world: int, rank: int, align: int = 8) -> tuple[int, int]:
    """[offset, length) of `rank`'s shard of a flat buffer of `total` elements; every shard
    starts on an `align`-element boundary and the last one takes the remainder."""
    per = ((total + world - 1) // world + align - 1) // align * align
    off = min(rank * per, total)
    return off, max(0, min(per, total - off))


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
        self.pad = SymmetricBuffer(PAD_SLOTS, torch.int64, device, self.group)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.budget_ns = int(budget_s * 1e9)
        self._ar = _lib_fn("z2h_allreduce", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong,
                                             c_int, c_int, c_void_p, c_void_p, c_ulonglong, c_void_p,
                                             c_int, c_void_p])
        torch.cuda.synchronize(device)
        dist.barrier(self.group)

    def allreduce_(self, buf: SymmetricBuffer, out: torch.Tensor | None = None, algo: int | None = None,
                   max_ctas: int = 0) -> torch.Tensor:
        """Sum all-reduce of a symmetric buffer. One-shot returns `out` (a local tensor), two-shot
        reduces in place. Default: one-shot up to 512 KiB, two-shot above."""
        t = buf.tensor
        nbytes = t.numel() * t.element_size()
        if algo is None:
            algo = ONE_SHOT if nbytes <= (512 << 10) else TWO_SHOT
        dtype = F32 if t.dtype == torch.float32 else BF16
        if algo == ONE_SHOT and out is None:
            out = torch.empty_like(t)
        rc = self._ar(_ptr_array(buf.ptrs), _ptr_array(self.pad.ptrs), _lib.ptr(out), self.rank,
                      self.world_size, t.numel(), dtype, algo, _lib.ptr(self.epoch),
                      _lib.ptr(self.done_counter), self.budget_ns,
                      _lib.ptr(_lib.status_word(self.device)), max_ctas, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"z2h_allreduce failed with code {rc}")
        return out if algo == ONE_SHOT else t


class FusedDDP(PeerComm):
    """Sharded-state data parallelism driven by the fused peer-memory kernels."""

    launches_per_step = 3

    def __init__(self, device: torch.device, group=None, budget_s: float = 2.0, nvls: bool = False,
                 bucket_mb: int = 0):
        """`nvls=True` asks for the multimem flavour (in-switch reduction and broadcast); it is
        used when the symmetric allocations come with a multicast address, otherwise the plain
        peer load / store kernels run (`self.nvls` tells which)."""
        super().__init__(device, group, budget_s)
        self._step = _lib_fn("z2h_fused_step_twoshot", [
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong,
            c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
            c_ulonglong, c_void_p, c_int, c_void_p])
        self._step_nvls = _lib_fn("z2h_fused_step_twoshot_nvls", [
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
            c_longlong, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
            c_void_p, c_ulonglong, c_void_p, c_int, c_void_p])
        self._want_nvls = nvls
        self.nvls = False
        self.bucket_mb = int(bucket_mb)
        self._first = True

    def setup(self, total: int, n_decay: int) -> None:
        dev = self.device
        self.total, self.n_decay = total, n_decay
        self.g_buf = SymmetricBuffer(total, torch.float32, dev, self.group)
        self.p16_buf = SymmetricBuffer(total, torch.bfloat16, dev, self.group)
        self.g, self.p16 = self.g_buf.tensor, self.p16_buf.tensor
        self.shard_off, self.shard_n = shard_bounds(total, self.world_size, self.rank)
        self.nvls = bool(self._want_nvls and self.g_buf.multicast_ptr and self.p16_buf.multicast_ptr)
        n = max(self.shard_n, 8)
        self.p32_shard = torch.zeros(n, device=dev)
        self.m_shard = torch.zeros(n, device=dev)
        self.v_shard = torch.zeros(n, device=dev)
        self.partials = torch.zeros(1024, device=dev)

    def load_master(self, full: torch.Tensor) -> None:
        self.p32_shard[:self.shard_n].copy_(full[self.shard_off:self.shard_off + self.shard_n])

    def gather_shards(self, shard: torch.Tensor) -> torch.Tensor:
        """All ranks' shards concatenated into the full flat vector (NCCL; off the hot path)."""
        per = shard_bounds(self.total, self.world_size, 0)[1]
        mine = torch.zeros(per, device=self.device)
        mine[:self.shard_n].copy_(shard[:self.shard_n])
        out = torch.empty(per * self.world_size, device=self.device)
        dist.all_gather_into_tensor(out, mine, group=self.group)
        return out[:self.total]

    def scatter_shards(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        shard[:self.shard_n].copy_(full[self.shard_off:self.shard_off + self.shard_n])

    def gather_master(self) -> torch.Tensor:
        return self.gather_shards(self.p32_shard)

    def fused_step(self, hyper: torch.Tensor, norm_out: torch.Tensor) -> None:
        if self._first:
            # ranks reach their first step seconds apart (graph capture, lazy module loading);
            # line them up once on the host so the in-kernel waits only ever see step skew
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            self._first = False
        if self.nvls:
            rc = self._step_nvls(_ptr_array(self.g_buf.ptrs), _ptr_array(self.p16_buf.ptrs),
                                 _ptr_array(self.pad.ptrs), self.g_buf.multicast_ptr,
                                 self.p16_buf.multicast_ptr, _lib.ptr(self.p32_shard),
                                 _lib.ptr(self.m_shard), _lib.ptr(self.v_shard), self.rank,
                                 self.world_size, self.shard_off, self.shard_n, self.total, self.n_decay,
                                 _lib.ptr(hyper), _lib.ptr(self.partials), _lib.ptr(norm_out),
                                 _lib.ptr(self.epoch), _lib.ptr(self.done_counter), self.budget_ns,
                                 _lib.ptr(_lib.status_word(self.device)), 0, _lib.stream_ptr())
            if rc != 0:
                raise RuntimeError(f"z2h_fused_step_twoshot_nvls failed with code {rc}")
            return
        rc = self._step(_ptr_array(self.g_buf.ptrs), _ptr_array(self.p16_buf.ptrs),
                        _ptr_array(self.pad.ptrs), _lib.ptr(self.p32_shard), _lib.ptr(self.m_shard),
                        _lib.ptr(self.v_shard), self.rank, self.world_size, self.shard_off,
                        self.shard_n, self.total, self.n_decay, _lib.ptr(hyper),
                        _lib.ptr(self.partials), _lib.ptr(norm_out), _lib.ptr(self.epoch),
                        _lib.ptr(self.done_counter), self.budget_ns,
                        _lib.ptr(_lib.status_word(self.device)), 0, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"z2h_fused_step_twoshot failed with code {rc}")


class TorchDDPComm:
    """Baseline communicator: library all-reduce + this package's AdamW kernels, replicated
    optimizer state. Works with NCCL on GPUs; `allreduce_flat` alone also works with gloo."""

    launches_per_step = 2

    def __init__(self, device: torch.device, group=None):
        self.device = device
        self.group = group or dist.group.WORLD
        self.rank, self.world_size = dist.get_rank(self.group), dist.get_world_size(self.group)

    def setup(self, total: int, n_decay: int) -> None:
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

    def fused_step(self, hyper: torch.Tensor, norm_out: torch.Tensor) -> None:
        dist.all_reduce(self.g, group=self.group)  # gradients are pre-scaled by 1/world
        n = N.gradnorm_partials(self.g, self.partials)
        N.adamw_step(self.p32_shard, self.g, self.m_shard, self.v_shard, self.p16, self.n_decay, hyper,
                     self.partials, n, norm_out, zero_grad=True)
