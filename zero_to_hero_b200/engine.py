"""Fused GPT-2 training engine: one hand-scheduled forward/backward over flat buffers.

Instead of an autograd graph (the reference trains through `loss.backward()` on a
`torch.compile`d module, nn/gpt2/train.py:116-127, nn/gpt2/train_ddp.py:134-143) the engine
owns

* one flat fp32 master-parameter buffer, its bf16 working copy, one flat fp32 gradient buffer
  and the AdamW moments; tensors with weight decay come first so a single index splits the
  two AdamW groups (`dim() >= 2` rule of nn/gpt2/train.py:73-84);
* every activation the backward pass needs, allocated once;
* a fixed kernel schedule for a micro-step (embedding, per block LayerNorm -> QKV GEMM ->
  flash attention -> projection GEMM with fused bias+residual -> LayerNorm -> GEMM with fused
  bias+GELU -> GEMM with fused bias+residual, final LayerNorm, lm_head GEMM, fused
  cross-entropy forward/backward, and the mirror-image backward with weight gradients
  accumulated in fp32 straight into the flat gradient buffer), captured once in a CUDA graph
  and replayed per micro-batch;
* the optimizer step: global grad-norm, clipping, AdamW, bf16 re-cast and gradient zeroing in
  two kernel launches, or, across ranks, the fused reduce-scatter + AdamW + all-gather kernel
  of `zero_to_hero_b200.parallel.fused_ddp`.

Gradient accumulation, absent from the reference, is the loop over micro-steps in
`train_step`; the 1/(tokens * micro_steps * world) factor is folded into the cross-entropy
backward so no separate scaling pass exists.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from .config import Config, ModelConfig
from .ops import _lib, gemm as G, native as N
from .ops.functional import pick_split_k
from .optim.schedule import lr_for

ALIGN = 64  # elements; keeps every tensor 256-byte (fp32) / 128-byte (bf16) aligned
HYPER_SLOTS = 8  # pinned staging slots for the per-step optimizer scalars


@dataclass
class ParamSpec:
    name: str
    shape: tuple[int, ...]
    offset: int
    decay: bool

    @property
    def numel(self) -> int:
        return math.prod(self.shape)


def _round_up(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


class ParamLayout:
    """Flat-buffer layout of a GPT-2 model; names are the Hugging Face GPT-2 state_dict keys."""

    def __init__(self, cfg: ModelConfig):
        C, L, V, T = cfg.emb_dim, cfg.num_layers, cfg.vocab_size, cfg.block_size
        decay: list[tuple[str, tuple[int, ...]]] = [
            ("transformer.wte.weight", (V, C)),
            ("transformer.wpe.weight", (T, C)),
        ]
        no_decay: list[tuple[str, tuple[int, ...]]] = []
        for i in range(L):
            p = f"transformer.h.{i}."
            decay += [
                (p + "attn.c_attn.weight", (3 * C, C)),
                (p + "attn.c_proj.weight", (C, C)),
                (p + "mlp.c_fc.weight", (4 * C, C)),
                (p + "mlp.c_proj.weight", (C, 4 * C)),
            ]
            no_decay += [(p + "ln_1.weight", (C,))]
            if cfg.ln_bias:
                no_decay += [(p + "ln_1.bias", (C,))]
            no_decay += [(p + "attn.c_attn.bias", (3 * C,)), (p + "attn.c_proj.bias", (C,)),
                         (p + "ln_2.weight", (C,))]
            if cfg.ln_bias:
                no_decay += [(p + "ln_2.bias", (C,))]
            no_decay += [(p + "mlp.c_fc.bias", (4 * C,)), (p + "mlp.c_proj.bias", (C,))]
        no_decay += [("transformer.ln_f.weight", (C,))]
        if cfg.ln_bias:
            no_decay += [("transformer.ln_f.bias", (C,))]
        self.specs: dict[str, ParamSpec] = {}
        off = 0
        for name, shape in decay:
            self.specs[name] = ParamSpec(name, shape, off, True)
            off = _round_up(off + math.prod(shape))
        self.n_decay = off
        for name, shape in no_decay:
            self.specs[name] = ParamSpec(name, shape, off, False)
            off = _round_up(off + math.prod(shape))
        self.total = off

    def backward_groups(self, num_layers: int) -> list[tuple[int, int, int]]:
        """(offset, elements, ready_key) pieces of the flat gradient buffer in the order in which
        the backward pass completes them: the matrices of layer L-1, ..., layer 0 (key = layer:
        final once that layer's backward is done), then what is final only at the very end
        (key -1): the embeddings (the tied wte receives the lm_head gradient first and the
        embedding scatter last) and the block of LayerNorm weights and biases."""
        groups = []
        for l in reversed(range(num_layers)):
            first = self.specs[f"transformer.h.{l}.attn.c_attn.weight"].offset
            nxt = (self.specs[f"transformer.h.{l + 1}.attn.c_attn.weight"].offset
                   if l + 1 < num_layers else self.n_decay)
            groups.append((first, nxt - first, l))
        emb_end = self.specs["transformer.h.0.attn.c_attn.weight"].offset if num_layers else self.n_decay
        groups.append((0, emb_end, -1))
        if self.total > self.n_decay:
            groups.append((self.n_decay, self.total - self.n_decay, -1))
        return groups

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        s = self.specs[name]
        return flat[s.offset:s.offset + s.numel].view(s.shape)

    def num_params(self) -> int:
        return sum(s.numel for s in self.specs.values())


class GPT2TrainEngine:
    """Trains a GPT-2 (`ModelConfig.kind == "gpt2"`) on one GPU, or one rank of a DDP job."""

    def __init__(self, cfg: Config, device: torch.device | str = "cuda", comm=None,
                 seed: int | None = None):
        mc = cfg.model
        if mc.kind != "gpt2":
            raise ValueError("the fused engine implements the GPT-2 architecture")
        if mc.head_dim != 64:
            raise ValueError("the flash-attention kernels are written for head_dim 64")
        if not 0.0 <= mc.dropout < 1.0:
            raise ValueError("dropout must be in [0, 1)")
        if mc.emb_dim % 8 or mc.emb_dim > 2048:
            raise ValueError("emb_dim must be a multiple of 8 and at most 2048")
        self.cfg = cfg
        self.mc = mc
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("GPT2TrainEngine needs a CUDA device (use models.GPT2 on CPU)")
        _lib.cuda_lib()  # fail loudly here if the native library was not built
        self.comm = comm
        self.world = 1 if comm is None else comm.world_size
        self.rank = 0 if comm is None else comm.rank
        self.layout = ParamLayout(mc)
        P = self.layout.total
        dev = self.device
        f32, bf16 = torch.float32, torch.bfloat16
        if comm is None:
            self.p16 = torch.zeros(P, device=dev, dtype=bf16)
            self.g = torch.zeros(P, device=dev, dtype=f32)
            self.p32 = torch.zeros(P, device=dev, dtype=f32)
            self.m = torch.zeros(P, device=dev, dtype=f32)
            self.v = torch.zeros(P, device=dev, dtype=f32)
        else:
            # gradients and the bf16 working copy live in peer-visible memory; the fp32 master
            # copy and the moments exist only for the shard this rank owns
            comm.setup(P, self.layout.n_decay, self.layout.backward_groups(mc.num_layers))
            self.p16, self.g = comm.p16, comm.g
            self.p32, self.m, self.v = comm.p32_shard, comm.m_shard, comm.v_shard
        self.hyper = torch.zeros(16, device=dev, dtype=f32)
        # The host runs ahead of the stream, so step N's hyper-parameters must not sit in memory
        # that step N+1 rewrites before the copy of step N has run: a ring of pinned slots, each
        # reused only after the event recorded behind its copy has completed.
        self._hyper_slots = [torch.zeros(16, dtype=f32).pin_memory() for _ in range(HYPER_SLOTS)]
        self._hyper_events: list[torch.cuda.Event | None] = [None] * HYPER_SLOTS
        self._hyper_next = 0
        self.partials = torch.zeros(1024, device=dev, dtype=f32)
        self.norm = torch.zeros(1, device=dev, dtype=f32)
        self.loss_accum = torch.zeros(1, device=dev, dtype=f32)
        self.loss_host = torch.zeros(1, dtype=f32).pin_memory()
        self.status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.eval_losses_buf = None
        self._eval_graphs: dict[tuple[int, int], torch.cuda.CUDAGraph] = {}
        self.opt_step = 0
        self.seed_value = cfg.train.seed if seed is None else seed
        self._alloc_activations(cfg.train.micro_batch, mc.block_size)
        self._side = torch.cuda.Stream(device=self.device)
        self._comm_stream = torch.cuda.Stream(device=self.device)
        self._side_done = []
        self._overlap = False
        self.deterministic = bool(cfg.train.deterministic)
        self._wgrad_slices = None  # K-slice workspace of the reproducible weight gradients
        # partial rows of the reproducible column sums (one buffer per stream that runs them)
        self._colsum_scratch = (torch.empty(N.colsum_scratch_elems(self.M, 4 * mc.emb_dim), device=self.device)
                                if self.deterministic else None)
        self._graphs: dict[tuple, torch.cuda.CUDAGraph] = {}
        self._reduced_in_backward = False
        self._n = 0
        self.launches_per_micro_step = 0
        self.launches_last_micro_step = 0
        self.init_weights(self.seed_value)

    # ------------------------------------------------------------------ parameters
    def init_weights(self, seed: int) -> None:
        """N(0, 0.02) for matrices and embeddings, residual projections scaled by
        1/sqrt(2 L), biases 0, LayerNorm weights 1 (nn/gpt2/modules.py:87-100)."""
        gen = torch.Generator(device="cpu").manual_seed(seed)
        full = torch.zeros(self.layout.total, dtype=torch.float32)
        L = self.mc.num_layers
        for name, s in self.layout.specs.items():
            v = full[s.offset:s.offset + s.numel].view(s.shape)
            if name.endswith("ln_1.weight") or name.endswith("ln_2.weight") or name.endswith("ln_f.weight"):
                v.fill_(1.0)
            elif name.endswith(".bias"):
                v.zero_()
            else:
                std = 0.02 / math.sqrt(2 * L) if name.endswith("c_proj.weight") else 0.02
                v.normal_(0.0, std, generator=gen)
        self.load_flat(full)

    def load_flat(self, full_fp32: torch.Tensor) -> None:
        """Install a full flat fp32 parameter vector (every rank passes the same values)."""
        full = full_fp32.to(self.device, torch.float32)
        self.p16.copy_(full.bfloat16())
        if self.comm is None:
            self.p32.copy_(full)
        else:
            self.comm.load_master(full)
        self.m.zero_()
        self.v.zero_()
        self.g.zero_()
        self.opt_step = 0

    def full_master(self) -> torch.Tensor:
        """The complete fp32 master vector (gathered across ranks when sharded)."""
        if self.comm is None:
            return self.p32.clone()
        return self.comm.gather_master()

    def state_dict(self) -> dict[str, torch.Tensor]:
        """fp32 parameters under Hugging Face GPT-2 names (Linear weights as (out, in))."""
        full = self.full_master()
        sd = {n: self.layout.view(full, n).clone() for n in self.layout.specs}
        sd["lm_head.weight"] = sd["transformer.wte.weight"]
        return sd

    def load_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        full = torch.zeros(self.layout.total, dtype=torch.float32)
        for n, s in self.layout.specs.items():
            full[s.offset:s.offset + s.numel] = sd[n].detach().float().reshape(-1).cpu()
        self.load_flat(full)

    def load_from_module(self, model: torch.nn.Module) -> None:
        self.load_state_dict(model.state_dict())

    def w(self, name: str) -> torch.Tensor:
        return self.layout.view(self.p16, name)

    def gw(self, name: str) -> torch.Tensor:
        return self.layout.view(self.g, name)

    # ------------------------------------------------------------------ activations
    def _alloc_activations(self, B: int, T: int) -> None:
        mc, dev = self.mc, self.device
        C, L, H = mc.emb_dim, mc.num_layers, mc.num_heads
        M = B * T
        self.B, self.T, self.M = B, T, M
        bf16, f32 = torch.bfloat16, torch.float32

        def buf(*shape, dtype=bf16):
            return torch.empty(*shape, device=dev, dtype=dtype)

        self.idx = torch.zeros(B, T, device=dev, dtype=torch.int64)
        self.tgt = torch.zeros(B, T, device=dev, dtype=torch.int64)
        self.resid = [buf(M, C) for _ in range(L + 1)]
        self.x_mid = [buf(M, C) for _ in range(L)]
        self.xn1 = [buf(M, C) for _ in range(L)]
        self.xn2 = [buf(M, C) for _ in range(L)]
        self.stats = [[buf(M, dtype=f32) for _ in range(4)] for _ in range(L)]
        self.qkv = [buf(M, 3 * C) for _ in range(L)]
        self.att = [buf(M, C) for _ in range(L)]
        self.lse = [buf(B, H, T, dtype=f32) for _ in range(L)]
        self.pre = [buf(M, 4 * C) for _ in range(L)]
        self.act = [buf(M, 4 * C) for _ in range(L)]
        self.xf = buf(M, C)
        self.stats_f = [buf(M, dtype=f32) for _ in range(2)]
        self.Vp = mc.padded_vocab
        self.logits = torch.zeros(M, self.Vp, device=dev, dtype=bf16)
        self.losses = buf(M, dtype=f32)
        # backward scratch
        self.d_resid = buf(M, C)
        self.d_resid_alt = buf(M, C)  # second residual-gradient buffer for the two-stream schedule
        self.d_c = buf(M, C)
        # dropout (the reference trains with 0.2): masks are a function of (seed, site, index),
        # the seed lives on the device so that a captured graph sees a new one at every replay
        self.drop_p = float(mc.dropout)
        self.drop_seed0 = int(self.seed_value) * 1_000_003 + 12345 + self.rank
        self.drop_seed = torch.full((1,), self.drop_seed0, device=dev, dtype=torch.int64)
        self.micro_steps_done = 0
        if self.drop_p > 0.0:
            self.drop_tmp = buf(M, C)  # projection output before dropout + residual
            self.d_drop = buf(M, C)    # gradient of that output
        self.d_4c = buf(M, 4 * C)
        self.d_qkv = buf(M, 3 * C)
        self.dq_accum = buf(N.flash_bwd_dq_elems(B, T, H), dtype=f32)
        self.attn_stats = buf(N.flash_bwd_stats_elems(B, T, H), dtype=f32)
        self.ln_scratch = buf(N.layernorm_bwd_num_partials(M) * 3 * C, dtype=f32)

    # ------------------------------------------------------------------ kernels schedule
    def _wgrad(self, dy: torch.Tensor, x: torch.Tensor, name: str) -> None:
        """g[name] += dy^T x with fp32 accumulation straight into the flat gradient buffer."""
        out = self.gw(name)
        n_out, k_in = out.shape
        tiles = math.ceil(n_out / 128) * math.ceil(k_in / 256)
        sk = pick_split_k(tiles, math.ceil(dy.shape[0] / 64))
        if sk > 1 and self.deterministic:
            # split-K pieces normally meet in atomics; here every K-slice is stored to its own copy of
            # the output and the copies are added in slice order
            n = out.numel()
            if self._wgrad_slices is None or self._wgrad_slices.numel() < sk * n:
                self._wgrad_slices = torch.empty(sk * n, device=self.device)
            G.gemm(dy, x, self._wgrad_slices[:n].view(n_out, k_in), a_mn=True, b_mn=True,
                   epi=G.EPI_SLICE_STORE, split_k=sk, slice_stride=n)
            G.fold_slices(self._wgrad_slices, sk, out)
            self._n += 2
            return
        if sk == 1:
            G.gemm(dy, x, out, a_mn=True, b_mn=True, epi=G.EPI_ACCUMULATE)
        else:
            G.gemm(dy, x, out, a_mn=True, b_mn=True, epi=G.EPI_ATOMIC_ADD, split_k=sk)
        self._n += 1

    # Two-stream schedule of the backward pass: the weight-gradient GEMMs and bias column sums of
    # a sub-layer do not feed the data-gradient chain, so they can run on a side stream and fill
    # the SMs that the chain's kernels leave idle in their last partial wave. A side group may lag
    # the chain by one sub-layer; the residual gradient alternates between two buffers so that the
    # chain never overwrites what a lagging group still reads.
    def _on_side(self, fn) -> None:
        if not self._overlap:
            fn()
            return
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(self._side):
            self._side.wait_event(ready)
            fn()
            done = torch.cuda.Event()
            done.record(self._side)
        self._side_done.append(done)

    def _join_side(self, keep_last: int = 0) -> None:
        main = torch.cuda.current_stream()
        while len(self._side_done) > keep_last:
            main.wait_event(self._side_done.pop(0))

    def _forward(self, B: int, T: int, pd: float) -> torch.Tensor:
        """Forward pass over the first B*T rows of the static buffers; returns the logits view
        [B*T, V]. `pd` is the dropout probability (0 for evaluation)."""
        mc = self.mc
        C, L, H, V = mc.emb_dim, mc.num_layers, mc.num_heads, mc.vocab_size
        M = B * T
        w = self.w
        has_lnb = mc.ln_bias

        def lnb(name):
            return w(name) if has_lnb else None

        def rows(t):
            return t[:M]

        seed = self.drop_seed
        idx = self.idx.view(-1)[:M].view(B, T)
        resid = [rows(t) for t in self.resid]
        N.embed_fwd(idx, w("transformer.wte.weight"), w("transformer.wpe.weight"), resid[0], T)
        self._n += 1
        if pd > 0.0:
            N.dropout_apply(resid[0], resid[0], pd, seed, 0)
            self._n += 1
        for l in range(L):
            p = f"transformer.h.{l}."
            st = [rows(t) for t in self.stats[l]]
            xn1, xn2, x_mid = rows(self.xn1[l]), rows(self.xn2[l]), rows(self.x_mid[l])
            qkv, att, pre, act = rows(self.qkv[l]), rows(self.att[l]), rows(self.pre[l]), rows(self.act[l])
            lse = self.lse[l].view(-1)[:B * H * T]
            N.layernorm_fwd(resid[l], w(p + "ln_1.weight"), lnb(p + "ln_1.bias"), xn1, st[0], st[1])
            G.gemm(xn1, w(p + "attn.c_attn.weight"), qkv, bias=w(p + "attn.c_attn.bias"))
            N.flash_fwd(qkv, att, lse, B, T, H, pd, seed, 1 + 3 * l)
            if pd > 0.0:
                tmp = rows(self.drop_tmp)
                G.gemm(att, w(p + "attn.c_proj.weight"), tmp, bias=w(p + "attn.c_proj.bias"))
                N.dropout_apply(tmp, x_mid, pd, seed, 2 + 3 * l, residual=resid[l])
                self._n += 1
            else:
                G.gemm(att, w(p + "attn.c_proj.weight"), x_mid, bias=w(p + "attn.c_proj.bias"),
                       residual=resid[l], epi=G.EPI_RESIDUAL)
            N.layernorm_fwd(x_mid, w(p + "ln_2.weight"), lnb(p + "ln_2.bias"), xn2, st[2], st[3])
            # `pre` receives gelu'(x), not x: the backward needs nothing else of the pre-activation,
            # and its GEMM epilogue becomes one load and one multiply
            G.gemm(xn2, w(p + "mlp.c_fc.weight"), act, bias=w(p + "mlp.c_fc.bias"), aux_out=pre,
                   epi=G.EPI_GELU_SAVE_GRAD)
            if pd > 0.0:
                tmp = rows(self.drop_tmp)
                G.gemm(act, w(p + "mlp.c_proj.weight"), tmp, bias=w(p + "mlp.c_proj.bias"))
                N.dropout_apply(tmp, resid[l + 1], pd, seed, 3 + 3 * l, residual=x_mid)
                self._n += 1
            else:
                G.gemm(act, w(p + "mlp.c_proj.weight"), resid[l + 1], bias=w(p + "mlp.c_proj.bias"),
                       residual=x_mid, epi=G.EPI_RESIDUAL)
            self._n += 7
        xf = rows(self.xf)
        N.layernorm_fwd(resid[L], w("transformer.ln_f.weight"), lnb("transformer.ln_f.bias"), xf,
                        rows(self.stats_f[0]), rows(self.stats_f[1]))
        logits_v = self.logits[:M, :V]
        G.gemm(xf, w("transformer.wte.weight"), logits_v)
        self._n += 2
        return logits_v

    def _reduce_ready(self, key: int) -> None:
        """Launch, on the communication stream, the reduction of the gradient buckets that the
        backward pass has just completed (`key` = layer index, -1 = end of backward). The stream
        first waits for everything issued so far on the compute streams."""
        buckets = self.comm.buckets_for(key)
        if not buckets:
            return
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        ev_side = None
        if self._overlap:
            ev_side = torch.cuda.Event()
            ev_side.record(self._side)
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ev)
            if ev_side is not None:
                self._comm_stream.wait_event(ev_side)
            for b in buckets:
                self.comm.reduce_bucket(b)
            self._n += len(buckets)
            if key < 0:
                done = torch.cuda.Event()
                done.record(self._comm_stream)
        if key < 0:
            main.wait_event(done)  # the optimizer phase follows on the main stream

    def _forward_backward(self, grad_scale: float, loss_scale: float, reduce: bool = False) -> None:
        """One micro-step on the static buffers `idx` / `tgt` (all launches, no host sync).
        `reduce`: this is the last micro-step of an optimizer step of a multi-rank job, so every
        gradient bucket is handed to the communicator as soon as it is final."""
        mc = self.mc
        C, L, H, V = mc.emb_dim, mc.num_layers, mc.num_heads, mc.vocab_size
        B, T, M = self.B, self.T, self.M
        w, gw = self.w, self.gw
        has_lnb = mc.ln_bias
        self._n = 0

        def glnb(name):
            return gw(name) if has_lnb else None

        # ---------------- forward
        pd, seed = self.drop_p, self.drop_seed
        logits_v = self._forward(B, T, pd)
        # loss and d(logits) in one pass, in place
        N.ce_fwd_bwd(self.logits, self.tgt, self.losses, V, grad_scale)
        N.reduce_sum(self.losses, self.loss_accum, scale=loss_scale, accumulate=True)
        self._n += 2

        # ---------------- backward
        G.gemm(logits_v, w("transformer.wte.weight"), self.d_c, b_mn=True)
        self._n += 1
        self._wgrad(logits_v, self.xf, "transformer.wte.weight")  # fills the machine by itself: main stream
        self._overlap = bool(self.cfg.train.overlap_wgrad) and pd == 0.0
        self._side_done = []
        R = [self.d_resid, self.d_resid_alt if self._overlap else self.d_resid]
        cur = 0  # R[cur] holds the residual-stream gradient
        # Without dropout the gradient of the residual stream IS the gradient of the projection
        # output that was added into it, so the LayerNorm backward that produces it also sums its
        # columns into that projection's bias gradient (no separate pass over it).
        fuse_db = pd == 0.0
        N.layernorm_bwd(self.d_c, self.resid[L], w("transformer.ln_f.weight"), self.stats_f[0],
                        self.stats_f[1], None, R[cur], gw("transformer.ln_f.weight"),
                        glnb("transformer.ln_f.bias"), self.ln_scratch,
                        dxsum=gw(f"transformer.h.{L - 1}.mlp.c_proj.bias") if fuse_db and L > 0 else None)
        self._n += 2
        for l in reversed(range(L)):
            p = f"transformer.h.{l}."
            st = self.stats[l]
            # MLP (the gradient of the projection output is the residual gradient through the
            # dropout mask of the forward pass)
            dy = R[cur]
            if pd > 0.0:
                N.dropout_apply(R[cur], self.d_drop, pd, seed, 3 + 3 * l)
                dy = self.d_drop
                self._n += 1

            def wg_mlp_proj(dy=dy, l=l, p=p):
                self._wgrad(dy, self.act[l], p + "mlp.c_proj.weight")
                if not fuse_db:
                    N.colsum_bf16(dy, gw(p + "mlp.c_proj.bias"), ordered=self.deterministic,
                                  scratch=self._colsum_scratch)

            self._on_side(wg_mlp_proj)
            # The c_fc bias gradient is the column sum of d_4c: a by-product of this GEMM's epilogue
            # (a column butterfly per 32 x 32 block; needs whole warps of rows). Against the separate
            # pass on the side stream it makes no measurable difference to the 124M step (950.3-952.6 k
            # tokens/s with it, 950.0-957.3 k without, alternating runs on one box) and saves a launch
            # per layer; Z2H_FC_BIAS_IN_GEMM=0 brings the separate pass back.
            fc_db_in_gemm = (self.M % 32 == 0 and os.environ.get("Z2H_FC_BIAS_IN_GEMM", "1") != "0"
                             and not self.deterministic)  # the by-product is added with atomics
            G.gemm(dy, w(p + "mlp.c_proj.weight"), self.d_4c, b_mn=True,
                   aux_in=self.pre[l], epi=G.EPI_MUL_AUX,
                   colsum=gw(p + "mlp.c_fc.bias") if fc_db_in_gemm else None)

            def wg_mlp_fc(l=l, p=p, fc_db_in_gemm=fc_db_in_gemm):
                self._wgrad(self.d_4c, self.xn2[l], p + "mlp.c_fc.weight")
                if not fc_db_in_gemm:
                    N.colsum_bf16(self.d_4c, gw(p + "mlp.c_fc.bias"), ordered=self.deterministic,
                                  scratch=self._colsum_scratch)

            self._on_side(wg_mlp_fc)
            G.gemm(self.d_4c, w(p + "mlp.c_fc.weight"), self.d_c, b_mn=True)
            self._join_side(keep_last=2)  # groups of the previous sub-layer read R[1 - cur]
            N.layernorm_bwd(self.d_c, self.x_mid[l], w(p + "ln_2.weight"), st[2], st[3],
                            R[cur], R[1 - cur], gw(p + "ln_2.weight"), glnb(p + "ln_2.bias"),
                            self.ln_scratch, dxsum=gw(p + "attn.c_proj.bias") if fuse_db else None)
            cur = 1 - cur
            # attention
            dy = R[cur]
            if pd > 0.0:
                N.dropout_apply(R[cur], self.d_drop, pd, seed, 2 + 3 * l)
                dy = self.d_drop
                self._n += 1

            def wg_attn_proj(dy=dy, l=l, p=p):
                self._wgrad(dy, self.att[l], p + "attn.c_proj.weight")
                if not fuse_db:
                    N.colsum_bf16(dy, gw(p + "attn.c_proj.bias"), ordered=self.deterministic,
                                  scratch=self._colsum_scratch)

            self._on_side(wg_attn_proj)
            G.gemm(dy, w(p + "attn.c_proj.weight"), self.d_c, b_mn=True)
            # the c_attn bias gradient (column sums of d_qkv) comes out of the attention kernels; in
            # the reproducible mode the attention backward runs one KV tile per launch (dQ accumulates
            # in a fixed order) and the bias gradient is a single-writer column sum
            det = self.deterministic
            N.flash_bwd(self.qkv[l], self.att[l], self.d_c, self.lse[l], self.d_qkv, self.dq_accum,
                        self.attn_stats, B, T, H, pd, seed, 1 + 3 * l,
                        dbias=None if det else gw(p + "attn.c_attn.bias"), ordered=det)

            def wg_attn_qkv(l=l, p=p, det=det):
                self._wgrad(self.d_qkv, self.xn1[l], p + "attn.c_attn.weight")
                if det:
                    N.colsum_bf16(self.d_qkv, gw(p + "attn.c_attn.bias"), ordered=True,
                                  scratch=self._colsum_scratch)

            self._on_side(wg_attn_qkv)
            G.gemm(self.d_qkv, w(p + "attn.c_attn.weight"), self.d_c, b_mn=True)
            self._join_side(keep_last=2)
            N.layernorm_bwd(self.d_c, self.resid[l], w(p + "ln_1.weight"), st[0], st[1],
                            R[cur], R[1 - cur], gw(p + "ln_1.weight"), glnb(p + "ln_1.bias"),
                            self.ln_scratch,
                            dxsum=gw(f"transformer.h.{l - 1}.mlp.c_proj.bias") if fuse_db and l > 0 else None)
            cur = 1 - cur
            # dgrad GEMMs, column-sum launches (the projection biases ride in the LayerNorm backward
            # without dropout, the QKV bias in the attention kernels, the c_fc bias usually in its
            # GEMM), LN bwd (2 kernels each), flash bwd (3)
            # (reproducible mode: the attention backward is one launch per KV tile, plus the QKV column sum)
            self._n += 4 + (0 if fuse_db else 2) + (0 if fc_db_in_gemm else 1) + 2 * 2
            self._n += (2 + (T + 127) // 128 + 1) if det else 3
            if reduce:
                self._reduce_ready(l)
        self._join_side()
        if pd > 0.0:
            N.dropout_apply(R[cur], R[cur], pd, seed, 0)
            self._n += 1
        N.embed_bwd(self.idx, R[cur], gw("transformer.wte.weight"),
                    gw("transformer.wpe.weight"), B, T, ordered=self.deterministic)
        self._n += 2
        if reduce:
            self._reduce_ready(-1)
            self.launches_last_micro_step = self._n
        else:
            self.launches_per_micro_step = self._n

    def dropout_seed_of_micro_step(self, k: int) -> int:
        """Seed of the dropout masks of the k-th micro-step this engine ran (k = 1, 2, ...); give it
        to `GPT2.counter_dropout_seed` to reproduce that micro-step with the PyTorch module."""
        return self.drop_seed0 + k * 0x9E3779B1

    # ------------------------------------------------------------------ public stepping API
    def micro_steps_per_step(self) -> int:
        tokens = self.B * self.T * self.world
        n = max(1, self.cfg.train.total_batch_tokens // tokens)
        return n

    def micro_step(self, idx: torch.Tensor, tgt: torch.Tensor, accum_steps: int, last: bool = False) -> None:
        """Forward + backward on one micro-batch; `idx`/`tgt` may be pinned host or device
        tensors of shape [micro_batch, block_size]. Gradients accumulate in the flat buffer.
        `last=True` marks the final micro-step before `optimizer_step`: with a communicator that
        supports it, the gradient buckets are then reduced across ranks while backward runs."""
        self.idx.copy_(idx, non_blocking=True)
        self.tgt.copy_(tgt, non_blocking=True)
        self.micro_steps_done += 1
        if self.drop_p > 0.0:
            self.drop_seed.add_(0x9E3779B1)  # new masks for this micro-step (also under graph replay)
        grad_scale = 1.0 / (self.M * accum_steps * self.world)
        loss_scale = 1.0 / (self.M * accum_steps)
        reduce = bool(last and self.comm is not None and getattr(self.comm, "supports_overlap", False))
        if reduce:
            self.comm.align_first()
            self._reduced_in_backward = True
        torch.cuda.nvtx.range_push("z2h.micro_step")
        if not self.cfg.train.use_cuda_graph:
            self._forward_backward(grad_scale, loss_scale, reduce)
            torch.cuda.nvtx.range_pop()
            return
        key = (grad_scale, loss_scale, reduce)
        graph = self._graphs.get(key)
        if graph is None:
            if any(k[:2] != key[:2] for k in self._graphs):
                self._graphs.clear()  # the accumulation factor changed: the old graphs are stale
            # warm-up outside capture (sets function attributes, loads modules), then undo its
            # side effects on the gradient / loss accumulators by capturing from a clean slate.
            # The warm-up never reduces: its signals would be taken for those of the real step.
            g_backup = self.g.clone()
            loss_backup = self.loss_accum.clone()
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._forward_backward(grad_scale, loss_scale, False)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            _lib.check_status(self.device)
            self.g.copy_(g_backup)
            self.loss_accum.copy_(loss_backup)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._forward_backward(grad_scale, loss_scale, reduce)
            self.g.copy_(g_backup)
            self.loss_accum.copy_(loss_backup)
            del g_backup
            self._graphs[key] = graph
        graph.replay()
        torch.cuda.nvtx.range_pop()

    def _write_hyper(self, lr: float) -> None:
        oc = self.cfg.optim
        t = self.opt_step
        k = self._hyper_next
        self._hyper_next = (k + 1) % HYPER_SLOTS
        ev = self._hyper_events[k]
        if ev is not None:
            ev.synchronize()  # the copy that last read this slot has run
        h = self._hyper_slots[k]
        h[0], h[1], h[2], h[3], h[4] = lr, oc.beta1, oc.beta2, oc.eps, oc.weight_decay
        h[5], h[6] = 1.0 - oc.beta1 ** t, 1.0 - oc.beta2 ** t
        h[7], h[8] = oc.clip_norm, 1.0
        self.hyper.copy_(h, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._hyper_events[k] = ev

    def optimizer_step(self, lr: float | None = None) -> None:
        """Global grad-norm clip + AdamW + bf16 re-cast + gradient zeroing."""
        self.opt_step += 1
        if lr is None:
            lr = lr_for(self.opt_step - 1, self.cfg.optim)
        self._write_hyper(lr)
        torch.cuda.nvtx.range_push("z2h.optimizer_step")
        if self.comm is None:
            n = N.gradnorm_partials(self.g, self.partials)
            N.adamw_step(self.p32, self.g, self.m, self.v, self.p16, self.layout.n_decay, self.hyper,
                         self.partials, n, self.norm, zero_grad=True)
        else:
            self.comm.fused_step(self.hyper, self.norm, reduced=self._reduced_in_backward)
            self._reduced_in_backward = False
        torch.cuda.nvtx.range_pop()

    def train_step(self, batches, lr: float | None = None) -> None:
        """One optimizer step over an iterable of (idx, tgt) micro-batches. Asynchronous: read
        the result with `read_loss()`."""
        batches = list(batches)
        self.loss_accum.zero_()
        for i, (idx, tgt) in enumerate(batches):
            self.micro_step(idx, tgt, len(batches), last=i == len(batches) - 1)
        self.optimizer_step(lr)

    def read_loss(self) -> float:
        """Device -> host read of the mean loss of the last step (synchronises the stream).
        The status word of the device travels with it: if any bounded wait of a kernel gave up
        (a peer that never signalled, a copy that never landed) the step is not trustworthy and
        this raises before the caller launches the next one."""
        status = _lib.status_word(self.device)
        self.loss_host.copy_(self.loss_accum, non_blocking=True)
        self.status_host.copy_(status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        code = int(self.status_host[0])
        if code != 0:
            status.zero_()
            raise RuntimeError(f"z2h kernel reported status {code}: "
                               f"{_lib.describe_status(code)}; the last step is invalid")
        return float(self.loss_host[0])

    # ------------------------------------------------------------------ evaluation (forward only)
    def eval_losses(self, idx: torch.Tensor, tgt: torch.Tensor) -> torch.Tensor:
        """Per-token cross-entropy [B, T] (fp32, on the device) of a forward-only pass with dropout
        off: what the reference gets from `model.eval()` + `model(X, Y)` (nn/gpt2/train.py:88-103).
        Any B x T that fits the engine's buffers (B*T <= micro_batch*block_size, T <= block_size)
        is accepted; each shape gets its own CUDA graph. Gradients, the loss accumulator, the
        dropout seed and the micro-step counter are left alone, so training is not perturbed."""
        B, T = idx.shape
        if T > self.mc.block_size or B * T > self.M:
            raise ValueError(f"batch {B}x{T} does not fit the engine's buffers ({self.M} tokens, "
                             f"context {self.mc.block_size})")
        M = B * T
        if self.eval_losses_buf is None:
            self.eval_losses_buf = torch.zeros(self.M, device=self.device, dtype=torch.float32)
        self.idx.view(-1)[:M].copy_(idx.reshape(-1), non_blocking=True)
        self.tgt.view(-1)[:M].copy_(tgt.reshape(-1), non_blocking=True)

        def run():
            saved = self._n
            logits_v = self._forward(B, T, 0.0)
            N.ce_fwd_bwd(self.logits[:M], self.tgt.view(-1)[:M], self.eval_losses_buf[:M],
                         self.mc.vocab_size, 0.0, write_grad=False)
            self._n = saved
            return logits_v

        if not self.cfg.train.use_cuda_graph:
            run()
        else:
            graph = self._eval_graphs.get((B, T))
            if graph is None:
                s = torch.cuda.Stream(device=self.device)
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    run()
                torch.cuda.current_stream().wait_stream(s)
                torch.cuda.synchronize()
                _lib.check_status(self.device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    run()
                self._eval_graphs[(B, T)] = graph
            graph.replay()
        return self.eval_losses_buf[:M].view(B, T)

    def eval_loss(self, idx: torch.Tensor, tgt: torch.Tensor) -> float:
        """Mean cross-entropy of one batch, forward only (synchronises)."""
        return float(self.eval_losses(idx, tgt).mean().item())

    def read_grad_norm(self) -> float:
        return float(self.norm.item())

    # ------------------------------------------------------------------ inference helpers
    @torch.no_grad()
    def export_to_module(self, model: torch.nn.Module) -> None:
        sd = self.state_dict()
        model.load_state_dict({k: v for k, v in sd.items()}, strict=False)

    def kernel_launches_per_step(self, micro_steps: int) -> int:
        """How many of this library's kernels one optimizer step launches."""
        if self.comm is None:
            return self.launches_per_micro_step * micro_steps + 2
        if self.launches_last_micro_step:  # the bucket reductions are counted in the last micro-step
            return (self.launches_per_micro_step * (micro_steps - 1) + self.launches_last_micro_step + 2)
        return self.launches_per_micro_step * micro_steps + self.comm.launches_per_step


def save_engine_checkpoint(engine: GPT2TrainEngine, path, data_state=None) -> None:
    """Rank 0 writes model (GPT-2 names), flat AdamW moments, step, RNG, dropout counters, data
    cursors and config. `data_state` is this rank's loader state; the states of all ranks are
    gathered and stored as a list, so that a resumed job gives every rank its own cursor back.
    Every rank returns only after the file is complete (a barrier follows the write): a rank that
    ran ahead into the next step would sit in the fused kernels' bounded device waits while
    rank 0 is still writing."""
    import torch.distributed as dist

    from .utils.checkpoint import save_checkpoint

    multi = engine.world > 1 and dist.is_initialized()
    if engine.comm is None:
        m, v = engine.m.cpu(), engine.v.cpu()
    else:
        m, v = engine.comm.gather_shards(engine.m).cpu(), engine.comm.gather_shards(engine.v).cpu()
    sd = engine.state_dict()  # gathers the sharded master weights: every rank takes part
    states = [data_state]
    if multi:
        states = [None] * engine.world
        dist.all_gather_object(states, data_state)
    if engine.rank == 0:
        optim = {"kind": "flat-adamw", "m": m, "v": v, "opt_step": engine.opt_step,
                 "drop_seed": int(engine.drop_seed.item()),
                 "micro_steps_done": engine.micro_steps_done}
        save_checkpoint(path, sd, optim, engine.opt_step,
                        {"world": engine.world, "per_rank": states}, engine.cfg.to_dict())
    if multi:
        dist.barrier()


def load_engine_checkpoint(engine: GPT2TrainEngine, path, elastic: bool = False) -> dict:
    """Restores parameters, moments, step, dropout counters and RNG; returns the checkpoint with
    `ck["data"]` replaced by THIS rank's loader state. Parameters and moments are stored whole, so
    they load into any number of ranks; the data cursors are per rank. If the job's world size
    differs from the one that wrote them this raises, unless `elastic` is set (a job that goes on
    with the ranks it has left, or was given more): the loader then gets all saved states and
    re-shards them itself (`select_rank_state`)."""
    from .utils.checkpoint import load_checkpoint, set_rng_state

    ck = load_checkpoint(path)
    engine.load_state_dict(ck["model"])
    opt = ck["optim"]
    if opt and opt.get("kind") == "flat-adamw":
        if engine.comm is None:
            engine.m.copy_(opt["m"])
            engine.v.copy_(opt["v"])
        else:
            engine.comm.scatter_shards(opt["m"], engine.m)
            engine.comm.scatter_shards(opt["v"], engine.v)
        engine.opt_step = int(opt["opt_step"])
        if "drop_seed" in opt:
            # the seed advances by a rank-independent stride; keep this rank's own offset
            advanced = int(opt["drop_seed"]) - (int(engine.seed_value) * 1_000_003 + 12345)
            engine.drop_seed.fill_(engine.drop_seed0 + advanced)
            engine.micro_steps_done = int(opt.get("micro_steps_done", 0))
    set_rng_state(ck["rng"])
    ck["data"] = select_rank_state(ck.get("data"), engine.rank, engine.world, elastic=elastic)
    return ck


def select_rank_state(data, rank: int, world: int, elastic: bool = False):
    """This rank's entry of the per-rank loader states a checkpoint holds. With another world size:
    an error, or with `elastic` a `{"reshard": True, "old_world": W, "per_rank": [...]}` record that
    the loaders' `load_state` turns into a position of their own (the token-file loader continues
    the global stream where the old job stopped, re-strided for the new rank count; the synthetic
    loader keeps the generator of the old rank with the same index, or starts a fresh stream)."""
    if not isinstance(data, dict) or "per_rank" not in data:
        return data  # a single-state checkpoint of a one-rank job
    if int(data["world"]) != world:
        if not elastic:
            raise ValueError(f"checkpoint holds data cursors of {data['world']} ranks; this job has {world} "
                             "(train.elastic_resume=true re-shards them)")
        return {"reshard": True, "old_world": int(data["world"]), "per_rank": list(data["per_rank"])}
    return data["per_rank"][rank]
