"""GPT-2: pre-LayerNorm decoder with a weight-tied lm_head.

Same network as the reference's `GPT` (nn/gpt2/modules.py:17-137): fused QKV projection with
bias, causal attention, output projection, tanh-GELU MLP, LayerNorms without bias (optional
here), learned token + position embeddings, a bias-free head tied to the token embedding,
N(0, 0.02) init with the residual projections scaled by 1/sqrt(2 * num_layers).

The module tree is laid out so that `state_dict()` keys are the Hugging Face GPT-2 names
(`transformer.wte.weight`, `transformer.h.0.attn.c_attn.weight`, ..., `lm_head.weight`);
`zero_to_hero_b200.utils.checkpoint` maps them from/to the reference's names.

`forward(X, Y=None) -> (logits, loss)` and `generate(...)` keep the reference's contract.
On a CUDA device the ops run the hand-written sm_100a kernels in bf16 through
`zero_to_hero_b200.ops.functional`; on CPU they run plain PyTorch in the parameter dtype.
For training at speed use `zero_to_hero_b200.engine.GPT2TrainEngine`, which runs the same
network as one hand-scheduled forward/backward over flat buffers.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import dropout as D
from ..ops import functional as Z


class LayerNorm(nn.Module):
    def __init__(self, dim: int, bias: bool, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim)) if bias else None
        self.eps = eps

    def forward(self, x):
        return Z.layer_norm(x, self.weight, self.bias, self.eps)


def _counter_dropout(x: torch.Tensor, p: float, seed: int, site: int) -> torch.Tensor:
    """Dropout with the counter-based mask the fused engine's kernels use (ops/dropout.py)."""
    keep = D.elementwise_keep(x.numel(), p, seed, site, x.device).view(x.shape)
    return x * (keep.to(x.dtype) * D.threshold_and_scale(p)[1])


def _counter_dropout_attention(qkv: torch.Tensor, num_heads: int, p: float, seed: int, site: int):
    """Plain causal attention whose probabilities are dropped with the engine's mask."""
    B, T, C3 = qkv.shape
    C = C3 // 3
    hd = C // num_heads
    q, k, v = (t.view(B, T, num_heads, hd).transpose(1, 2) for t in qkv.split(C, dim=-1))
    att = (q @ k.transpose(-2, -1)) * hd ** -0.5
    causal = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    att = att.masked_fill(~causal, float("-inf")).softmax(dim=-1)
    keep = D.attention_keep(B, num_heads, T, p, seed, site, qkv.device)
    att = att * (keep.to(att.dtype) * D.threshold_and_scale(p)[1])
    return (att @ v).transpose(1, 2).contiguous().view(B, T, C)


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        assert cfg.emb_dim % cfg.num_heads == 0
        self.c_attn = nn.Linear(cfg.emb_dim, 3 * cfg.emb_dim)
        self.c_proj = nn.Linear(cfg.emb_dim, cfg.emb_dim)
        self.num_heads = cfg.num_heads
        self.dropout = cfg.dropout

    def forward(self, x, residual, cdrop=None):
        """`cdrop` = (seed, layer) selects the counter-based masks of the fused engine instead
        of torch's generator, so that the module reproduces an engine step exactly."""
        qkv = Z.linear(x, self.c_attn.weight, self.c_attn.bias)
        p = self.dropout if self.training else 0.0
        if p > 0.0 and cdrop is not None:
            seed, layer = cdrop
            y = _counter_dropout_attention(qkv, self.num_heads, p, seed, 1 + 3 * layer)
            y = Z.linear(y, self.c_proj.weight, self.c_proj.bias)
            return residual + _counter_dropout(y, p, seed, 2 + 3 * layer)
        y = Z.causal_attention(qkv, self.num_heads, dropout_p=p)
        if p > 0.0:
            y = Z.linear(y, self.c_proj.weight, self.c_proj.bias)
            return residual + F.dropout(y, p, True)
        return Z.linear(y, self.c_proj.weight, self.c_proj.bias, residual=residual)


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, expansion: int = 4):
        super().__init__()
        self.c_fc = nn.Linear(cfg.emb_dim, expansion * cfg.emb_dim)
        self.c_proj = nn.Linear(expansion * cfg.emb_dim, cfg.emb_dim)
        self.dropout = cfg.dropout

    def forward(self, x, residual, cdrop=None):
        h = Z.linear(x, self.c_fc.weight, self.c_fc.bias, act="gelu_tanh")
        if self.training and self.dropout > 0.0:
            y = Z.linear(h, self.c_proj.weight, self.c_proj.bias)
            if cdrop is not None:
                return residual + _counter_dropout(y, self.dropout, cdrop[0], 3 + 3 * cdrop[1])
            return residual + F.dropout(y, self.dropout, True)
        return Z.linear(h, self.c_proj.weight, self.c_proj.bias, residual=residual)


class Block(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.ln_1 = LayerNorm(cfg.emb_dim, cfg.ln_bias)
        self.attn = Attention(cfg)
        self.ln_2 = LayerNorm(cfg.emb_dim, cfg.ln_bias)
        self.mlp = MLP(cfg)

    def forward(self, x, cdrop=None):
        x = self.attn(self.ln_1(x), x, cdrop)  # pre-norm; the residual add is fused into the projection
        x = self.mlp(self.ln_2(x), x, cdrop)
        return x


class Transformer(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.wte = nn.Embedding(cfg.vocab_size, cfg.emb_dim)
        self.wpe = nn.Embedding(cfg.block_size, cfg.emb_dim)
        self.h = nn.ModuleList([Block(cfg) for _ in range(cfg.num_layers)])
        self.ln_f = LayerNorm(cfg.emb_dim, cfg.ln_bias)


class GPT2(nn.Module):
    def __init__(self, config: ModelConfig):
        super().__init__()
        self.config = config
        self.transformer = Transformer(config)
        self.lm_head = nn.Linear(config.emb_dim, config.vocab_size, bias=False)
        self.lm_head.weight = self.transformer.wte.weight  # weight tying
        # None: torch's generator drives dropout. An integer: the counter-based masks of the fused
        # engine with that seed (GPT2TrainEngine.dropout_seed_of_micro_step gives the engine's).
        self.counter_dropout_seed: int | None = None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        std = 0.02
        for name, module in self.named_modules():
            if isinstance(module, nn.Linear):
                s = std
                if name.endswith("c_proj"):  # the two residual projections of every block
                    s /= (2 * self.config.num_layers) ** 0.5
                nn.init.normal_(module.weight, mean=0.0, std=s)
                if module.bias is not None:
                    nn.init.zeros_(module.bias)
            elif isinstance(module, nn.Embedding):
                nn.init.normal_(module.weight, mean=0.0, std=std)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def hidden(self, X: torch.Tensor) -> torch.Tensor:
        B, T = X.shape
        assert T <= self.config.block_size, "sequence longer than block_size"
        tr = self.transformer
        x = Z.embedding(X, tr.wte.weight, tr.wpe.weight)
        seed = self.counter_dropout_seed
        if self.training and self.config.dropout > 0.0:
            x = F.dropout(x, self.config.dropout, True) if seed is None else \
                _counter_dropout(x, self.config.dropout, seed, 0)
        for layer, block in enumerate(tr.h):
            x = block(x, None if seed is None else (seed, layer))
        return tr.ln_f(x)

    def forward(self, X: torch.Tensor, Y: torch.Tensor | None = None):
        x = self.hidden(X)
        if Y is None:
            logits = Z.linear(x[:, [-1], :], self.lm_head.weight)
            return logits, None
        logits = Z.linear(x, self.lm_head.weight)
        B, T, V = logits.shape
        loss = Z.cross_entropy(logits.view(B * T, V), Y.reshape(B * T))
        return logits, loss

    @torch.inference_mode()
    def generate(self, X: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
                 top_k: int | None = None, generator: torch.Generator | None = None):
        """Autoregressive sampling (nn/gpt2/modules.py:121-137): crop to block_size, scale the
        last-position logits by 1/temperature, optional top-k, softmax, multinomial."""
        from ..ops.sampling import sample_next

        for _ in range(max_new_tokens):
            ctx = X if X.size(1) <= self.config.block_size else X[:, -self.config.block_size:]
            logits, _ = self(ctx)
            nxt = sample_next(logits[:, -1, :].float(), temperature, top_k, generator)
            X = torch.cat((X, nxt), dim=1)
        return X
