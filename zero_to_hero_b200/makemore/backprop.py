"""Back-propagation by hand through a one-hidden-layer MLP with batch norm, checked against
autograd (nn/makemore/3_1_backprop.py of the reference): the forward pass is split into atomic
steps, every intermediate gets a hand-derived gradient, and two fused shortcuts (softmax
cross-entropy, batch norm with Bessel's correction) are derived as single expressions."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def init_params(vocab: int, block_size: int = 3, emb: int = 10, hidden: int = 64, seed: int = 2147483647):
    g = torch.Generator().manual_seed(seed)
    p = {
        "C": torch.randn(vocab, emb, generator=g),
        "W1": torch.randn(emb * block_size, hidden, generator=g) * (5 / 3) / (emb * block_size) ** 0.5,
        "b1": torch.randn(hidden, generator=g) * 0.1,
        "W2": torch.randn(hidden, vocab, generator=g) * 0.1,
        "b2": torch.randn(vocab, generator=g) * 0.1,
        "bngain": torch.randn(1, hidden, generator=g) * 0.1 + 1.0,
        "bnbias": torch.randn(1, hidden, generator=g) * 0.1,
    }
    for t in p.values():
        t.requires_grad_(True)
    return p


def forward_atomic(p, Xb, Yb):
    """Forward pass in atomic steps; returns (loss, dict of every intermediate)."""
    n = Xb.shape[0]
    t = {}
    t["emb"] = p["C"][Xb]
    t["embcat"] = t["emb"].view(n, -1)
    t["hprebn"] = t["embcat"] @ p["W1"] + p["b1"]
    t["bnmeani"] = t["hprebn"].sum(0, keepdim=True) / n
    t["bndiff"] = t["hprebn"] - t["bnmeani"]
    t["bndiff2"] = t["bndiff"] ** 2
    t["bnvar"] = t["bndiff2"].sum(0, keepdim=True) / (n - 1)
    t["bnvar_inv"] = (t["bnvar"] + 1e-5) ** -0.5
    t["bnraw"] = t["bndiff"] * t["bnvar_inv"]
    t["hpreact"] = p["bngain"] * t["bnraw"] + p["bnbias"]
    t["h"] = torch.tanh(t["hpreact"])
    t["logits"] = t["h"] @ p["W2"] + p["b2"]
    t["logit_maxes"] = t["logits"].max(1, keepdim=True).values
    t["norm_logits"] = t["logits"] - t["logit_maxes"]
    t["counts"] = t["norm_logits"].exp()
    t["counts_sum"] = t["counts"].sum(1, keepdim=True)
    t["counts_sum_inv"] = t["counts_sum"] ** -1
    t["probs"] = t["counts"] * t["counts_sum_inv"]
    t["logprobs"] = t["probs"].log()
    loss = -t["logprobs"][range(n), Yb].mean()
    return loss, t


@torch.no_grad()
def manual_backward(p, t, Xb, Yb) -> dict[str, torch.Tensor]:
    """Hand-derived gradient of the loss w.r.t. every intermediate and parameter."""
    n = Xb.shape[0]
    d = {}
    d["logprobs"] = -F.one_hot(Yb, t["logprobs"].shape[1]).float() / n
    d["probs"] = d["logprobs"] / t["probs"]
    d["counts_sum_inv"] = (t["counts"] * d["probs"]).sum(1, keepdim=True)
    d["counts_sum"] = -t["counts_sum"] ** -2 * d["counts_sum_inv"]
    d["counts"] = t["counts_sum_inv"] * d["probs"] + d["counts_sum"]
    d["norm_logits"] = t["counts"] * d["counts"]
    d["logit_maxes"] = -d["norm_logits"].sum(1, keepdim=True)
    d["logits"] = d["norm_logits"] + F.one_hot(t["logits"].max(1).indices, t["logits"].shape[1]) * d["logit_maxes"]
    d["h"] = d["logits"] @ p["W2"].T
    d["W2"] = t["h"].T @ d["logits"]
    d["b2"] = d["logits"].sum(0)
    d["hpreact"] = (1 - t["h"] ** 2) * d["h"]
    d["bngain"] = (t["bnraw"] * d["hpreact"]).sum(0, keepdim=True)
    d["bnraw"] = p["bngain"] * d["hpreact"]
    d["bnbias"] = d["hpreact"].sum(0, keepdim=True)
    d["bnvar_inv"] = (t["bndiff"] * d["bnraw"]).sum(0, keepdim=True)
    d["bnvar"] = -0.5 * (t["bnvar"] + 1e-5) ** -1.5 * d["bnvar_inv"]
    d["bndiff2"] = torch.ones_like(t["bndiff2"]) / (n - 1) * d["bnvar"]
    d["bndiff"] = t["bnvar_inv"] * d["bnraw"] + 2 * t["bndiff"] * d["bndiff2"]
    d["bnmeani"] = -d["bndiff"].sum(0, keepdim=True)
    d["hprebn"] = d["bndiff"] + d["bnmeani"] / n
    d["embcat"] = d["hprebn"] @ p["W1"].T
    d["W1"] = t["embcat"].T @ d["hprebn"]
    d["b1"] = d["hprebn"].sum(0)
    d["emb"] = d["embcat"].view(t["emb"].shape)
    d["C"] = torch.zeros_like(p["C"]).index_add_(0, Xb.view(-1), d["emb"].view(-1, d["emb"].shape[-1]))
    return d


@torch.no_grad()
def fused_cross_entropy_backward(logits, Yb):
    """d loss / d logits in one expression: (softmax - onehot) / n."""
    n = logits.shape[0]
    d = F.softmax(logits, 1)
    d[range(n), Yb] -= 1
    return d / n


@torch.no_grad()
def fused_batchnorm_backward(dhpreact, bngain, bnvar_inv, bnraw):
    """d loss / d hprebn through batch norm with the (n-1) variance, in one expression."""
    n = dhpreact.shape[0]
    return bngain * bnvar_inv / n * (n * dhpreact - dhpreact.sum(0) - n / (n - 1) * bnraw * (dhpreact * bnraw).sum(0))


def check(p, Xb, Yb) -> dict[str, float]:
    """Max abs difference between every manual gradient and autograd's."""
    for v in p.values():
        v.grad = None
    loss, t = forward_atomic(p, Xb, Yb)
    for v in t.values():
        v.retain_grad()
    loss.backward()
    d = manual_backward(p, t, Xb, Yb)
    out = {}
    for k, g in d.items():
        ref = (p[k] if k in p else t[k]).grad
        out[k] = float((g - ref).abs().max())
    out["fused_ce"] = float((fused_cross_entropy_backward(t["logits"].detach(), Yb) - t["logits"].grad).abs().max())
    out["fused_bn"] = float((fused_batchnorm_backward(t["hpreact"].grad, p["bngain"].detach(), t["bnvar_inv"].detach(),
                                                      t["bnraw"].detach()) - t["hprebn"].grad).abs().max())
    return out
