"""`python -m zero_to_hero_b200.makemore.cli <model> [--names FILE]` with model in
bigram-count | bigram-nn | mlp-raw | mlp | backprop | wavenet."""
from __future__ import annotations

import argparse

import torch

from . import backprop, bigram, models, raw_mlp
from .data import CharCodec, build_dataset, load_names, split_names, synthetic_names


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("model", choices=["bigram-count", "bigram-nn", "mlp-raw", "mlp", "backprop", "wavenet"])
    ap.add_argument("--names", default="")
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--seed", type=int, default=42)
    a = ap.parse_args(argv)
    try:
        names = load_names(a.names or None)
    except FileNotFoundError:
        names = synthetic_names(4000, a.seed)
        print("names file not found: using a synthetic corpus")
    codec = CharCodec(names)
    g = torch.Generator().manual_seed(a.seed)
    if a.model == "bigram-count":
        counts = bigram.bigram_counts(names, codec)
        probs = bigram.bigram_probs(counts)
        print("samples:", bigram.sample_names(probs, codec, 8, g))
        print(f"avg nll {bigram.average_nll(names, bigram.bigram_probs(counts, 1), codec):.4f} (add-one smoothed)")
    elif a.model == "bigram-nn":
        W, losses = bigram.train_bigram_torch(names, codec, epochs=min(a.steps, 256))
        print(f"loss {losses[0]:.4f} -> {losses[-1]:.4f}")
    elif a.model == "backprop":
        X, Y = build_dataset(names, codec, 3)
        ix = torch.randint(0, X.shape[0], (32,), generator=g)
        for k, v in backprop.check(backprop.init_params(codec.size), X[ix], Y[ix]).items():
            print(f"{k:16s} max diff {v:.3e}")
    elif a.model == "mlp-raw":
        # bare tensors, hand-kept batch-norm running statistics, step-decay learning rate
        tr, va, _ = split_names(names, a.seed)
        Xtr, Ytr = build_dataset(tr, codec, 4)
        Xva, Yva = build_dataset(va, codec, 4)
        m = raw_mlp.init_raw_mlp(codec.size, 4, generator=g)
        losses = raw_mlp.train_raw_mlp(m, Xtr, Ytr, a.steps, generator=g)
        print(f"train loss {losses[0]:.4f} -> {sum(losses[-50:]) / 50:.4f}; "
              f"val {raw_mlp.evaluate_raw_mlp(m, Xva, Yva):.4f} (running statistics)")
        print("samples:", raw_mlp.sample_raw_mlp(m, codec, 4, 8, g))
    else:
        block = 4 if a.model == "mlp" else 8
        tr, va, _ = split_names(names, a.seed)
        Xtr, Ytr = build_dataset(tr, codec, block)
        Xva, Yva = build_dataset(va, codec, block)
        model = (models.build_mlp if a.model == "mlp" else models.build_wavenet)(codec.size, block, generator=g)
        losses = models.train_model(model, Xtr, Ytr, a.steps, generator=g)
        print(f"train loss {losses[0]:.4f} -> {sum(losses[-50:]) / 50:.4f}; val {models.evaluate(model, Xva, Yva):.4f}")
        print("samples:", models.sample(model, codec, block, 8, g))


if __name__ == "__main__":
    main()
