"""makemore: bigram models agree with each other, the module system trains, every hand-derived
gradient matches autograd (CPU)."""
import math

import pytest
import torch

from zero_to_hero_b200.makemore import backprop, bigram, models
from zero_to_hero_b200.makemore.data import CharCodec, build_dataset, split_names, synthetic_names
from zero_to_hero_b200.makemore.layers import BatchNorm1d, FlattenConsecutive, Linear, Sequential, Tanh


@pytest.fixture(scope="module")
def corpus():
    names = synthetic_names(1500, seed=1)
    return names, CharCodec(names)


def test_dataset_windows(corpus):
    names, codec = corpus
    X, Y = build_dataset(["ab"], CharCodec(["ab"]), 3)
    assert X.tolist() == [[0, 0, 0], [0, 0, 1], [0, 1, 2]] and Y.tolist() == [1, 2, 0]
    tr, va, te = split_names(names)
    assert len(tr) + len(va) + len(te) == len(names) and len(tr) == 1200


def test_bigram_count_model(corpus):
    names, codec = corpus
    counts = bigram.bigram_counts(names, codec)
    assert int(counts.sum()) == sum(len(n) + 1 for n in names)
    probs = bigram.bigram_probs(counts)
    assert torch.allclose(probs.sum(1)[counts.sum(1) > 0], torch.ones(1))
    nll = bigram.average_nll(names, bigram.bigram_probs(counts, 1), codec)
    assert 1.0 < nll < math.log(codec.size)
    out = bigram.sample_names(probs, codec, 5, torch.Generator().manual_seed(0))
    assert len(out) == 5 and all(isinstance(s, str) for s in out)


def test_bigram_network_approaches_count_model(corpus):
    names, codec = corpus
    target = bigram.average_nll(names, bigram.bigram_probs(bigram.bigram_counts(names, codec), 1), codec)
    W, losses = bigram.train_bigram_torch(names, codec, epochs=200, lr=50.0)
    assert losses[-1] < losses[0] and losses[-1] < target + 0.15


def test_bigram_micrograd_matches_torch_gradient_step():
    names = ["ab", "ba"]
    codec = CharCodec(names)
    W, losses = bigram.train_bigram_micrograd(names, codec, epochs=3, lr=1.0, seed=0)
    assert losses[-1] < losses[0]


def test_layers_and_module_registry():
    g = torch.Generator().manual_seed(0)
    net = Sequential(Linear(6, 8, bias=False, generator=g), BatchNorm1d(8), Tanh(), Linear(8, 3, generator=g))
    assert len(net.parameters()) == 1 + 2 + 2
    x = torch.randn(16, 6, generator=g)
    y = net(x)
    assert y.shape == (16, 3)
    bn = net.layers[1]
    assert not torch.allclose(bn.running_mean, torch.zeros(8))  # updated in training mode
    net.eval()
    assert net.layers[1].training is False and net(x[:1]).shape == (1, 3)  # running stats: batch of 1 is fine
    f = FlattenConsecutive(2)
    assert f(torch.zeros(4, 8, 10)).shape == (4, 4, 20) and f(torch.zeros(4, 2, 10)).shape == (4, 20)
    bn3 = BatchNorm1d(5)
    out = bn3(torch.randn(7, 3, 5))
    assert out.shape == (7, 3, 5) and out.mean((0, 1)).abs().max() < 1e-5


@pytest.mark.parametrize("kind", ["mlp", "wavenet"])
def test_models_train(corpus, kind):
    names, codec = corpus
    block = 4 if kind == "mlp" else 8
    g = torch.Generator().manual_seed(0)
    X, Y = build_dataset(names, codec, block)
    build = models.build_mlp if kind == "mlp" else models.build_wavenet
    model = build(codec.size, block, hidden=64, generator=g) if kind == "wavenet" else build(codec.size, block, hidden=64, depth=2, generator=g)
    first = models.evaluate(model, X[:2000], Y[:2000])
    assert first == pytest.approx(math.log(codec.size), abs=0.5)  # calibrated initial loss
    models.train_model(model, X, Y, steps=300, batch_size=64, lr=0.1, generator=g)
    assert models.evaluate(model, X[:2000], Y[:2000]) < first - 0.5
    assert len(models.sample(model, codec, block, 3, g)) == 3


def test_manual_backprop_matches_autograd(corpus):
    names, codec = corpus
    X, Y = build_dataset(names, codec, 3)
    g = torch.Generator().manual_seed(0)
    ix = torch.randint(0, X.shape[0], (32,), generator=g)
    diffs = backprop.check(backprop.init_params(codec.size), X[ix], Y[ix])
    assert set(diffs) >= {"logits", "W1", "C", "bnvar", "fused_ce", "fused_bn"}
    assert max(diffs.values()) < 1e-6, diffs


def test_raw_tensor_mlp_with_hand_kept_batchnorm_statistics(corpus):
    """The bare-tensor MLP (nn/makemore/2_1_mlp.py): running statistics follow the batches with
    momentum 0.1 and biased variance, evaluation uses them instead of batch statistics, the
    step-decay schedule divides by the LAST divisor passed, and SGD by hand learns."""
    from zero_to_hero_b200.makemore import raw_mlp as R

    names, codec = corpus
    X, Y = build_dataset(names, codec, 4)
    g = torch.Generator().manual_seed(24)
    m = R.init_raw_mlp(codec.size, 4, emb_dim=8, hidden=32, generator=g)
    # one training forward: running stats move a tenth of the way to the batch statistics
    pre = (m.emb[X[:64]].flatten(1) @ m.w1 + m.b1).detach()
    R.forward(m, X[:64], True)
    assert torch.allclose(m.running_mean, 0.1 * pre.mean(0, keepdim=True), atol=1e-6)
    assert torch.allclose(m.running_var, 0.9 + 0.1 * pre.var(0, keepdim=True, unbiased=False), atol=1e-6)
    before = (m.running_mean.clone(), m.running_var.clone())
    a = R.forward(m, X[:7], False)
    b = R.forward(m, X[:7], False)
    assert torch.equal(a, b) and torch.equal(m.running_mean, before[0])   # eval: no update, no batch stats
    assert not torch.allclose(R.forward(m, X[:7], True), a)
    # schedule: 0.16 until 68 % of the run, then 0.04; later points (same divisor) change nothing
    assert R.step_decay_lr(0, 1000, 0.16) == 0.16 and R.step_decay_lr(679, 1000, 0.16) == 0.16
    assert R.step_decay_lr(680, 1000, 0.16) == 0.04 and R.step_decay_lr(999, 1000, 0.16) == 0.04
    assert R.step_decay_lr(900, 1000, 1.0, (0.5, 0.8), (2, 10)) == 0.1
    first = R.evaluate_raw_mlp(m, X[:2000], Y[:2000])
    losses = R.train_raw_mlp(m, X, Y, steps=400, batch_size=64, lr=0.16, generator=g)
    assert len(losses) == 400 and R.evaluate_raw_mlp(m, X[:2000], Y[:2000]) < first - 0.4
    assert len(R.sample_raw_mlp(m, codec, 4, 3, g)) == 3
