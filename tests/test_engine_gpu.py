"""The fused engine against the PyTorch module trained on CPU in fp32 with the same data."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg():
    from zero_to_hero_b200.config import get_preset
    cfg = get_preset("gpt2-tiny")
    cfg.model.emb_dim, cfg.model.num_heads, cfg.model.num_layers = 256, 4, 3
    cfg.model.vocab_size, cfg.model.block_size = 1000, 256
    cfg.train.micro_batch = 4
    cfg.optim.warmup_steps, cfg.optim.schedule, cfg.optim.lr_max = 0, "constant", 1e-3
    return cfg


def _batches(g, n=2):
    out = []
    for _ in range(n):
        tok = torch.randint(0, 1000, (4 * 256 + 1,), generator=g)
        out.append((tok[:-1].view(4, 256).pin_memory(), tok[1:].view(4, 256).pin_memory()))
    return out


@pytest.mark.parametrize("graph,overlap", [(False, False), (True, False), (False, True), (True, True)])
def test_engine_tracks_fp32_reference_training(graph, overlap):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.engine import GPT2TrainEngine
    from zero_to_hero_b200.models.gpt2 import GPT2
    from zero_to_hero_b200.ops import _lib
    from zero_to_hero_b200.optim.adamw import build_optimizer

    cfg = _cfg()
    cfg.train.use_cuda_graph = graph
    cfg.train.overlap_wgrad = overlap  # weight gradients on a second stream
    eng = GPT2TrainEngine(cfg, "cuda", seed=1)
    ref = GPT2(cfg.model).float()
    ref.load_state_dict({k: v.cpu() for k, v in eng.state_dict().items()})
    opt = build_optimizer(ref, cfg.optim, "cpu")
    g = torch.Generator().manual_seed(0)
    for step in range(3):
        batches = _batches(g)
        eng.train_step(batches, lr=1e-3)
        loss_e, gn_e = eng.read_loss(), eng.read_grad_norm()
        opt.zero_grad()
        loss_r = 0.0
        for X, Y in batches:
            _, l = ref(X, Y)
            (l / 2).backward()
            loss_r += l.item() / 2
        gn_r = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0).item()
        opt.step()
        assert loss_e == pytest.approx(loss_r, abs=5e-3)
        assert gn_e == pytest.approx(gn_r, rel=2e-2)
        sd, rsd = eng.state_dict(), ref.state_dict()
        # AdamW's first steps move every weight by ~lr regardless of gradient size, so a
        # bf16-level sign disagreement on a tiny gradient costs at most 2 * lr per step
        assert max((sd[k].cpu() - rsd[k]).abs().max().item() for k in rsd) < 2.5e-3 * (step + 1)
    _lib.check_status()
    assert eng.kernel_launches_per_step(2) > 100


def test_module_path_uses_native_kernels_and_matches_cpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.models.gpt2 import GPT2
    from zero_to_hero_b200.ops.functional import FALLBACK_COUNTS

    cfg = _cfg()
    torch.manual_seed(0)
    cpu = GPT2(cfg.model).float()
    gpu = GPT2(cfg.model).float().cuda()
    gpu.load_state_dict(cpu.state_dict())
    X = torch.randint(0, 1000, (2, 256))
    Y = torch.randint(0, 1000, (2, 256))
    FALLBACK_COUNTS.clear()
    lg, loss_g = gpu(X.cuda(), Y.cuda())
    loss_g.backward()
    lc, loss_c = cpu(X, Y)
    loss_c.backward()
    assert not FALLBACK_COUNTS, dict(FALLBACK_COUNTS)
    assert loss_g.item() == pytest.approx(loss_c.item(), abs=5e-3)
    for (k, p), q in zip(gpu.named_parameters(), cpu.parameters()):
        scale = q.grad.abs().max().item() + 1e-9
        assert (p.grad.cpu() - q.grad).abs().max().item() / scale < 3e-2, k
    out = gpu.generate(X[:, :8].cuda(), 8, top_k=5)
    assert out.shape == (2, 16)


def test_engine_checkpoint_round_trip(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.engine import GPT2TrainEngine, load_engine_checkpoint, save_engine_checkpoint

    cfg = _cfg()
    g = torch.Generator().manual_seed(0)
    a = GPT2TrainEngine(cfg, "cuda", seed=3)
    a.train_step(_batches(g), lr=1e-3)
    save_engine_checkpoint(a, tmp_path / "e.pt")
    b = GPT2TrainEngine(cfg, "cuda", seed=99)
    load_engine_checkpoint(b, tmp_path / "e.pt")
    nxt = _batches(g)
    a.train_step(nxt, lr=1e-3)
    b.train_step(nxt, lr=1e-3)
    assert a.read_loss() == pytest.approx(b.read_loss(), abs=1e-4)
    assert torch.allclose(a.p32, b.p32, atol=1e-6)


def test_engine_with_dropout_tracks_module_with_the_same_masks():
    """Dropout 0.2 at all four sites of the reference model: the engine's counter-based masks are
    restated on the host, so the fp32 PyTorch module can replay the very same masks."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.engine import GPT2TrainEngine
    from zero_to_hero_b200.models.gpt2 import GPT2
    from zero_to_hero_b200.ops import _lib
    from zero_to_hero_b200.optim.adamw import build_optimizer

    cfg = _cfg()
    cfg.model.dropout = 0.2
    cfg.model.num_layers = 2
    eng = GPT2TrainEngine(cfg, "cuda", seed=3)
    ref = GPT2(cfg.model).float().train()
    ref.load_state_dict({k: v.cpu() for k, v in eng.state_dict().items()})
    opt = build_optimizer(ref, cfg.optim, "cpu")
    g = torch.Generator().manual_seed(0)
    k = 0
    for step in range(2):
        batches = _batches(g)
        eng.train_step(batches, lr=1e-3)
        loss_e, gn_e = eng.read_loss(), eng.read_grad_norm()
        opt.zero_grad()
        loss_r = 0.0
        for X, Y in batches:
            k += 1
            ref.counter_dropout_seed = eng.dropout_seed_of_micro_step(k)
            _, l = ref(X, Y)
            (l / 2).backward()
            loss_r += l.item() / 2
        gn_r = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0).item()
        opt.step()
        assert loss_e == pytest.approx(loss_r, abs=1e-2)
        assert gn_e == pytest.approx(gn_r, rel=3e-2)
    # a run without dropout gives a different loss: the masks really are applied
    cfg0 = _cfg()
    cfg0.model.num_layers = 2
    eng0 = GPT2TrainEngine(cfg0, "cuda", seed=3)
    eng0.train_step(_batches(torch.Generator().manual_seed(0)), lr=1e-3)
    eng1 = GPT2TrainEngine(cfg, "cuda", seed=3)
    eng1.train_step(_batches(torch.Generator().manual_seed(0)), lr=1e-3)
    assert abs(eng0.read_loss() - eng1.read_loss()) > 1e-3
    _lib.check_status()


def test_eval_path_is_forward_only_and_leaves_training_alone():
    """Validation through the engine: dropout off, matches the fp32 module in eval mode, and the
    gradients, dropout seed, micro-step counter and training graph are untouched by it."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.engine import GPT2TrainEngine
    from zero_to_hero_b200.models.gpt2 import GPT2

    cfg = _cfg()
    cfg.model.dropout = 0.2
    cfg.model.num_layers = 2
    eng = GPT2TrainEngine(cfg, "cuda", seed=5)
    ref = GPT2(cfg.model).float().eval()
    ref.load_state_dict({k: v.cpu() for k, v in eng.state_dict().items()})
    g = torch.Generator().manual_seed(0)
    (X, Y), = _batches(g, 1)
    with torch.no_grad():
        _, want = ref(X, Y)
    # accumulate half a step, evaluate in the middle, finish the step
    b = _batches(g, 2)
    eng.loss_accum.zero_()
    eng.micro_step(*b[0], 2)
    g_before = eng.g.clone()
    seed_before, n_before = int(eng.drop_seed.item()), eng.micro_steps_done
    graphs_before = dict(eng._graphs)
    got = eng.eval_loss(X, Y)
    got2 = eng.eval_loss(X, Y)          # second call replays the captured forward-only graph
    assert got == pytest.approx(want.item(), abs=5e-3) and got2 == pytest.approx(got, abs=1e-6)
    assert torch.equal(eng.g, g_before)
    assert int(eng.drop_seed.item()) == seed_before and eng.micro_steps_done == n_before
    assert eng._graphs == graphs_before and len(eng._eval_graphs) == 1
    # a smaller batch shape (the (4, 256) of the multiple-choice evaluation is the engine's own
    # here, so take (2, 128)): per-token losses against the module
    Xs, Ys = X[:2, :128].contiguous(), Y[:2, :128].contiguous()
    with torch.no_grad():
        logits, _ = ref(Xs, Ys)
    want_tok = torch.nn.functional.cross_entropy(logits.view(-1, logits.size(-1)), Ys.view(-1),
                                                 reduction="none").view(2, 128)
    got_tok = eng.eval_losses(Xs, Ys).cpu()
    assert (got_tok - want_tok).abs().max().item() < 3e-2
    eng.micro_step(*b[1], 2, last=True)
    eng.optimizer_step(1e-3)
    assert eng.read_loss() == eng.read_loss()


def test_hellaswag_through_engine_matches_module():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.engine import GPT2TrainEngine
    from zero_to_hero_b200.eval.hellaswag import evaluate, evaluate_losses_fn
    from zero_to_hero_b200.models.gpt2 import GPT2

    cfg = _cfg()
    cfg.model.num_layers = 2
    eng = GPT2TrainEngine(cfg, "cuda", seed=11)
    ref = GPT2(cfg.model).float().eval()
    ref.load_state_dict({k: v.cpu() for k, v in eng.state_dict().items()})
    g = torch.Generator().manual_seed(4)
    examples = []
    for i in range(6):
        ctx = torch.randint(0, 1000, (int(torch.randint(5, 40, (1,), generator=g)),), generator=g).tolist()
        ends = [torch.randint(0, 1000, (int(torch.randint(3, 20, (1,), generator=g)),), generator=g).tolist()
                for _ in range(4)]
        examples.append({"ctx_tokens": ctx, "ending_tokens": ends, "label": i % 4})
    c_ref, n_ref = evaluate(ref, examples, "cpu", cfg.model.block_size)
    c_eng, n_eng = evaluate_losses_fn(eng.eval_losses, examples, eng.device, cfg.model.block_size)
    assert int(n_ref) == int(n_eng) == 6
    # random weights score at chance; what must agree is WHICH ending each model prefers, up to
    # bf16-level ties: allow one example of six to differ
    assert abs(int(c_ref) - int(c_eng)) <= 1
    # rank-strided sharding covers every example exactly once
    parts = [evaluate_losses_fn(eng.eval_losses, examples, eng.device, cfg.model.block_size, r, 3)
             for r in range(3)]
    assert sum(int(n) for _, n in parts) == 6 and sum(int(c) for c, _ in parts) == int(c_eng)


def test_hyper_parameters_survive_a_host_that_runs_ahead():
    """Several optimizer steps queued without any host sync, each with its own learning rate:
    every step must see its own value (staging ring), i.e. the result equals a run that
    synchronises after every step."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.engine import GPT2TrainEngine

    cfg = _cfg()
    cfg.model.num_layers = 2
    lrs = [1e-3, 5e-5, 2e-3, 1e-5, 7e-4, 3e-3, 1e-4, 9e-4, 2e-4, 4e-3, 6e-5, 8e-4]
    finals = []
    for sync in (False, True):
        eng = GPT2TrainEngine(cfg, "cuda", seed=2)
        g = torch.Generator().manual_seed(0)
        data = [_batches(g, 1) for _ in lrs]
        dev = [[(x.cuda(), y.cuda()) for x, y in b] for b in data]
        torch.cuda.synchronize()
        for b, lr in zip(dev, lrs):
            eng.train_step(b, lr=lr)
            if sync:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        finals.append(eng.p32.clone())
    # the step itself is reproducible only up to the order of its atomic accumulations, so the two
    # runs are compared on average: a step that saw a neighbour's learning rate (they differ by up
    # to 100x here) would move EVERY weight by about that difference, ~1e-3
    assert (finals[0] - finals[1]).abs().mean().item() < 2e-5


def test_checkpoint_restores_dropout_counters_and_rank_state(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.engine import (GPT2TrainEngine, load_engine_checkpoint, save_engine_checkpoint,
                                          select_rank_state)

    cfg = _cfg()
    cfg.model.dropout = 0.1
    cfg.model.num_layers = 2
    g = torch.Generator().manual_seed(0)
    a = GPT2TrainEngine(cfg, "cuda", seed=3)
    a.train_step(_batches(g), lr=1e-3)
    save_engine_checkpoint(a, tmp_path / "d.pt", {"cursor": 123})
    b = GPT2TrainEngine(cfg, "cuda", seed=3)
    ck = load_engine_checkpoint(b, tmp_path / "d.pt")
    assert ck["data"] == {"cursor": 123}
    assert int(b.drop_seed.item()) == int(a.drop_seed.item()) and b.micro_steps_done == a.micro_steps_done == 2
    nxt = _batches(g)
    a.train_step(nxt, lr=1e-3)
    b.train_step(nxt, lr=1e-3)
    assert a.read_loss() == pytest.approx(b.read_loss(), abs=1e-4)   # same masks after the restore
    with pytest.raises(ValueError):
        select_rank_state({"world": 2, "per_rank": [1, 2]}, 0, 4)
    assert select_rank_state({"world": 2, "per_rank": ["r0", "r1"]}, 1, 2) == "r1"


def test_train_loop_with_eval_hellaswag_checkpoint_and_resume(tmp_path):
    """The trainer end to end on one GPU: fused engine, forward-only validation, HellaSwag scoring
    through the engine, JSONL log, a checkpoint, and a resume that continues from it."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import json

    from zero_to_hero_b200.config import get_preset
    from zero_to_hero_b200.train import train

    g = torch.Generator().manual_seed(0)
    examples = []
    for i in range(3):
        ctx = torch.randint(0, 500, (10 + i,), generator=g).tolist()
        ends = [torch.randint(0, 500, (4 + j,), generator=g).tolist() for j in range(4)]
        examples.append({"ctx_tokens": ctx, "ending_tokens": ends, "label": i})
    hs = tmp_path / "hs.jsonl"
    hs.write_text("\n".join(json.dumps(e) for e in examples))

    def cfg(steps):
        c = get_preset("gpt2-tiny")
        c.model.block_size = 256          # the multiple-choice batches are (4, 256)
        c.train.micro_batch, c.train.total_batch_tokens = 4, 4 * 256 * 2
        c.train.steps, c.train.eval_interval, c.train.eval_batches = steps, 1, 1
        c.train.hellaswag = str(hs)
        c.train.checkpoint_dir, c.train.checkpoint_interval = str(tmp_path / "ck"), 2
        c.train.log_jsonl = str(tmp_path / f"log{steps}.jsonl")
        return c

    out = train(cfg(3))
    hist = out["history"]
    assert len(hist) == 3 and all(h["train"] == h["train"] for h in hist)
    assert all("val" in h and 0.0 <= h["hellaswag"] <= 1.0 for h in hist)
    assert hist[-1]["train"] < hist[0]["train"] + 0.5
    ck = tmp_path / "ck" / "step00000002.pt"
    assert ck.exists()
    lines = [json.loads(l) for l in (tmp_path / "log3.jsonl").read_text().splitlines()]
    assert len(lines) == 3 and "tok_s" in lines[0]
    resumed = train(cfg(4), resume=str(ck))
    assert [h["step"] for h in resumed["history"]] == [2, 3]
    # step 2 of the resumed run repeats step 2 of the first run (same weights, moments, data cursor)
    assert resumed["history"][0]["train"] == pytest.approx(hist[2]["train"], abs=2e-3)


@pytest.mark.parametrize("dropout", [0.0, 0.1])
def test_deterministic_mode_repeats_training_bit_for_bit(dropout):
    """`train.deterministic=true`: two engines from the same seed on the same batches end three steps
    with bitwise equal master weights, moments, losses and gradient norms (weight gradients without
    split-K, dQ accumulated one KV tile per launch, bias and embedding gradients by single writers),
    and they track the default mode's result to rounding."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.engine import GPT2TrainEngine
    from zero_to_hero_b200.ops import _lib

    def run(deterministic):
        cfg = _cfg()
        cfg.model.dropout = dropout
        cfg.train.deterministic = deterministic
        eng = GPT2TrainEngine(cfg, "cuda", seed=3)
        g = torch.Generator().manual_seed(5)
        losses = []
        for _ in range(3):
            eng.train_step(_batches(g), lr=1e-3)
            losses.append((eng.read_loss(), eng.read_grad_norm()))
        return eng.p32.clone(), eng.m.clone(), eng.v.clone(), losses

    a, b, plain = run(True), run(True), run(False)
    assert a[3] == b[3]
    for x, y in zip(a[:3], b[:3]):
        assert torch.equal(x, y)
    # same mathematics as the default mode
    assert a[3][-1][0] == pytest.approx(plain[3][-1][0], abs=2e-3)
    assert (a[0] - plain[0]).abs().max().item() < 2.5e-3 * 3
    _lib.check_status()
