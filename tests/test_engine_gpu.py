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
