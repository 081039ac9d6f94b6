"""Model parity against the reference's own classes, loaded read-only from its tree (CPU)."""
import importlib.util

import pytest
import torch

from zero_to_hero_b200.config import ModelConfig
from zero_to_hero_b200.models.gpt import BigramLM, GPTLM, Vocab, causal_average_variants
from zero_to_hero_b200.models.gpt2 import GPT2
from zero_to_hero_b200.utils import checkpoint as ck


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def ref_gpt2(reference_root):
    return _load(reference_root / "nn" / "gpt2" / "modules.py", "ref_gpt2_modules")


@pytest.fixture(scope="module")
def ref_gpt(reference_root):
    return _load(reference_root / "nn" / "gpt" / "3_gpt.py", "ref_gpt_char")


def _pair(ref_gpt2, dropout=0.0):
    torch.manual_seed(0)
    rcfg = ref_gpt2.Config(vocab_size=97, block_size=32, emb_dim=48, num_heads=3, num_layers=2, dropout=dropout)
    r = ref_gpt2.GPT(rcfg)
    m = GPT2(ModelConfig(vocab_size=97, block_size=32, emb_dim=48, num_heads=3, num_layers=2, dropout=dropout))
    m.load_state_dict(ck.from_reference_state_dict(r.state_dict()))
    return r, m


def test_gpt2_logits_loss_grads_match_reference(ref_gpt2):
    r, m = _pair(ref_gpt2)
    X = torch.randint(0, 97, (4, 32))
    Y = torch.randint(0, 97, (4, 32))
    lr_, loss_r = r(X, Y)
    lm_, loss_m = m(X, Y)
    assert torch.allclose(lr_, lm_, atol=1e-5)
    assert loss_r.item() == pytest.approx(loss_m.item(), abs=1e-6)
    loss_r.backward()
    loss_m.backward()
    rg = ck.from_reference_state_dict({k: p.grad for k, p in r.named_parameters()})
    for k, p in m.named_parameters():
        assert torch.allclose(p.grad, rg[k], atol=2e-5), k
    # without targets only the last position goes through the head (nn/gpt2/modules.py:111-113)
    lo, none = m(X)
    assert none is None and lo.shape == (4, 1, 97)
    assert torch.allclose(lo, r(X)[0], atol=1e-5)


def test_gpt2_init_statistics():
    m = GPT2(ModelConfig(vocab_size=512, block_size=64, emb_dim=256, num_heads=4, num_layers=4))
    sd = m.state_dict()
    assert sd["transformer.h.0.attn.c_attn.weight"].std().item() == pytest.approx(0.02, rel=0.1)
    assert sd["transformer.h.0.mlp.c_proj.weight"].std().item() == pytest.approx(0.02 / 8 ** 0.5, rel=0.1)
    assert sd["transformer.h.0.attn.c_proj.bias"].abs().max().item() == 0.0
    assert m.lm_head.weight is m.transformer.wte.weight


def test_generate_matches_reference_token_for_token(ref_gpt2):
    r, m = _pair(ref_gpt2)
    r.eval(), m.eval()
    X = torch.randint(0, 97, (2, 5))
    torch.manual_seed(123)
    a = r.generate(X.clone(), 40, temperature=0.8, top_k=10)
    torch.manual_seed(123)
    b = m.generate(X.clone(), 40, temperature=0.8, top_k=10)
    assert torch.equal(a, b) and a.shape == (2, 45)


def test_state_dict_name_mapping_round_trip(ref_gpt2):
    r, m = _pair(ref_gpt2)
    back = ck.to_reference_state_dict(m.state_dict())
    assert set(back) == set(r.state_dict())
    hf = ck.to_hf_disk_format(m.state_dict())
    assert hf["transformer.h.0.attn.c_attn.weight"].shape == (48, 144)  # Conv1D is (in, out)
    assert "transformer.h.0.ln_1.bias" in hf
    again = ck.from_hf_disk_format(hf)
    for k, v in m.state_dict().items():
        assert torch.equal(again[k], v), k
    hf["transformer.ln_f.bias"] = torch.ones(48)
    with pytest.raises(ValueError):
        ck.from_hf_disk_format(hf)


def test_checkpoint_save_load(tmp_path, ref_gpt2):
    _, m = _pair(ref_gpt2)
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3)
    X = torch.randint(0, 97, (2, 16))
    m(X, X)[1].backward()
    opt.step()
    ck.save_checkpoint(tmp_path / "c.pt", m.state_dict(), opt.state_dict(), 7, {"cursor": 3}, {"a": 1})
    loaded = ck.load_checkpoint(tmp_path / "c.pt")
    assert loaded["step"] == 7 and loaded["data"] == {"cursor": 3}
    m2 = GPT2(m.config)
    m2.load_state_dict(loaded["model"])
    assert torch.allclose(m2(X)[0], m(X)[0])


def test_char_gpt_matches_reference(ref_gpt):
    torch.manual_seed(0)
    r = ref_gpt.GPTLM(65, 32, 48, 2, 3, 0.0)
    m = GPTLM(65, 32, 48, 2, 3, 0.0)
    m.load_reference_state_dict(r.state_dict())
    X = torch.randint(0, 65, (3, 32))
    Y = torch.randint(0, 65, (3, 32))
    a, la = r(X, Y)
    b, lb = m(X, Y)
    assert torch.allclose(a, b, atol=1e-5) and la.item() == pytest.approx(lb.item(), abs=1e-6)
    la.backward()
    lb.backward()
    rg = {k: p.grad for k, p in r.named_parameters()}
    for k, p in m.named_parameters():
        assert torch.allclose(p.grad, rg[k], atol=2e-5), k
    torch.manual_seed(5)
    ga = r.generate(X[:1, :4].clone(), 20)
    torch.manual_seed(5)
    gb = m.generate(X[:1, :4].clone(), 20)
    assert torch.equal(ga, gb)
    # the benchmark configuration of the char model: 10,788,929 parameters
    big = GPTLM(65, 256, 384, 6, 6, 0.2)
    assert sum(p.numel() for p in big.parameters()) == 10_788_929


def test_vocab_bigram_masking():
    v = Vocab("hello world")
    assert "".join(v.decode(v.encode("hello"))) == "hello" and v.size == 8
    b = BigramLM(v.size)
    X = torch.tensor([v.encode("hello worl")])
    Y = torch.tensor([v.encode("ello world")])
    logits, loss = b(X, Y)
    assert logits.shape == (1, 10, 8) and loss.item() > 0
    assert b.generate(X[:, :1], 5).shape == (1, 6)
    a, b2, c = causal_average_variants(torch.randn(2, 6, 3))
    assert torch.allclose(a, b2, atol=1e-6) and torch.allclose(a, c, atol=1e-6)


def test_counter_dropout_masks_are_deterministic_and_calibrated():
    """The host restatement of the kernels' dropout masks: reproducible, site-dependent, and with
    the requested drop rate (quantised to 1/256); the module can run with those masks on CPU."""
    import torch
    from zero_to_hero_b200.config import get_preset
    from zero_to_hero_b200.models.gpt2 import GPT2
    from zero_to_hero_b200.ops import dropout as D

    a = D.elementwise_keep(100_000, 0.2, 11, 3)
    assert torch.equal(a, D.elementwise_keep(100_000, 0.2, 11, 3))
    assert not torch.equal(a, D.elementwise_keep(100_000, 0.2, 11, 4))
    assert not torch.equal(a, D.elementwise_keep(100_000, 0.2, 12, 3))
    assert abs((1 - a.float().mean().item()) - 51 / 256) < 0.01
    m = D.attention_keep(2, 3, 50, 0.5, 7, 1)
    assert m.shape == (2, 3, 50, 50) and abs(m.float().mean().item() - 0.5) < 0.03
    assert D.threshold_and_scale(0.001) == (0, 1.0)  # below 1/512: nothing is dropped

    cfg = get_preset("gpt2-tiny").model
    cfg.dropout = 0.3
    torch.manual_seed(0)
    model = GPT2(cfg).train()
    X = torch.randint(0, cfg.vocab_size, (2, 16))
    model.counter_dropout_seed = 5
    l1 = model(X, X)[1].item()
    l2 = model(X, X)[1].item()
    model.counter_dropout_seed = 6
    l3 = model(X, X)[1].item()
    assert l1 == l2 and l1 != l3
