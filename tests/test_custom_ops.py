"""The `z2h` custom operators: CPU kernels against PyTorch, autograd of layernorm_linear, and
(on a GPU) the CUDA kernels against the CPU kernels."""
import pytest
import torch
import torch.nn.functional as F

import zero_to_hero_b200.ops.custom_ops  # noqa: F401  (registers torch.ops.z2h.*)

ops = torch.ops.z2h


def _cases():
    torch.manual_seed(0)
    x, k = torch.arange(15.0), torch.arange(4.0)
    B, S, H, O = 4, 4, 8, 16
    return dict(conv=(x, k), sm=(torch.randn(128),), att=(torch.randn(16), torch.randn(16, 16), torch.randn(16, 16)),
                emb=(torch.randint(0, 100, (8, 32)), torch.randn(100, 64)),
                lnl=(torch.randn(B, S, H), torch.rand(H) + 0.5, torch.randn(H), torch.randn(O, H), torch.randn(O)))


def test_cpu_kernels_match_pytorch():
    c = _cases()
    x, k = c["conv"]
    ref = torch.stack([(torch.cat([x, torch.zeros(3)])[i:i + 4] * k).sum() for i in range(15)])
    assert torch.allclose(ops.conv1d(x, k), ref)
    assert torch.allclose(ops.softmax(*c["sm"]), torch.softmax(c["sm"][0], 0), atol=1e-6)
    q, kk, v = c["att"]
    assert torch.allclose(ops.attention(q, kk, v), torch.softmax(kk @ q, 0) @ v, atol=1e-6)
    idx, w = c["emb"]
    assert torch.equal(ops.embedding(idx, w), w[idx])
    xx, g, b, W, bias = c["lnl"]
    assert torch.allclose(ops.layernorm_linear(xx, g, b, W, bias), F.linear(F.layer_norm(xx, (8,), g, b), W, bias), atol=1e-5)


def test_layernorm_linear_autograd_cpu():
    xx, g, b, W, bias = [t.clone().requires_grad_(True) for t in _cases()["lnl"]]
    ref_in = [t.detach().clone().requires_grad_(True) for t in (xx, g, b, W, bias)]
    dy = torch.randn(4, 4, 16)
    ops.layernorm_linear(xx, g, b, W, bias).backward(dy)
    F.linear(F.layer_norm(ref_in[0], (8,), ref_in[1], ref_in[2]), ref_in[3], ref_in[4]).backward(dy)
    for a, r in zip((xx, g, b, W, bias), ref_in):
        assert torch.allclose(a.grad, r.grad, atol=1e-4)


def test_ops_pass_opcheck_on_cpu():
    c = _cases()
    torch.library.opcheck(ops.conv1d.default, c["conv"], test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(ops.layernorm_linear.default, c["lnl"], test_utils=("test_schema", "test_faketensor"))


@pytest.mark.gpu
def test_cuda_kernels_match_cpu_kernels():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    c = _cases()
    for name, op in [("conv", ops.conv1d), ("sm", ops.softmax), ("att", ops.attention), ("emb", ops.embedding),
                     ("lnl", ops.layernorm_linear)]:
        cpu = op(*c[name])
        gpu = op(*[t.cuda() for t in c[name]])
        assert torch.allclose(gpu.cpu(), cpu, atol=1e-4), name
    xx, g, b, W, bias = [t.cuda().requires_grad_(True) for t in c["lnl"]]
    dy = torch.randn(4, 4, 16)
    ops.layernorm_linear(xx, g, b, W, bias).backward(dy.cuda())
    ref = [t.clone().requires_grad_(True) for t in c["lnl"]]
    ops.layernorm_linear(*ref).backward(dy)
    for a, r in zip((xx, g, b, W, bias), ref):
        assert torch.allclose(a.grad.cpu(), r.grad, atol=1e-4)
