"""The teaching primitives against CPU oracles, on the shapes the reference's puzzles use and on
larger / ragged ones."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def P():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.ops import primitives
    torch.manual_seed(0)
    return primitives


def cu(x):
    return x.float().cuda()


def close(a, b, tol=1e-5):
    a, b = a.float().cpu(), b.float().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    assert torch.allclose(a, b, atol=tol, rtol=tol), (a - b).abs().max()


def test_maps_and_indexing(P):
    a = torch.arange(4.0)
    close(P.add10(cu(a), block=4), a + 10)
    close(P.zip_add(cu(a), cu(a * 2), block=4), a * 3)
    close(P.add10(cu(torch.arange(9.0)), block=4), torch.arange(9.0) + 10)  # 3 blocks of 4, n = 9
    big = torch.randn(1_000_003)
    close(P.add10(cu(big), vectorized=True), big + 10)
    m = torch.arange(25.0).view(5, 5)
    close(P.add10_2d(cu(m), block=(3, 3)), m + 10)
    close(P.broadcast_add(cu(torch.arange(2.0)), cu(torch.arange(2.0) * 10)), torch.tensor([[0., 1.], [10., 11.]]))
    close(P.add10_shared(cu(torch.ones(8)), block=4), torch.full((8,), 11.0))


def test_pool_dot_conv_scan_axis_sum(P):
    a = torch.arange(8.0)
    close(P.pool3(cu(a)), P.oracle_pool3(a))
    x = torch.randn(777)
    close(P.pool3(cu(x), block=64), P.oracle_pool3(x))
    close(P.dot(cu(a), cu(a)), (a * a).sum().reshape(1))
    y = torch.randn(5000)
    close(P.dot(cu(x.repeat(7)[:5000]), cu(y), block=256), (x.repeat(7)[:5000] * y).sum().reshape(1), 1e-3)
    close(P.conv1d(cu(torch.arange(6.0)), cu(torch.arange(3.0))), P.oracle_conv1d(torch.arange(6.0), torch.arange(3.0)))
    close(P.conv1d(cu(torch.arange(15.0)), cu(torch.arange(4.0)), block=8),
          P.oracle_conv1d(torch.arange(15.0), torch.arange(4.0)))
    close(P.prefix_sum(cu(torch.arange(8.0))), torch.cumsum(torch.arange(8.0), 0))
    close(P.prefix_sum(cu(torch.arange(15.0)), block=8), torch.cumsum(torch.arange(15.0), 0))
    z = torch.randn(1000)
    close(P.prefix_sum(cu(z), block=128), torch.cumsum(z, 0), 1e-3)
    m = torch.arange(24.0).view(4, 6)
    close(P.axis_sum(cu(m)), m.sum(1))


def test_debug_exercises_and_checked_accessor(P):
    a = torch.arange(4.0)
    close(P.sliding_window3(cu(a)), P.oracle_sliding_window3(a))
    close(P.collaborative_filter(cu(a)), P.oracle_collaborative_filter(a))
    m = torch.arange(4.0).view(2, 2)
    close(P.shared_sum_broadcast(cu(m)), torch.full((2, 2), 6.0))
    src = torch.arange(10.0)
    out, bad, who, idx = P.checked_gather(cu(src), torch.tensor([0, 3, 42, 9, -1]).cuda())
    close(out, torch.tensor([0., 3., 0., 9., 0.]))
    assert bad == 2 and (who, idx) in [(2, 42), (4, -1)]
    assert float(torch.ones(4, device="cuda").sum()) == 4.0  # no fault happened


@pytest.mark.parametrize("variant", ["naive", "single_block", "tiled", "tf32_mma", "tcgen05"])
def test_matmul_variants(P, variant):
    shapes = [(2, 2, 2), (9, 9, 9)] if variant == "single_block" else [(9, 9, 9), (130, 70, 50), (256, 128, 64)]
    for M, N, K in shapes:
        if variant == "tcgen05" and (K % 8 or N % 8):
            continue
        a, b = torch.randn(M, K), torch.randn(K, N)
        tol = 1e-4 if variant in ("naive", "single_block", "tiled") else 3e-2
        got = P.matmul(cu(a), cu(b), variant)
        ref = a @ b
        assert (got.cpu() - ref).abs().max() / ref.abs().max() < tol, (variant, M, N, K)


def test_tf32_tensor_core_matmul_reference_tolerance(P):
    # 1024^3 with the reference's tolerance (atol 1e-3 ... rtol 2e-2, p33.mojo:413-415)
    a, b = torch.randn(1024, 1024) * 0.1, torch.randn(1024, 1024) * 0.1
    got = P.matmul(cu(a), cu(b), "tf32_mma").cpu()
    assert torch.allclose(got, a @ b, atol=1e-2, rtol=2e-2)


def test_transpose_softmax_attention(P):
    m = torch.randn(37, 53)
    close(P.transpose(cu(m)), m.t())
    v = torch.randn(128)
    close(P.softmax(cu(v)), torch.softmax(v, 0), 1e-6)
    close(P.softmax(cu(torch.randn(5, 1000))).sum(-1), torch.ones(5), 1e-5)
    q, k, vv = torch.randn(16), torch.randn(16, 16), torch.randn(16, 16)
    close(P.attention_vec(cu(q), cu(k), cu(vv)), torch.softmax(k @ q, 0) @ vv, 1e-5)
    q, k, vv = torch.randn(64), torch.randn(300, 64), torch.randn(300, 64)
    close(P.attention_vec(cu(q), cu(k), cu(vv)), torch.softmax(k @ q, 0) @ vv, 1e-4)


def test_embedding_variants(P):
    w = torch.randn(1000, 64)
    idx = torch.randint(0, 1000, (4, 33))
    for variant in ("coalesced", "2d"):
        close(P.embedding(idx.cuda(), cu(w), variant), w[idx])
    bad = torch.tensor([[1, 5000]])
    out = P.embedding(bad.cuda(), cu(w)).cpu()
    assert torch.equal(out[0, 0], w[1]) and out[0, 1].abs().max() == 0  # out-of-range id reads as zeros


def test_layernorm_linear_fwd_bwd(P):
    B, S, H, O = 4, 4, 8, 16
    x = torch.randn(B, S, H, requires_grad=True)
    gamma, beta = (torch.randn(H) * 0.5 + 1).requires_grad_(), torch.randn(H).requires_grad_()
    w, bias = torch.randn(O, H).requires_grad_(), torch.randn(O).requires_grad_()
    ref = torch.nn.functional.linear(torch.nn.functional.layer_norm(x, (H,), gamma, beta, 1e-5), w, bias)
    for fused in (True, False):
        close(P.ln_linear_fwd(cu(x.detach()), cu(gamma.detach()), cu(beta.detach()), cu(w.detach()), cu(bias.detach()),
                              fused=fused), ref.detach(), 1e-4)
    dy = torch.randn(B, S, O)
    ref.backward(dy)
    for det in (True, False):
        dx, dg, db, dw, dbias = P.ln_linear_bwd(cu(dy), cu(x.detach()), cu(gamma.detach()), cu(beta.detach()),
                                                cu(w.detach()), deterministic=det)
        close(dx, x.grad, 1e-4), close(dg, gamma.grad, 1e-4), close(db, beta.grad, 1e-4)
        close(dw, w.grad, 1e-4), close(dbias, bias.grad, 1e-4)
    a1 = P.ln_linear_bwd(cu(dy), cu(x.detach()), cu(gamma.detach()), cu(beta.detach()), cu(w.detach()))
    a2 = P.ln_linear_bwd(cu(dy), cu(x.detach()), cu(gamma.detach()), cu(beta.detach()), cu(w.detach()))
    assert all(torch.equal(p, q) for p, q in zip(a1, a2))  # the deterministic form is bitwise stable


def test_elementwise_and_warp_level(P):
    a, b = torch.randn(1024), torch.randn(1024)
    for variant in ("scalar", "tiled", "vectorized"):
        close(P.elementwise_add(cu(a), cu(b), variant), a + b)
    close(P.elementwise_add(cu(torch.randn(100_003)), cu(torch.zeros(100_003))) * 0, torch.zeros(100_003))
    x, y = torch.randn(96), torch.randn(96)
    close(P.warp_dot(cu(x), cu(y)), (x * y).view(3, 32).sum(1), 1e-5)
    assert P.warp_sum_int(torch.arange(64).cuda()).tolist() == [sum(range(32)), sum(range(32, 64))]
    for op in P.WARP_OPS:
        for n in (32, 64):
            v = torch.randn(n)
            close(P.warp_op(cu(v), op), P.oracle_warp_op(v, op), 1e-5)
    v = torch.tensor([3., 7., 1., 8., 2., 9., 4., 6.])
    close(P.warp_partition(cu(v), 5.0), torch.tensor([3., 1., 2., 4., 7., 8., 9., 6.]))
    r = torch.rand(32) * 10
    got = P.warp_partition(cu(r), 5.0).cpu()
    assert torch.equal(got, torch.cat([r[r < 5], r[r >= 5]]))


def test_block_level(P):
    a = torch.rand(128)
    close(P.block_dot(cu(a), cu(a)), (a * a).sum().reshape(1), 1e-4)
    for tb in (0, 3, 7):
        vals, n = P.block_histogram_bin_extract(cu(a), tb, 8)
        ref = a[(a * 8).floor().clamp(0, 7) == tb]
        assert n == ref.numel()
        close(vals, ref)
    close(P.block_normalize(cu(a)), a / a.mean(), 1e-5)


def test_async_copy_pipelines_and_study_kernels(P):
    from zero_to_hero_b200.ops import _lib
    a, w5 = torch.randn(16384), torch.tensor([0.1, 0.2, 0.4, 0.2, 0.1])
    ref = P.oracle_async_copy_conv(a[:1024], w5)
    for bulk in (False, True):
        close(P.async_copy_conv(cu(a), cu(w5), bulk=bulk)[:1024], ref, 1e-5)
    close(P.async_copy_conv(cu(a[:700]), cu(w5), bulk=True), P.oracle_async_copy_conv(a[:700], w5), 1e-5)
    x = torch.randn(1024)
    close(P.pipeline_blur(cu(x)), P.oracle_pipeline_blur(x), 1e-5)
    close(P.double_buffer_stencil(cu(x), 3), P.oracle_double_buffer_stencil(x, 3), 1e-5)
    close(P.double_buffer_stencil(cu(x[:900]), 4), P.oracle_double_buffer_stencil(x[:900], 4), 1e-5)
    torch.cuda.synchronize()
    _lib.check_status()
    p, q = torch.randn(8192), torch.randn(8192)
    for mode in ("coalesced", "strided", "reversed"):
        close(P.access_pattern_add(cu(p), cu(q), mode), p + q)
    for smem in (4096, 16 * 1024, 48 * 1024):
        close(P.occupancy_saxpy(cu(p), cu(q), 2.0, smem), 2.0 * q + p)
    for stride in (1, 2):
        close(P.bank_conflict(cu(p), stride), (p + 10) * 2)


def test_clusters(P):
    a = torch.randn(1024)
    ref = torch.stack([(a[i * 256:(i + 1) * 256] * (i + 1)).sum() for i in range(4)])
    for we in (False, True):
        close(P.cluster_block_sums(cu(a), 256, 4, we), ref, 1e-3)
    for dsmem in (False, True):
        close(P.cluster_reduce(cu(a), 256, 4, dsmem), a.sum().reshape(1), 1e-3)
    b = torch.randn(4096)
    close(P.cluster_reduce(cu(b), 256, 4, True), b.view(4, 1024).sum(1), 1e-3)


def test_benchmark_mode_of_the_puzzle_cli(capsys):
    """`pNN --benchmark`: the size sweeps of the reference's in-puzzle Bench harnesses."""
    import json

    from zero_to_hero_b200 import puzzles
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    assert puzzles.main(["p32", "--benchmark"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert len(lines) == 4 and all(l["us"] > 0 and l["gbs"] > 0 for l in lines)
    assert {l["variant"] for l in lines} == {"stride 1", "stride 2"}
    assert puzzles.main(["p01", "--benchmark"]) == 2      # no sweep for that puzzle
