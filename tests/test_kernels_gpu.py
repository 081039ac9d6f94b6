"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.ops import _lib
    _lib.cuda_lib()  # a missing native library is a failure on a GPU box, not a skip
    torch.manual_seed(0)
    return torch.device("cuda")


def rel_err(got, ref, rtol=5e-2, atol_rms=5e-2):
    """Largest error relative to the largest reference value (what the callers bound), after a
    per-element check: |got - ref| <= atol_rms * rms(ref) + rtol * |ref| for all but a 1e-4
    fraction of the elements. The second part is what catches a kernel that is only wrong where
    the reference is small (a dropped tile, a missed tail): the max-normalised figure alone
    would let that pass."""
    got, ref = got.float(), ref.float()
    err = (got - ref).abs()
    rms = ref.pow(2).mean().sqrt().item()
    bad = err > atol_rms * rms + rtol * ref.abs()
    n_bad = int(bad.sum().item())
    assert n_bad <= 1e-4 * ref.numel(), (
        f"{n_bad} of {ref.numel()} elements off by more than {atol_rms} rms + {rtol} |ref| "
        f"(rms {rms:.3e}, worst error {err.max().item():.3e})")
    return err.max().item() / (ref.abs().max().item() + 1e-9)


def status_ok():
    from zero_to_hero_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.check_status()


# ------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (384, 768, 768), (200, 264, 136), (1024, 2304, 768),
                                   (64, 1600, 1600)])
def test_gemm_all_layouts(dev, a_mn, b_mn, M, N, K):
    from zero_to_hero_b200.ops import gemm as G
    A = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    B = (torch.randn(N, K, device=dev) * 0.5).bfloat16()
    ref = A.float() @ B.float().t()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    G.gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B, out,
           a_mn=bool(a_mn), b_mn=bool(b_mn))
    status_ok()
    assert rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("algo", [1, 2])
@pytest.mark.parametrize("M,N,K,b_mn", [
    (16384, 768, 3072, 0),    # GPT-2 124M: second MLP projection (2.6 waves of 256 x 256 tiles)
    (16384, 50304, 768, 0),   # lm_head over the padded vocabulary
    (16384, 768, 50304, 1),   # its data gradient
    (8192, 4800, 1600, 0),    # GPT-2 1.5B: QKV projection (C = 1600 = 6.25 x 256: ragged tiles)
    (8192, 1600, 6400, 0),    # GPT-2 1.5B: second MLP projection
    (8192, 6400, 1600, 1),    # and a data-gradient layout at that width
])
def test_gemm_benchmark_shapes(dev, algo, M, N, K, b_mn):
    """The shapes the benchmark configurations actually run, through the CTA-pair kernel
    explicitly (algo 1) and through the automatic choice (algo 2)."""
    from zero_to_hero_b200.ops import gemm as G
    A = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    B = (torch.randn(N, K, device=dev) * 0.5).bfloat16()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    G.set_algo(algo)
    try:
        G.gemm(A, B.t().contiguous() if b_mn else B, out, b_mn=bool(b_mn))
        status_ok()
    finally:
        G.set_algo(2)
    rows = torch.randint(0, M, (512,), device=dev)   # a row sample keeps the fp32 reference small
    rows[:4] = torch.tensor([0, 1, M - 2, M - 1], device=dev)
    ref = A[rows].float() @ B.float().t()
    assert rel_err(out[rows], ref) < 1e-2


@pytest.mark.parametrize("b_mn", [0, 1])
def test_gemm_stream_k_fixup_matches_whole_tiles(dev, b_mn):
    """80 tiles of 256 x 256 on 74 CTA pairs (1.08 waves): the balanced schedule cuts tiles between
    neighbouring pairs and one of them adds the other's piece before the epilogue. Every epilogue,
    ragged M / N / K, against fp32 and against the whole-tile schedule of the same kernel."""
    from zero_to_hero_b200.ops import gemm as G
    M, N, K = 5000, 1000, 520
    A = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    B = (torch.randn(N, K, device=dev) * 0.5).bfloat16()
    Bop = B.t().contiguous() if b_mn else B
    bias = torch.randn(N, device=dev).bfloat16()
    res = torch.randn(M, N, device=dev).bfloat16()
    base = A.float() @ B.float().t() + bias.float()
    outs = {}
    for fix in (True, False):
        G.set_fixup(fix)
        try:
            o_none = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            G.gemm(A, Bop, o_none, b_mn=bool(b_mn), bias=bias)
            o_res = torch.empty_like(o_none)
            G.gemm(A, Bop, o_res, b_mn=bool(b_mn), bias=bias, residual=res, epi=G.EPI_RESIDUAL)
            o_act, o_pre = torch.empty_like(o_none), torch.empty_like(o_none)
            G.gemm(A, Bop, o_act, b_mn=bool(b_mn), bias=bias, aux_out=o_pre, epi=G.EPI_GELU)
            o_gg = torch.empty_like(o_none)
            G.gemm(A, Bop, o_gg, b_mn=bool(b_mn), aux_in=o_pre, epi=G.EPI_GELU_GRAD)
            status_ok()
        finally:
            G.set_fixup(False)
        outs[fix] = (o_none, o_res, o_act, o_pre, o_gg)
        assert rel_err(o_none, base) < 1e-2
        assert rel_err(o_res, base + res.float()) < 1e-2
        assert rel_err(o_pre, base) < 1e-2
        assert rel_err(o_act, F.gelu(o_pre.float(), approximate="tanh")) < 1e-2
    # same products, same fp32 sums up to the order of two partial sums: bf16 outputs agree closely
    for a, b in zip(outs[True], outs[False]):
        assert rel_err(a, b.float()) < 1e-2
    # and the balanced schedule is reproducible run to run
    o2 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    G.set_fixup(True)
    try:
        G.gemm(A, Bop, o2, b_mn=bool(b_mn), bias=bias)
    finally:
        G.set_fixup(False)
    assert torch.equal(o2, outs[True][0])


def test_gemm_epilogues(dev):
    from zero_to_hero_b200.ops import gemm as G
    M, N, K = 520, 776, 264  # tails in every dimension
    A = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    B = (torch.randn(N, K, device=dev) * 0.5).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    res = torch.randn(M, N, device=dev).bfloat16()
    base = A.float() @ B.float().t()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    G.gemm(A, B, out, bias=bias)
    assert rel_err(out, base + bias.float()) < 1e-2
    G.gemm(A, B, out, bias=bias, residual=res, epi=G.EPI_RESIDUAL)
    assert rel_err(out, base + bias.float() + res.float()) < 1e-2
    pre = torch.empty_like(out)
    G.gemm(A, B, out, bias=bias, aux_out=pre, epi=G.EPI_GELU)
    assert rel_err(pre, base + bias.float()) < 1e-2
    assert rel_err(out, F.gelu(pre.float(), approximate="tanh")) < 1e-2
    x = pre.float().requires_grad_(True)
    F.gelu(x, approximate="tanh").sum().backward()
    G.gemm(A, B, out, aux_in=pre, epi=G.EPI_GELU_GRAD)
    assert rel_err(out, base * x.grad) < 1e-2
    # the training pair: the forward stores gelu'(x), the backward multiplies by it
    deriv = torch.empty_like(out)
    G.gemm(A, B, out, bias=bias, aux_out=deriv, epi=G.EPI_GELU_SAVE_GRAD)
    xb = (base + bias.float()).requires_grad_(True)
    F.gelu(xb, approximate="tanh").sum().backward()
    assert rel_err(out, F.gelu(xb.detach(), approximate="tanh")) < 1e-2
    assert rel_err(deriv, xb.grad) < 1e-2
    G.gemm(A, B, out, aux_in=deriv, epi=G.EPI_MUL_AUX)
    assert rel_err(out, base * deriv.float()) < 1e-2
    o32 = torch.zeros(M, N, device=dev)
    G.gemm(A, B, o32, epi=G.EPI_ATOMIC_ADD, split_k=3)
    assert rel_err(o32, base) < 1e-4
    G.gemm(A, B, o32, epi=G.EPI_ACCUMULATE)
    assert rel_err(o32, 2 * base) < 1e-4
    o32 = torch.empty(M, N, device=dev)
    G.gemm(A, B, o32)
    assert rel_err(o32, base) < 1e-4
    status_ok()


@pytest.mark.parametrize("algo", [0, 1])
@pytest.mark.parametrize("M,N,K", [(512, 768, 264), (16384, 3072, 768), (2080, 352, 96)])
def test_gemm_column_sums_of_the_output(dev, algo, M, N, K):
    """The epilogue's by-product: the column sums of C as stored (bf16) are added to an fp32
    vector; against a separate fp32 sum over the rows of the same C."""
    from zero_to_hero_b200.ops import gemm as G
    torch.manual_seed(M + N)
    A = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    B = (torch.randn(K, N, device=dev) * 0.5).bfloat16()
    pre = torch.randn(M, N, device=dev).bfloat16()
    G.set_algo(algo)
    try:
        for epi, kw in ((G.EPI_GELU_GRAD, dict(aux_in=pre)), (G.EPI_NONE, {})):
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            start = torch.randn(N, device=dev)
            acc = start.clone()
            G.gemm(A, B, out, b_mn=True, epi=epi, colsum=acc, **kw)
            ref = torch.empty_like(out)
            G.gemm(A, B, ref, b_mn=True, epi=epi, **kw)
            assert torch.equal(out, ref)  # the by-product leaves C alone
            want = start + out.float().sum(0)
            assert (acc - want).abs().max().item() <= 1e-4 * out.float().abs().sum(0).max().item() + 1e-4
        # a shape whose rows do not fill whole warps is refused, not computed wrongly
        with pytest.raises(RuntimeError):
            G.gemm(A[:40], B, torch.empty(40, N, device=dev, dtype=torch.bfloat16), b_mn=True,
                   colsum=torch.zeros(N, device=dev))
    finally:
        G.set_algo(2)
    status_ok()


def test_gemm_deterministic_without_atomics(dev):
    from zero_to_hero_b200.ops import gemm as G
    A = torch.randn(1024, 768, device=dev).bfloat16()
    B = torch.randn(2304, 768, device=dev).bfloat16()
    o1 = torch.empty(1024, 2304, device=dev, dtype=torch.bfloat16)
    o2 = torch.empty_like(o1)
    G.gemm(A, B, o1)
    G.gemm(A, B, o2)
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("algo", [0, 1])
@pytest.mark.parametrize("M,N,K", [(768, 768, 4096), (2304, 768, 2048), (300, 520, 1000), (256, 256, 64)])
def test_gemm_stream_k(dev, algo, M, N, K):
    """Weight-gradient form (both operands MN-major, fp32 atomic accumulation) under the stream-K
    schedule: every CTA gets an equal run of k-blocks that may span several output tiles."""
    from zero_to_hero_b200.ops import gemm as G
    Kp = (K + 7) // 8 * 8
    Mp, Np = (M + 7) // 8 * 8, (N + 7) // 8 * 8
    At = torch.randn(Kp, Mp, device=dev).bfloat16()[:K, :M]  # [K, M], pitch a multiple of 8
    Bt = torch.randn(Kp, Np, device=dev).bfloat16()[:K, :N]
    base = At.float().t() @ Bt.float()
    start = torch.randn(M, Np, device=dev)[:, :N]
    out = start.clone()
    prev = G.get_algo()
    try:
        G.set_algo(algo)
        G.gemm(At, Bt, out, a_mn=True, b_mn=True, epi=G.EPI_ATOMIC_ADD, split_k=0)
    finally:
        G.set_algo(prev)
    assert rel_err(out, base + start) < 1e-4
    status_ok()


def test_gemm_rejects_unaligned(dev):
    from zero_to_hero_b200.ops import gemm as G
    A = torch.randn(64, 68, device=dev).bfloat16()[:, :65]  # pitch 68 is not a multiple of 8
    B = torch.randn(64, 65, device=dev).bfloat16()
    with pytest.raises(RuntimeError):
        G.gemm(A, B, torch.empty(64, 64, device=dev, dtype=torch.bfloat16))


# ------------------------------------------------------------------------------ attention
@pytest.mark.parametrize("B,T,H", [(2, 256, 3), (1, 1024, 2), (2, 200, 2), (1, 77, 1)])
def test_flash_attention_fwd_bwd(dev, B, T, H):
    from zero_to_hero_b200.ops import native as N
    C = H * 64
    qkv = (torch.randn(B * T, 3 * C, device=dev) * 0.7).bfloat16()
    out = torch.empty(B * T, C, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev)
    N.flash_fwd(qkv, out, lse, B, T, H)
    status_ok()
    q, k, v = [x.reshape(B, T, H, 64).transpose(1, 2).float().requires_grad_(True)
               for x in qkv.float().split(C, dim=1)]
    s = (q @ k.transpose(-1, -2)) * 0.125
    mask = torch.ones(T, T, device=dev, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    ref = torch.softmax(s, -1) @ v  # plain fp32 attention
    assert rel_err(out, ref.transpose(1, 2).reshape(B * T, C)) < 1e-2
    assert rel_err(lse, torch.logsumexp(s, -1)) < 1e-3
    dout = (torch.randn(B * T, C, device=dev) * 0.5).bfloat16()
    ref.backward(dout.float().reshape(B, T, H, 64).transpose(1, 2))
    refd = torch.cat([g.grad.transpose(1, 2).reshape(B * T, C) for g in (q, k, v)], 1)
    dqkv = torch.zeros_like(qkv)
    dqa = torch.empty(N.flash_bwd_dq_elems(B, T, H), device=dev)
    stats = torch.empty(N.flash_bwd_stats_elems(B, T, H), device=dev)
    N.flash_bwd(qkv, out, dout, lse, dqkv, dqa, stats, B, T, H)
    status_ok()
    for i, name in enumerate("qkv"):
        assert rel_err(dqkv[:, i * C:(i + 1) * C], refd[:, i * C:(i + 1) * C]) < 2e-2, name
    # the by-product: column sums of dqkv (the QKV bias gradient) added to an fp32 vector
    start = torch.randn(3 * C, device=dev)
    dbias = start.clone()
    dqkv2 = torch.zeros_like(qkv)
    N.flash_bwd(qkv, out, dout, lse, dqkv2, dqa, stats, B, T, H, dbias=dbias)
    status_ok()
    assert rel_err(dqkv2, dqkv) < 1e-3  # same kernels (atomic dQ accumulation: not bitwise)
    want = start + dqkv2.float().sum(0)
    assert (dbias - want).abs().max().item() <= 1e-4 * dqkv2.float().abs().sum(0).max().item() + 1e-4


def test_flash_forward_run_twice_bitwise(dev):
    from zero_to_hero_b200.ops import native as N
    B, T, H = 2, 512, 4
    qkv = torch.randn(B * T, 3 * H * 64, device=dev).bfloat16()
    o1 = torch.empty(B * T, H * 64, device=dev, dtype=torch.bfloat16)
    o2 = torch.empty_like(o1)
    lse = torch.empty(B, H, T, device=dev)
    N.flash_fwd(qkv, o1, lse, B, T, H)
    N.flash_fwd(qkv, o2, lse, B, T, H)
    assert torch.equal(o1, o2)


# ------------------------------------------------------------------------------ layernorm
@pytest.mark.parametrize("M,C,has_bias", [(1000, 768, False), (512, 1024, True), (300, 1600, True),
                                          (64, 384, True), (7, 2048, False)])
def test_layernorm_fwd_bwd(dev, M, C, has_bias):
    from zero_to_hero_b200.ops import native as N
    x = torch.randn(M, C, device=dev).bfloat16()
    w = (torch.randn(C, device=dev) * 0.5 + 1).bfloat16()
    b = torch.randn(C, device=dev).bfloat16() if has_bias else None
    y = torch.empty_like(x)
    mean = torch.empty(M, device=dev)
    rstd = torch.empty(M, device=dev)
    N.layernorm_fwd(x, w, b, y, mean, rstd)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    bf = b.float().requires_grad_(True) if has_bias else None
    ref = F.layer_norm(xf, (C,), wf, bf, 1e-5)
    assert rel_err(y, ref) < 1e-2
    dy = torch.randn(M, C, device=dev).bfloat16()
    dres = torch.randn(M, C, device=dev).bfloat16()
    ref.backward(dy.float())
    dx = torch.empty_like(x)
    dw = torch.zeros(C, device=dev)
    db = torch.zeros(C, device=dev) if has_bias else None
    scratch = torch.empty(N.layernorm_bwd_num_partials(M) * 2 * C, device=dev)
    N.layernorm_bwd(dy, x, w, mean, rstd, dres, dx, dw, db, scratch, accumulate=True)
    assert rel_err(dx, xf.grad + dres.float()) < 1e-2
    assert rel_err(dw, wf.grad) < 1e-4
    if has_bias:
        assert rel_err(db, bf.grad) < 1e-4
    # deterministic two-stage reduction: a second run gives the same bits
    dw2 = torch.zeros(C, device=dev)
    N.layernorm_bwd(dy, x, w, mean, rstd, dres, dx, dw2, torch.zeros(C, device=dev) if has_bias else None,
                    scratch, accumulate=True)
    assert torch.equal(dw, dw2)
    # fused column sums of the output (the bias gradient of the projection that feeds this
    # residual stream): accumulated on top of what is there, other outputs unchanged
    dx3 = torch.empty_like(x)
    dw3 = torch.zeros(C, device=dev)
    dxsum = torch.full((C,), 2.0, device=dev)
    scratch3 = torch.empty(N.layernorm_bwd_num_partials(M) * 3 * C, device=dev)
    N.layernorm_bwd(dy, x, w, mean, rstd, dres, dx3, dw3, torch.zeros(C, device=dev) if has_bias else None,
                    scratch3, accumulate=True, dxsum=dxsum)
    assert torch.equal(dx3, dx) and torch.equal(dw3, dw)
    assert rel_err(dxsum, 2.0 + (xf.grad + dres.float()).sum(0)) < 1e-3
    status_ok()


# ------------------------------------------------------------------- embedding / CE / optim
def test_embedding_fwd_bwd(dev):
    from zero_to_hero_b200.ops import native as N
    B, T, C, V = 4, 64, 768, 1000
    idx = torch.randint(0, V, (B, T), device=dev)
    wte = torch.randn(V, C, device=dev).bfloat16()
    wpe = torch.randn(T, C, device=dev).bfloat16()
    out = torch.empty(B * T, C, device=dev, dtype=torch.bfloat16)
    N.embed_fwd(idx, wte, wpe, out, T)
    assert rel_err(out, (wte.float()[idx] + wpe.float()[None]).reshape(B * T, C)) < 5e-3
    dx = torch.randn(B * T, C, device=dev).bfloat16()
    dwte = torch.zeros(V, C, device=dev)
    dwpe = torch.zeros(T, C, device=dev)
    N.embed_bwd(idx, dx, dwte, dwpe, B, T)
    ref = torch.zeros(V, C, device=dev).index_add_(0, idx.reshape(-1), dx.float())
    assert rel_err(dwte, ref) < 1e-5
    assert rel_err(dwpe, dx.float().reshape(B, T, C).sum(0)) < 1e-5
    N.embed_fwd(idx.int(), wte, wpe, out, T)  # int32 ids take the same path
    assert rel_err(out, (wte.float()[idx] + wpe.float()[None]).reshape(B * T, C)) < 5e-3
    status_ok()


def test_embedding_out_of_range_id_sets_status_not_fault(dev):
    from zero_to_hero_b200.ops import _lib, native as N
    idx = torch.tensor([[0, 5, 99999]], device=dev)
    wte = torch.randn(10, 64, device=dev).bfloat16()
    out = torch.empty(3, 64, device=dev, dtype=torch.bfloat16)
    N.embed_fwd(idx, wte, None, out, 3)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        _lib.check_status()
    _lib.check_status()  # cleared


@pytest.mark.parametrize("M,Vr,Vp", [(512, 50257, 50304), (33, 65, 72), (64, 50304, 50304)])
def test_cross_entropy_fwd_bwd(dev, M, Vr, Vp):
    from zero_to_hero_b200.ops import native as N
    logits = (torch.randn(M, Vp, device=dev) * 2).bfloat16()
    tg = torch.randint(0, Vr, (M,), device=dev)
    lf = logits.float()[:, :Vr].clone().requires_grad_(True)
    rl = F.cross_entropy(lf, tg, reduction="none")
    rl.mean().backward()
    losses = torch.empty(M, device=dev)
    N.ce_fwd_bwd(logits, tg, losses, Vr, 1.0 / M)
    assert rel_err(losses, rl) < 1e-4
    assert rel_err(logits[:, :Vr], lf.grad) < 1e-2
    if Vp > Vr:
        assert logits[:, Vr:].abs().max().item() == 0.0
    status_ok()


def test_adamw_matches_torch(dev):
    from zero_to_hero_b200.ops import native as N
    n, nd = 1_000_003, 700_000
    p = torch.randn(n, device=dev) * 0.02
    g = torch.zeros(n, device=dev)
    m = torch.zeros(n, device=dev)
    v = torch.zeros(n, device=dev)
    p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    pr = [p[:nd].clone().requires_grad_(True), p[nd:].clone().requires_grad_(True)]
    opt = torch.optim.AdamW([{"params": [pr[0]], "weight_decay": 0.1}, {"params": [pr[1]], "weight_decay": 0.0}],
                            lr=6e-4, betas=(0.9, 0.95), eps=1e-8)
    partials = torch.empty(1024, device=dev)
    norm = torch.zeros(1, device=dev)
    hyper = torch.zeros(16, device=dev)
    for step in range(1, 4):
        gg = torch.randn(n, device=dev) * 1e-2
        g.copy_(gg)
        pr[0].grad, pr[1].grad = gg[:nd].clone(), gg[nd:].clone()
        tn = torch.nn.utils.clip_grad_norm_(pr, 1.0)
        opt.step()
        hyper.copy_(torch.tensor([6e-4, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** step, 1 - 0.95 ** step, 1.0, 1.0] + [0] * 7))
        npart = N.gradnorm_partials(g, partials)
        N.adamw_step(p, g, m, v, p16, nd, hyper, partials, npart, norm)
        assert rel_err(norm, tn.reshape(1)) < 1e-5
        assert rel_err(p, torch.cat([pr[0], pr[1]]).detach()) < 1e-5
    assert rel_err(p16, p) < 5e-3 and g.abs().max().item() == 0.0
    status_ok()


def test_colsum_and_cast(dev):
    from zero_to_hero_b200.ops import native as N
    dy = torch.randn(3000, 2304, device=dev).bfloat16()
    db = torch.zeros(2304, device=dev)
    N.colsum_bf16(dy, db)
    assert rel_err(db, dy.float().sum(0)) < 1e-5
    x = torch.randn(100003, device=dev)
    y = torch.empty(100003, device=dev, dtype=torch.bfloat16)
    N.cast_f32_to_bf16(x, y)
    assert torch.equal(y, x.bfloat16())
    status_ok()


# ------------------------------------------------------------------- bounded device waits
def test_bounded_peer_wait_times_out_with_status_and_context_survives(dev):
    """A wait on a flag nobody sets must end by itself, report kTimeoutPeer, and leave the
    context usable; a flag that is set lets the wait succeed."""
    import ctypes
    from zero_to_hero_b200.ops import _lib
    lib = _lib.cuda_lib()
    lib.z2h_wait_probe.restype = ctypes.c_int
    lib.z2h_wait_probe.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_uint,
                                   ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    pad = torch.zeros(64, dtype=torch.int64, device=dev)
    result = torch.full((1,), -1, dtype=torch.int32, device=dev)
    status = _lib.status_word(dev)
    rc = lib.z2h_wait_probe(_lib.ptr(pad), 0, 1, 5, 50_000_000, _lib.ptr(status), _lib.ptr(result),
                            _lib.stream_ptr())  # 50 ms budget, epoch 5 never arrives
    assert rc == 0
    torch.cuda.synchronize()
    assert int(result.item()) == 0
    with pytest.raises(RuntimeError, match="peer"):
        _lib.check_status(dev)
    pad[1] = 5 << 32  # slot (kind 0, src 1) now carries epoch 5
    rc = lib.z2h_wait_probe(_lib.ptr(pad), 0, 1, 5, 50_000_000, _lib.ptr(status), _lib.ptr(result),
                            _lib.stream_ptr())
    torch.cuda.synchronize()
    assert rc == 0 and int(result.item()) == 1
    _lib.check_status(dev)
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0  # the context still works


# ------------------------------------------------------------------------------ sampling
def test_sample_topk_distribution_and_support(dev):
    from zero_to_hero_b200.ops.sampling import sample_topk_native
    V = 1000
    logits = torch.randn(V, device=dev) * 2
    rows = logits.repeat(4096, 1)  # every row draws with its own counter
    ids = sample_topk_native(rows, temperature=0.8, top_k=None, seed=7).view(-1)
    p = torch.softmax(logits / 0.8, 0)
    freq = torch.bincount(ids, minlength=V).float() / ids.numel()
    assert (freq - p).abs().max().item() < 0.02
    assert freq[p.argmax()].item() == pytest.approx(p.max().item(), abs=0.02)
    # top-k keeps exactly the k largest (no ties here) and renormalises among them
    k = 5
    ids = sample_topk_native(rows, temperature=1.0, top_k=k, seed=11).view(-1)
    top = torch.topk(logits, k).indices
    assert set(ids.unique().tolist()) <= set(top.tolist())
    pk = torch.softmax(logits[top], 0)
    fk = torch.stack([(ids == t).float().mean() for t in top])
    assert (fk - pk).abs().max().item() < 0.03
    # a very low temperature is an arg-max; same seed and offset reproduce
    assert sample_topk_native(rows[:8], 1e-3, None, 3).view(-1).tolist() == [int(logits.argmax())] * 8
    a = sample_topk_native(rows[:64], 1.0, 50, seed=5, offset=9)
    b = sample_topk_native(rows[:64], 1.0, 50, seed=5, offset=9)
    assert torch.equal(a, b)
    # ties at the k-th value are all kept, as `logits < kth` masking does
    t = torch.tensor([[1.0, 3.0, 3.0, 3.0, 0.0]], device=dev).repeat(512, 1)
    seen = set(sample_topk_native(t, 1.0, 2, seed=1).view(-1).tolist())
    assert seen == {1, 2, 3}
    status_ok()


# ------------------------------------------------------------------------------ dropout
@pytest.mark.parametrize("p", [0.1, 0.5])
def test_dropout_apply_matches_host_mask(dev, p):
    from zero_to_hero_b200.ops import dropout as D, native as N
    n = 4096 * 24
    x = torch.randn(n, device=dev).bfloat16()
    res = torch.randn(n, device=dev).bfloat16()
    seed = torch.tensor([987654321], device=dev, dtype=torch.int64)
    out = torch.empty_like(x)
    N.dropout_apply(x, out, p, seed, 5, residual=res)
    keep = D.elementwise_keep(n, p, 987654321, 5, dev)
    _, scale = D.threshold_and_scale(p)
    ref = (torch.where(keep, x.float() * scale, torch.zeros((), device=dev)) + res.float()).bfloat16()
    assert torch.equal(out, ref)
    frac = 1.0 - keep.float().mean().item()
    assert abs(frac - round(p * 256) / 256) < 0.01
    # the backward of a site is the same call on the gradient, in place allowed
    g = torch.randn(n, device=dev).bfloat16()
    g_ref = torch.where(keep, g.float() * scale, torch.zeros((), device=dev)).bfloat16()
    N.dropout_apply(g, g, p, seed, 5)
    assert torch.equal(g, g_ref)
    # another site or seed gives another mask
    assert not torch.equal(keep, D.elementwise_keep(n, p, 987654321, 6, dev))


@pytest.mark.parametrize("B,T,H", [(2, 256, 2), (1, 200, 3)])
def test_flash_attention_dropout_against_masked_reference(dev, B, T, H):
    from zero_to_hero_b200.ops import dropout as D, native as N
    p, seed_v, site = 0.25, 4242, 7
    C = H * 64
    qkv = (torch.randn(B * T, 3 * C, device=dev) * 0.7).bfloat16()
    dout = torch.randn(B * T, C, device=dev).bfloat16()
    seed = torch.tensor([seed_v], device=dev, dtype=torch.int64)
    out = torch.empty(B * T, C, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev)
    N.flash_fwd(qkv, out, lse, B, T, H, p, seed, site)
    dqkv = torch.empty_like(qkv)
    dq_acc = torch.empty(N.flash_bwd_dq_elems(B, T, H), device=dev)
    stats = torch.empty(N.flash_bwd_stats_elems(B, T, H), device=dev)
    N.flash_bwd(qkv, out, dout, lse, dqkv, dq_acc, stats, B, T, H, p, seed, site)
    # reference: explicit attention in fp32 with the same mask
    x = qkv.float().view(B, T, 3, H, 64).requires_grad_(True)
    q, k, v = (x[:, :, i].transpose(1, 2) for i in range(3))
    att = (q @ k.transpose(-2, -1)) * 0.125
    causal = torch.ones(T, T, dtype=torch.bool, device=dev).tril()
    att = att.masked_fill(~causal, float("-inf")).softmax(-1)
    keep = D.attention_keep(B, H, T, p, seed_v, site, dev)
    att = att * keep * D.threshold_and_scale(p)[1]
    ref = (att @ v).transpose(1, 2).reshape(B * T, C)
    ref.backward(dout.float())
    assert rel_err(out, ref) < 2e-2
    assert rel_err(dqkv, x.grad.reshape(B * T, 3 * C)) < 3e-2
    status_ok()


def test_mma_probe_reports_sane_costs(dev):
    """The tcgen05.mma cost probe runs to completion (its wait is bounded) and its figures keep the
    order the attention kernels are designed around: wider outputs cost more, an A operand in tensor
    memory costs less than one in shared memory."""
    from zero_to_hero_b200.utils.mma_probe import probe
    n64 = probe(0, 64, 0)["done_cycles_per_mma"]
    n256 = probe(2, 64, 0)["done_cycles_per_mma"]
    ts64 = probe(5, 64, 0)["done_cycles_per_mma"]
    assert 20 < ts64 < n64 < n256 < 400, (ts64, n64, n256)
    status_ok()


def test_ordered_kernels_repeat_bit_for_bit_and_match_the_default_ones(dev):
    """The fixed-order variants behind `train.deterministic`: embedding backward (one writer per
    vocabulary row, ascending position), column sums (one CTA per column block), attention backward
    (one KV tile per launch). Each equals the default kernel to rounding and itself bit for bit."""
    from zero_to_hero_b200.ops import native as N
    torch.manual_seed(11)
    # embedding: many repeats of few tokens, a vocabulary that is not a multiple of 8, C > 256
    B, T, C, V = 4, 300, 776, 203
    idx = torch.randint(0, 37, (B, T), device=dev)
    idx[0, :5] = V - 1
    dx = torch.randn(B * T, C, device=dev).bfloat16()
    ref = torch.zeros(V, C, device=dev).index_add_(0, idx.reshape(-1), dx.float())
    outs = []
    for _ in range(2):
        dwte = torch.zeros(V, C, device=dev)
        dwpe = torch.zeros(T, C, device=dev)
        N.embed_bwd(idx, dx, dwte, dwpe, B, T, ordered=True)
        outs.append(dwte)
    assert rel_err(outs[0], ref) < 1e-5 and torch.equal(outs[0], outs[1])
    # column sums
    dy = torch.randn(5000, 2304, device=dev).bfloat16()
    for scratch in (None, torch.full((N.colsum_scratch_elems(5000, 2304),), float("nan"), device=dev)):
        sums = []
        for _ in range(2):
            db = torch.ones(2304, device=dev)
            N.colsum_bf16(dy, db, ordered=True, scratch=scratch)  # one slab, or partial rows folded in order
            sums.append(db)
        assert rel_err(sums[0], 1 + dy.float().sum(0)) < 1e-5 and torch.equal(sums[0], sums[1])
    # attention backward
    B, T, H = 2, 520, 3
    C = H * 64
    qkv = (torch.randn(B * T, 3 * C, device=dev) * 0.7).bfloat16()
    out = torch.empty(B * T, C, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev)
    N.flash_fwd(qkv, out, lse, B, T, H)
    dout = (torch.randn(B * T, C, device=dev) * 0.5).bfloat16()
    dqa = torch.empty(N.flash_bwd_dq_elems(B, T, H), device=dev)
    stats = torch.empty(N.flash_bwd_stats_elems(B, T, H), device=dev)
    plain = torch.zeros_like(qkv)
    N.flash_bwd(qkv, out, dout, lse, plain, dqa, stats, B, T, H)
    grads = []
    for _ in range(2):
        d = torch.zeros_like(qkv)
        N.flash_bwd(qkv, out, dout, lse, d, dqa, stats, B, T, H, ordered=True)
        grads.append(d)
    assert torch.equal(grads[0], grads[1])
    assert rel_err(grads[0], plain) < 2e-3
    status_ok()


@pytest.mark.parametrize("split", [2, 5, 8])
def test_gemm_split_k_without_atomics_repeats_bit_for_bit(dev, split):
    """K-slices stored to their own copies of the output and folded in slice order: the sum equals the
    atomic split-K result to rounding and is the same bits on every run (a slice count that leaves the
    last slice without k-blocks included: it must contribute zeros, not stale memory)."""
    from zero_to_hero_b200.ops import gemm as G
    torch.manual_seed(split)
    K, M, N = 1024 + 64, 520, 776  # weight-gradient layout: A is [K, M], B is [K, N]
    A = (torch.randn(K, M, device=dev) * 0.5).bfloat16()
    B = (torch.randn(K, N, device=dev) * 0.5).bfloat16()
    start = torch.randn(M, N, device=dev)
    want = start + A.float().t() @ B.float()
    results = []
    for _ in range(2):
        ws = torch.full((split * M * N,), float("nan"), device=dev)
        G.gemm(A, B, ws[:M * N].view(M, N), a_mn=True, b_mn=True, epi=G.EPI_SLICE_STORE, split_k=split,
               slice_stride=M * N)
        out = start.clone()
        G.fold_slices(ws, split, out)
        results.append(out)
    assert torch.equal(results[0], results[1])
    assert rel_err(results[0], want) < 1e-4
    status_ok()
