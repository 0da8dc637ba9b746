"""tcgen05 grouped GEMM against a plain PyTorch fp32 reference of the same contraction."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["one_cta", "cta_pair"], autouse=True)
def kernel_variant(request):
    """Every case runs on the one-CTA kernel and on the CTA-pair (cta_group::2) kernel."""
    from fast_b200.ops import gemm

    old = gemm.USE_PAIR
    gemm.USE_PAIR = request.param == "cta_pair"
    yield request.param
    gemm.USE_PAIR = old


def _setup(G, N, K, counts, seed=0):
    from fast_b200.ops import pad_group_offsets

    g = torch.Generator(device="cuda").manual_seed(seed)
    counts = torch.tensor(counts, device="cuda")
    off = pad_group_offsets(counts)
    R = int(off[-1].item())
    a = torch.zeros(R, K, device="cuda", dtype=torch.bfloat16)
    for i in range(G):
        s, c = int(off[i]), int(counts[i])
        a[s:s + c] = torch.randn(c, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(G, N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    return counts, off, R, a, w


def _close(got, want, tol=2e-2):
    if want.numel() == 0:
        return
    err = (got.float() - want).abs().max().item()
    scale = want.abs().max().item() + 1e-6
    assert err / scale < tol, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("G,N,K,counts", [(1, 256, 64, [128]), (1, 256, 256, [128]), (2, 512, 320, [200, 77]), (4, 768, 512, [0, 300, 128, 1])])
def test_forward(G, N, K, counts):
    from fast_b200.ops import gemm

    counts, off, R, a, w = _setup(G, N, K, counts)
    out = torch.full((R, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_fwd(a, w, off, out)
    gemm.check()
    for i in range(G):
        s, e = int(off[i]), int(off[i + 1])
        _close(out[s:e], a[s:e].float() @ w[i].float().T)


def test_forward_swiglu():
    from fast_b200.ops import gemm

    G, N, K = 2, 512, 256
    counts, off, R, a, w = _setup(G, N, K, [130, 256], seed=3)
    act = torch.empty(R, N // 2, device="cuda", dtype=torch.bfloat16)
    gu = torch.empty(R, N, device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_fwd(a, w, off, act, swiglu=True, gate_up_out=gu)
    gemm.check()
    for i in range(G):
        s, e = int(off[i]), int(off[i + 1])
        full = a[s:e].float() @ w[i].float().T
        _close(gu[s:e], full)
        t = full.view(e - s, N // 256, 2, 128)
        _close(act[s:e], (torch.nn.functional.silu(t[:, :, 0]) * t[:, :, 1]).reshape(e - s, N // 2))


@pytest.mark.parametrize("G,N,K,counts", [(1, 64, 256, [128]), (2, 320, 512, [200, 77]), (3, 512, 768, [1, 0, 257])])
def test_dgrad(G, N, K, counts):
    from fast_b200.ops import gemm

    counts, off, R, dy, w = _setup(G, K, N, counts, seed=5)  # dy [R, N]; w [G, N, K]
    w = w.transpose(1, 2).contiguous()  # [G, N, K]
    out = torch.full((R, K), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_dgrad(dy, w, off, out)
    gemm.check()
    for i in range(G):
        s, e = int(off[i]), int(off[i + 1])
        _close(out[s:e], dy[s:e].float() @ w[i].float())


@pytest.mark.parametrize("G,N,K,counts", [(1, 256, 256, [128]), (2, 256, 512, [200, 77]), (3, 512, 256, [1, 0, 257])])
def test_wgrad(G, N, K, counts):
    from fast_b200.ops import gemm

    counts, off, R, x, _ = _setup(G, 256, K, counts, seed=7)
    g = torch.Generator(device="cuda").manual_seed(11)
    dy = torch.zeros(R, N, device="cuda", dtype=torch.bfloat16)
    for i in range(G):
        s, c = int(off[i]), int(counts[i])
        dy[s:s + c] = torch.randn(c, N, generator=g, device="cuda").to(torch.bfloat16)
    out = torch.full((G, N, K), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_wgrad(dy, x, off, out)
    gemm.check()
    for i in range(G):
        s, e = int(off[i]), int(off[i + 1])
        _close(out[i], dy[s:e].float().T @ x[s:e].float())


def test_large_shape_matches():
    from fast_b200.ops import gemm

    G, N, K = 2, 2048, 1024
    counts, off, R, a, w = _setup(G, N, K, [1500, 900], seed=9)
    out = torch.empty(R, N, device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_fwd(a, w, off, out)
    gemm.check()
    for i in range(G):
        s, e = int(off[i]), int(off[i + 1])
        _close(out[s:e], a[s:e].float() @ w[i].float().T)


def test_dgrad_with_fused_swiglu_backward(kernel_variant):
    """dgrad of the second projection with the SwiGLU backward applied in its epilogue."""
    if kernel_variant != "cta_pair":
        pytest.skip("only the CTA-pair kernel carries this epilogue")
    from fast_b200.ops import gemm

    G, H, I = 2, 256, 512
    counts, off, R, dy, _ = _setup(G, 256, H, [300, 200], seed=13)  # dy [R, H]
    g = torch.Generator(device="cuda").manual_seed(17)
    w2 = (torch.randn(G, H, I, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    gu = torch.randn(R, 2 * I, generator=g, device="cuda").to(torch.bfloat16)
    dgu = torch.full((R, 2 * I), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_dgrad(dy, w2, off, dgu, swiglu_bwd_of=gu)
    gemm.check()
    for i in range(G):
        s, e = int(off[i]), int(off[i + 1])
        dact = (dy[s:e].float() @ w2[i].float()).to(torch.bfloat16).float()
        t = gu[s:e].float().view(e - s, I // 128, 2, 128)
        gt, ut = t[:, :, 0].reshape(e - s, I).requires_grad_(), t[:, :, 1].reshape(e - s, I).requires_grad_()
        (torch.nn.functional.silu(gt) * ut).backward(dact)
        got = dgu[s:e].float().view(e - s, I // 128, 2, 128)
        _close(got[:, :, 0].reshape(e - s, I), gt.grad)
        _close(got[:, :, 1].reshape(e - s, I), ut.grad)


def test_custom_operators_run_the_same_kernels():
    """torch.ops.fast_b200.* (schemas, mutation annotations) give the same bits as the direct calls."""
    from fast_b200.ops import gemm, registry  # noqa: F401

    G, N, K = 2, 512, 256
    counts, off, R, a, w = _setup(G, N, K, [200, 77], seed=5)
    direct = torch.zeros(R, N, device="cuda", dtype=torch.bfloat16)
    via_op = torch.zeros(R, N, device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_fwd(a, w, off, direct)
    torch.ops.fast_b200.grouped_gemm_fwd(a, w, off, via_op, False, None)
    gemm.check()
    assert torch.equal(direct, via_op)
    dx1, dx2 = torch.zeros_like(a), torch.zeros_like(a)
    gemm.grouped_gemm_dgrad(direct, w, off, dx1)
    torch.ops.fast_b200.grouped_gemm_dgrad(direct, w, off, dx2, None)
    dw1, dw2 = torch.zeros_like(w), torch.zeros_like(w)
    gemm.grouped_gemm_wgrad(direct, a, off, dw1)
    torch.ops.fast_b200.grouped_gemm_wgrad(direct, a, off, dw2)
    gemm.check()
    assert torch.equal(dx1, dx2) and torch.equal(dw1, dw2)
    logits = torch.randn(300, 16, device="cuda")
    idx, wts = torch.ops.fast_b200.route_topk(logits, None, 2)
    ref = torch.softmax(logits, -1).topk(2, dim=-1)
    assert torch.equal(idx.long(), ref.indices) and torch.allclose(wts, ref.values / ref.values.sum(-1, keepdim=True), atol=1e-5)


def _quant_e4m3_1x128(a):
    """bf16 [R, K] -> (uint8 e4m3 [R, K], fp32 scales [R, K/128]) with amax / 448 scales, and the dequantised fp32 matrix
    (rounded to bf16, which is what the kernel feeds the tensor core)."""
    R, K = a.shape
    g = a.float().view(R, K // 128, 128)
    sc = g.abs().amax(-1).clamp_min(1e-12) / 448.0
    sc = ((sc.view(torch.int32) + 0xFFFF) & ~0xFFFF).view(torch.float32)   # rounded up to bf16 precision, as the dispatch kernel does
    q = (g / sc.unsqueeze(-1)).to(torch.float8_e4m3fn)
    deq = (q.float() * sc.unsqueeze(-1)).to(torch.bfloat16).float().view(R, K)
    return q.view(R, K).view(torch.uint8).contiguous(), sc.contiguous(), deq


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("G,N,K,counts", [(1, 256, 128, [256]), (2, 512, 384, [200, 77]), (4, 768, 512, [0, 300, 128, 1])])
def test_forward_from_e4m3_rows(G, N, K, counts, swiglu, kernel_variant):
    """Operand A as e4m3 bytes + 1x128 scales, converted to bf16 tiles inside the kernel: equals the
    product of the dequantised matrix; rows past a group's real end count as zeros even when the
    buffer holds stale bytes and scales there."""
    if kernel_variant != "cta_pair":
        pytest.skip("the e4m3 operand feed belongs to the CTA-pair kernel")
    from fast_b200.ops import gemm

    counts_t, off, R, a, w = _setup(G, N, K, counts, seed=5)
    q, sc, deq = _quant_e4m3_1x128(a)
    # stale content in the pad rows: must not leak into anything
    real = torch.zeros(R, dtype=torch.bool, device="cuda")
    for i in range(G):
        real[int(off[i]):int(off[i]) + int(counts_t[i])] = True
    q[~real] = 0x7E                       # 448 in e4m3
    sc[~real] = 3.0e38
    out = torch.full((R, N // 2 if swiglu else N), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_fwd(q, w, off, out, swiglu=swiglu, a_scales=sc, group_rows=counts_t.to(torch.int32))
    gemm.check()
    for i in range(G):
        s, e = int(off[i]), int(off[i + 1])
        full = (deq[s:e] * real[s:e].unsqueeze(1)) @ w[i].float().T
        if swiglu:
            t = full.view(e - s, N // 256, 2, 128)
            full = (torch.nn.functional.silu(t[:, :, 0]) * t[:, :, 1]).reshape(e - s, N // 2)
        _close(out[s:e], full)
        assert float(out[s + int(counts_t[i]):e].float().abs().max() if e > s + int(counts_t[i]) else 0.0) == 0.0
