"""MoE kernels and the expert-parallel layer against plain fp32 PyTorch references (single rank;
the multi-rank path runs in tests/mp_moe_worker.py when at least 2 GPUs are present)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_forward(x, gate, w13, w2, top_k, bias=None, idx=None):
    """fp32 reference. `idx` pins the expert choice (near-ties may flip between bf16 and fp32 logits)."""
    from fast_b200.models.moe import split_gate_up

    xf = x.float()
    logits = xf @ gate.float().t()
    if idx is None:
        sel = logits + (bias.float() if bias is not None else 0.0)
        idx = sel.topk(top_k, dim=-1).indices
    w = torch.softmax(logits.gather(1, idx), dim=-1)
    w1, w3 = split_gate_up(w13.float())
    out = torch.zeros_like(xf)
    for e in range(w13.shape[0]):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok]
        a = torch.nn.functional.silu(h @ w1[e].t()) * (h @ w3[e].t())
        out = out.index_add(0, tok, (a @ w2[e].float().t()) * w[tok, slot].unsqueeze(1))
    return out, idx, w


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()


@pytest.mark.parametrize("E,K", [(8, 2), (256, 8), (64, 6)])
def test_route_topk_matches_torch(E, K):
    from fast_b200 import runtime

    C = runtime.ext()
    T = 1000
    g = torch.Generator(device="cuda").manual_seed(E)
    logits = torch.randn(T, E, generator=g, device="cuda")
    bias = torch.randn(E, generator=g, device="cuda") * 1.5
    nb = (T + C.ROUTE_TOKENS_PER_BLOCK - 1) // C.ROUTE_TOKENS_PER_BLOCK
    idx = torch.empty(T, K, dtype=torch.int32, device="cuda")
    w = torch.empty(T, K, dtype=torch.float32, device="cuda")
    slot = torch.zeros(nb * C.ROUTE_TOKENS_PER_BLOCK, K, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(nb, E, dtype=torch.int32, device="cuda")
    C.route_topk(logits, bias, K, idx, w, slot, cnt)
    ref_idx = (logits + bias).topk(K, dim=-1).indices
    assert torch.equal(idx.long(), ref_idx)
    ref_w = torch.softmax(logits.gather(1, ref_idx), dim=-1)
    assert torch.allclose(w, ref_w, atol=1e-5)
    # histogram and stable in-block ranks
    for b in range(nb):
        blk = idx[b * 128:(b + 1) * 128].reshape(-1).long()
        assert torch.equal(cnt[b].long(), torch.bincount(blk, minlength=E))
    flat = idx.reshape(-1).cpu()
    s = slot[:T].reshape(-1).cpu()
    seen = {}
    for i in range(min(flat.numel(), 128 * K)):
        e = int(flat[i])
        assert int(s[i]) == seen.get(e, 0)
        seen[e] = seen.get(e, 0) + 1


def test_route_topk_is_total_on_nan_inf_and_masked_rows():
    """Rows of NaN, of -inf, or with fewer than K selectable experts still get K distinct ids inside
    [0, E) and finite weights; rows with enough finite values route exactly like PyTorch."""
    from fast_b200 import runtime

    C = runtime.ext()
    T, E, K = 256, 64, 6
    g = torch.Generator(device="cuda").manual_seed(9)
    logits = torch.randn(T, E, generator=g, device="cuda")
    logits[0] = float("nan")
    logits[1] = float("-inf")
    logits[2, 3:] = float("-inf")            # three selectable experts, K = 6
    logits[3, ::2] = float("nan")            # half the experts unusable, still >= K finite
    logits[4, 5] = float("inf")
    idx = torch.empty(T, K, dtype=torch.int32, device="cuda")
    w = torch.empty(T, K, dtype=torch.float32, device="cuda")
    slot = torch.zeros(256, K, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(2, E, dtype=torch.int32, device="cuda")
    C.route_topk(logits, None, K, idx, w, slot, cnt)
    torch.cuda.synchronize()
    assert int(idx.min()) >= 0 and int(idx.max()) < E
    assert all(len(set(r)) == K for r in idx[:8].cpu().tolist())
    assert bool(torch.isfinite(w[[0, 1, 2, 3] + list(range(5, T))]).all())
    assert float(w[0].abs().sum()) == 0.0 and float(w[1].abs().sum()) == 0.0
    assert sorted(idx[2, :3].cpu().tolist()) == [0, 1, 2] and abs(float(w[2, :3].sum()) - 1.0) < 1e-5 and float(w[2, 3:].abs().sum()) == 0.0
    assert all(e % 2 == 1 for e in idx[3].cpu().tolist())
    ref = logits[5:].topk(K, dim=-1).indices
    assert torch.equal(idx[5:].long(), ref)
    assert int(cnt.sum()) == T * K


def test_expert_ids_out_of_range_are_skipped_and_reported():
    """Routing tables that name an expert outside [0, E) (a caller's own router gone wrong) are not
    used as indices: the entries are skipped, the status block names the site, the context lives."""
    from fast_b200 import runtime
    from fast_b200.models import MoELayer
    from fast_b200.parallel import Communicator

    comm = Communicator(heap_bytes=128 << 20, device=0)
    layer = MoELayer(comm, 256, 256, 4, 2, max_tokens=512, training=False)
    eng = layer.engine
    x = torch.randn(300, 256, device="cuda").to(torch.bfloat16)
    rs = eng.route((x @ layer.gate.t()).float())
    rs.topk_idx[7, 1] = 0x7FFFFFFF
    rs.topk_idx[9, 0] = -3
    eng.dispatch(x, rs)
    with pytest.raises(runtime.CollectiveTimeout) as e:
        comm.check()
    assert e.value.code == 2 and e.value.site == 11 and e.value.want == 4
    comm.reset()
    out = torch.empty(300, 256, dtype=torch.bfloat16, device="cuda")
    eng._C.combine_pull(comm.heap, eng.E, rs.topk_idx, rs.dest_row, rs.topk_w, eng._off(eng.y), eng._flag_off(1), 0, out, None, None, eng.H, eng.status,
                        eng.timeout_ns, 8, 0)
    with pytest.raises(runtime.CollectiveTimeout) as e:
        comm.check()
    assert e.value.site == 11
    assert int((torch.ones(8, device="cuda") * 3).sum().item()) == 24  # context still healthy


@pytest.mark.parametrize("T,H,E,K", [(300, 256, 8, 2), (1000, 512, 32, 6), (129, 1024, 4, 1)])
def test_fused_norm_router_forward_and_backward_match_torch(T, H, E, K):
    """RMSNorm + router logits + top-k (+ softmax-over-top-k weights) in one kernel, and its backward
    (gate, norm-weight and input gradients), against the same chain of plain fp32 PyTorch ops."""
    from fast_b200 import runtime

    C = runtime.ext()
    g = torch.Generator(device="cuda").manual_seed(T + E)
    h = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    nw = (1.0 + 0.1 * torch.randn(H, generator=g, device="cuda")).to(torch.bfloat16)
    gate = (torch.randn(E, H, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    nb = (T + C.ROUTE_TOKENS_PER_BLOCK - 1) // C.ROUTE_TOKENS_PER_BLOCK
    hn = torch.empty_like(h)
    rstd = torch.empty(T, device="cuda")
    logits = torch.empty(T, E, device="cuda")
    idx = torch.empty(T, K, dtype=torch.int32, device="cuda")
    w = torch.empty(T, K, device="cuda")
    slot = torch.zeros(nb * C.ROUTE_TOKENS_PER_BLOCK, K, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(nb, E, dtype=torch.int32, device="cuda")
    eps = 1e-5
    C.norm_gate_route(h, nw, gate, None, K, eps, hn, rstd, logits, idx, w, slot, cnt)
    # fp32 reference with autograd; the expert choice is pinned to the kernel's (near-ties may flip)
    hr = h.float().requires_grad_()
    nwr = nw.float().requires_grad_()
    gr = gate.float().requires_grad_()
    hn_ref = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + eps) * nwr
    lg_ref = hn_ref @ gr.t()
    assert _rel(hn, hn_ref) < 1e-2 and _rel(logits, lg_ref) < 1e-2
    top_ref = lg_ref.topk(K, dim=-1)
    agree = (idx.long().sort(-1).values == top_ref.indices.sort(-1).values).all(-1).float().mean().item()
    assert agree > 0.98                                       # bf16 rounding of hn may flip near-ties
    assert int(idx.min()) >= 0 and int(idx.max()) < E and int(cnt.sum()) == T * K
    w_ref = torch.softmax(lg_ref.gather(1, idx.long()), dim=-1)
    assert torch.allclose(w, w_ref, atol=2e-2)
    for b in range(nb):
        blk = idx[b * 128:(b + 1) * 128].reshape(-1).long()
        assert torch.equal(cnt[b].long(), torch.bincount(blk, minlength=E))
    # backward: loss = sum(w * gw) + sum(hn * ghn)
    gw = torch.randn(T, K, generator=g, device="cuda")
    ghn = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    ((w_ref * gw).sum() + (hn_ref * ghn.float()).sum()).backward()
    grad_h = torch.empty_like(h)
    d_gate = torch.zeros(E, H, device="cuda")
    d_nw = torch.zeros(H, device="cuda")
    C.norm_gate_bwd(h, nw, gate, rstd, idx, w, gw, ghn, grad_h, d_gate, d_nw)
    assert _rel(grad_h, hr.grad) < 2e-2
    assert _rel(d_gate, gr.grad) < 2e-2
    assert _rel(d_nw, nwr.grad) < 2e-2


def test_elementwise_kernels():
    from fast_b200 import runtime
    from fast_b200.models.moe import split_gate_up

    C = runtime.ext()
    g = torch.Generator(device="cuda").manual_seed(1)
    rows, inter = 300, 384
    gu = torch.randn(rows, 2 * inter, generator=g, device="cuda").to(torch.bfloat16)
    act = torch.empty(rows, inter, device="cuda", dtype=torch.bfloat16)
    C.swiglu_fwd(gu, act)
    gt, ut = split_gate_up(gu.float().t().reshape(1, 2 * inter, rows))
    gt, ut = gt[0].t().requires_grad_(), ut[0].t().requires_grad_()
    ref = torch.nn.functional.silu(gt) * ut
    assert _rel(act, ref) < 1e-2
    dact = torch.randn(rows, inter, generator=g, device="cuda").to(torch.bfloat16)
    dgu = torch.empty_like(gu)
    C.swiglu_bwd(gu, dact, dgu, 0)
    ref.backward(dact.float())
    dg, du = split_gate_up(dgu.float().t().reshape(1, 2 * inter, rows))
    assert _rel(dg[0].t(), gt.grad) < 1e-2 and _rel(du[0].t(), ut.grad) < 1e-2
    # AdamW against torch.optim.AdamW on fp32
    p = torch.randn(4096, generator=g, device="cuda")
    grad = torch.randn(4096, generator=g, device="cuda").to(torch.bfloat16)
    pb = p.to(torch.bfloat16)
    master, m, v = pb.float().clone(), torch.zeros(4096, device="cuda"), torch.zeros(4096, device="cuda")
    ref_p = pb.float().clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in (1, 2, 3):
        C.adamw(pb, master, m, v, grad, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0)
        ref_p.grad = grad.float()
        opt.step()
    assert torch.allclose(master, ref_p.detach(), atol=1e-5, rtol=1e-5)
    assert torch.equal(pb, master.to(torch.bfloat16))


def test_quantise_rows_matches_a_torch_restatement():
    """Rows to e4m3 in 1 x 128 blocks: the scale is amax / 448 rounded up to a bf16 value, the bytes are
    round-to-nearest e4m3 of value / scale; value x scale comes back within e4m3's half-ulp."""
    from fast_b200 import runtime

    C = runtime.ext()
    g = torch.Generator(device="cuda").manual_seed(3)
    T, H = 77, 768
    x = (torch.randn(T, H, generator=g, device="cuda") * torch.logspace(-3, 2, T, device="cuda").unsqueeze(1)).to(torch.bfloat16)
    x[5, 128:256] = 0  # an all-zero block keeps a tiny positive scale
    q = torch.empty(T, H, dtype=torch.uint8, device="cuda")
    sc = torch.empty(T, H // 128, dtype=torch.float32, device="cuda")
    C.quantise_rows(x, q, sc, 8)
    blocks = x.float().reshape(T, H // 128, 128)
    want = blocks.abs().amax(-1).clamp_min(1e-12) / 448.0
    want = ((want.view(torch.int32) + 0xFFFF) & -65536).view(torch.float32)  # up to the next bf16 value
    assert torch.equal(sc, want)
    ref_q = (blocks / want.unsqueeze(-1)).to(torch.float8_e4m3fn)
    got = q.view(torch.float8_e4m3fn).reshape(T, H // 128, 128)
    # the kernel multiplies by a reciprocal: a value on a rounding boundary may land one code away
    assert (got.float() != ref_q.float()).float().mean().item() < 1e-3
    back = got.float() * sc.unsqueeze(-1)
    assert ((back - blocks).abs() <= blocks.abs().amax(-1, keepdim=True) * (1.0 / 14) + 1e-12).all()
    assert torch.count_nonzero(back[5, 1]) == 0


def test_embedding_index_is_a_stable_sort_by_id():
    """The counting sort that feeds the embedding gradient equals torch's stable sort, with few and with heavy duplicates."""
    from fast_b200 import runtime

    C = runtime.ext()
    g = torch.Generator(device="cuda").manual_seed(11)
    for T, V, hot in ((5000, 3000, 0), (4097, 70000, 0), (3000, 50, 0), (2500, 1000, 2000)):
        ids = torch.randint(0, V, (T,), generator=g, device="cuda")
        if hot:
            ids[torch.randperm(T, generator=g, device="cuda")[:hot]] = 7     # one id taking most of the positions
        sid, perm = C.embedding_index(ids, V)
        rs, rp = torch.sort(ids, stable=True)
        assert torch.equal(sid, rs) and torch.equal(perm, rp)


def test_fused_embedding_and_loss_match_torch():
    from fast_b200.ops import fused

    g = torch.Generator(device="cuda").manual_seed(5)
    table = (torch.randn(300, 256, generator=g, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    ids = torch.randint(0, 300, (4, 500), generator=g, device="cuda")
    other = (torch.randn(2000, 256, generator=g, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    loss = fused.residual_mean_square(fused.embedding(ids.reshape(-1), table), other)
    loss.backward()
    t2 = table.detach().clone().requires_grad_()
    o2 = other.detach().clone().requires_grad_()
    ref = (torch.nn.functional.embedding(ids.reshape(-1), t2) + o2).float().pow(2).mean()
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-3 * abs(ref.item())
    assert _rel(other.grad, o2.grad) < 2e-2
    assert _rel(table.grad, t2.grad) < 2e-2


@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("E,K,H,I,T,fp8", [(4, 2, 256, 256, 300, False), (8, 2, 512, 384, 1000, False), (32, 8, 256, 128, 513, False), (8, 2, 256, 256, 300, True),
                                           (8, 2, 256, 256, 300, "direct")])
def test_moe_forward_single_rank(E, K, H, I, T, fp8, overlap):
    from fast_b200.models import MoELayer
    from fast_b200.parallel import Communicator

    comm = Communicator(heap_bytes=256 << 20, device=0)
    layer = MoELayer(comm, H, I, E, K, max_tokens=1024, fp8_dispatch=bool(fp8), training=False, router_bias=True, overlap_dispatch=overlap,
                     fp8_direct=fp8 == "direct")
    layer.eval()
    g = torch.Generator(device="cuda").manual_seed(7)
    layer.router_bias.data = torch.randn(E, generator=g, device="cuda") * 0.5
    x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        out = layer(x)
        out2 = layer(x)  # second call: epochs, counters and pads must be reusable
    comm.check()
    ref, _, _ = _ref_forward(x, layer.gate, layer.w13, layer.w2, K, layer.router_bias, idx=layer.last_route.topk_idx.long())
    tol = 6e-2 if fp8 else 2e-2
    assert _rel(out, ref) < tol
    assert torch.equal(out, out2)
    tm = layer.engine.traffic_matrix()
    assert int(tm.sum().item()) == T * K


def test_forward_layer_in_cuda_graph():
    """The forward-only layer captured in a CUDA graph replays correctly on new inputs (the step's
    epoch lives in device memory, so a replay is a new step)."""
    from fast_b200.models import MoELayer
    from fast_b200.parallel import Communicator

    E, K, H, I, T = 8, 2, 256, 256, 384
    comm = Communicator(heap_bytes=256 << 20, device=0)
    layer = MoELayer(comm, H, I, E, K, max_tokens=512, training=False, graph_mode=True)
    layer.eval()
    layer.capture(T)
    g = torch.Generator(device="cuda").manual_seed(21)
    for it in range(3):
        x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
        out = layer.forward_graphed(x).clone()
        comm.check()
        ref, _, _ = _ref_forward(x, layer.gate, layer.w13, layer.w2, K, idx=layer.last_route.topk_idx[:T].long())
        assert _rel(out, ref) < 2e-2, f"replay {it}"
    assert int(layer.engine.epoch_dev.item()) == 2 + 3  # two warm-up steps + three replays


def test_receive_capacity_guard_refuses_step():
    """A step that needs more receive rows than the buffers hold is refused on the device
    (no row is written out of bounds) and reported through the status block."""
    from fast_b200 import runtime
    from fast_b200.models import MoELayer
    from fast_b200.parallel import Communicator

    comm = Communicator(heap_bytes=128 << 20, device=0)
    layer = MoELayer(comm, 256, 256, 4, 2, max_tokens=1024, training=False, capacity_rows=512)
    layer.eval()
    x = torch.randn(900, 256, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        layer(x)  # needs ~1800 rows (+ padding) > 512
    with pytest.raises(runtime.CollectiveTimeout) as e:
        comm.check()
    assert e.value.site == 10 and e.value.want == 512 and e.value.seen > 512
    assert int((torch.ones(8, device="cuda") * 3).sum().item()) == 24  # context still healthy


def test_moe_backward_single_rank():
    from fast_b200.models import MoELayer
    from fast_b200.parallel import Communicator

    E, K, H, I, T = 8, 2, 256, 256, 600
    comm = Communicator(heap_bytes=256 << 20, device=0)
    layer = MoELayer(comm, H, I, E, K, max_tokens=1024)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16).requires_grad_()
    gout = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    out = layer(x)
    out.backward(gout)
    comm.check()
    # fp32 reference with autograd
    xr = x.detach().float().requires_grad_()
    gate = layer.gate.detach().float().requires_grad_()
    w13 = layer.w13.detach().float().requires_grad_()
    w2 = layer.w2.detach().float().requires_grad_()
    ref, _, _ = _ref_forward(xr, gate, w13, w2, K, idx=layer.last_route.topk_idx.long())
    ref.backward(gout.float())
    assert _rel(out, ref) < 2e-2
    assert _rel(x.grad, xr.grad) < 3e-2
    assert _rel(layer.w13.grad, w13.grad) < 3e-2
    assert _rel(layer.w2.grad, w2.grad) < 3e-2
    assert _rel(layer.gate.grad, gate.grad) < 5e-2


def test_block_model_trains():
    from fast_b200.models import MixtralBlockModel
    from fast_b200.parallel import Communicator
    from fast_b200.utils import FusedAdamW

    comm = Communicator(heap_bytes=256 << 20, device=0)
    model = MixtralBlockModel(comm, vocab=512, hidden=256, inter=256, num_experts=4, top_k=2, max_tokens=512)
    opt = FusedAdamW(model.expert_parameters(), lr=5e-3)
    ids = torch.randint(0, 512, (2, 256), device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = model(ids)
        loss.backward()
        opt.step()
        losses.append(float(loss.item()))
    comm.check()
    assert all(l == l for l in losses) and losses[-1] < losses[0]


def test_optimizer_in_backward_matches_late_step():
    """Applying W2's AdamW update inside the backward pass (side stream) gives bit-identical weights."""
    from fast_b200.models import MixtralBlockModel
    from fast_b200.parallel import Communicator
    from fast_b200.utils import FusedAdamW

    ids = torch.randint(0, 512, (2, 256), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    results = []
    for early in (False, True):
        comm = Communicator(heap_bytes=256 << 20, device=0)
        model = MixtralBlockModel(comm, vocab=512, hidden=256, inter=256, num_experts=4, top_k=2, max_tokens=512, seed=3)
        opt = FusedAdamW(model.expert_parameters(), lr=1e-2)
        if early:
            model.moe.attach_optimizer(opt)
        for _ in range(3):
            opt.zero_grad()
            model(ids).backward()
            opt.step()
        comm.check()
        torch.cuda.synchronize()
        results.append((model.moe.w13.detach().clone(), model.moe.w2.detach().clone()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    assert not torch.equal(results[0][1], torch.zeros_like(results[0][1]))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_moe_multi_process():
    n = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                        "--master-port", "29543", os.path.join(os.path.dirname(__file__), "mp_moe_worker.py")], capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MOE_MP_OK" in r.stdout
