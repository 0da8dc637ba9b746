"""Child of test_moe_multi_process: expert-parallel forward/backward on real peers vs a full
single-device fp32 reference built from the gathered expert weights."""
import os
import sys

os.environ.setdefault("FASTB_CHECK_SYMM", "1")  # every symmetric allocation is compared across the ranks (read at import)

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fast_b200.models import MoELayer  # noqa: E402
from fast_b200.parallel import Communicator  # noqa: E402
from tests.test_moe_gpu import _ref_forward, _rel  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    comm = Communicator(heap_bytes=512 << 20)
    for ci, (E, K, H, I, T, fp8) in enumerate([(8, 2, 256, 256, 700, False), (16, 4, 512, 256, 333 + 17 * rank, False), (8, 2, 256, 256, 500, True)]):
        layer = MoELayer(comm, H, I, E, K, max_tokens=1024, fp8_dispatch=fp8, training=not fp8, overlap_dispatch=(ci == 1))
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16).requires_grad_(not fp8)
        gout = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
        # full weights everywhere for the reference
        w13_all = [torch.empty_like(layer.w13.data) for _ in range(world)]
        w2_all = [torch.empty_like(layer.w2.data) for _ in range(world)]
        dist.all_gather(w13_all, layer.w13.data)
        dist.all_gather(w2_all, layer.w2.data)
        w13_all, w2_all = torch.cat(w13_all), torch.cat(w2_all)
        if fp8:
            layer.eval()
            with torch.no_grad():
                out = layer(x)
            comm.check()
            ref, _, _ = _ref_forward(x, layer.gate, w13_all, w2_all, K, idx=layer.last_route.topk_idx.long())
            assert _rel(out, ref) < 6e-2, f"fp8 forward rank {rank}: {_rel(out, ref)}"
            continue
        for it in range(2):
            x.grad = None
            layer.zero_grad()
            out = layer(x)
            out.backward(gout)
        comm.check()
        xr = x.detach().float().requires_grad_()
        gate = layer.gate.detach().float().requires_grad_()
        w13r, w2r = w13_all.float().requires_grad_(), w2_all.float().requires_grad_()
        ref, _, _ = _ref_forward(xr, gate, w13r, w2r, K, idx=layer.last_route.topk_idx.long())
        ref.backward(gout.float())
        assert _rel(out, ref) < 2e-2, f"forward rank {rank}: {_rel(out, ref)}"
        assert _rel(x.grad, xr.grad) < 3e-2, f"dx rank {rank}"
        # expert grads: sum over ranks of the reference grads restricted to my experts
        g13, g2 = w13r.grad.clone(), w2r.grad.clone()
        dist.all_reduce(g13)
        dist.all_reduce(g2)
        El = E // world
        assert _rel(layer.w13.grad, g13[rank * El:(rank + 1) * El]) < 3e-2, f"dw13 rank {rank}"
        assert _rel(layer.w2.grad, g2[rank * El:(rank + 1) * El]) < 3e-2, f"dw2 rank {rank}"
        plan, cost = layer.engine.plan_last_step()
        assert plan.validate() == "" and int(plan.matrix.sum()) == int(layer.engine.traffic_matrix().sum().item()) * H * 2
        assert cost["total_us"] >= cost["lower_bound_us"] > 0
        dist.barrier()
    if rank == 0:
        print("MOE_MP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
