"""One tiny forward+backward+optimizer step of the MoE block model on cuda:0 (single rank)."""
import torch


def run_smoke():
    from ..parallel import Communicator
    from ..utils import FusedAdamW
    from . import MixtralBlockModel

    torch.cuda.set_device(0)
    comm = Communicator(heap_bytes=256 << 20, device=0)
    model = MixtralBlockModel(comm, vocab=1024, hidden=256, inter=256, num_experts=4, top_k=2, max_tokens=512)
    opt = FusedAdamW(model.expert_parameters(), lr=1e-3)
    ids = torch.randint(0, 1024, (2, 256), device="cuda")
    loss = model(ids)
    loss.backward()
    opt.step()
    comm.check()
    val = float(loss.item())
    assert val == val and val > 0.0, "smoke loss is not a positive finite number"
    print(f"smoke ok: loss={val:.6f}")
