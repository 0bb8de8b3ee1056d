"""Worker for the multi-GPU tests (launched with torch.distributed.run): trains the same model with the
peer-memory sharded engine (multimem and unicast flavours, mask and sparse labels), the collective-based sharded
engine and — on rank 0 — the single-GPU engine on the
concatenated batch, and checks that losses and final tables agree."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dice_embeddings_b200.data.datasets import KvsAll  # noqa: E402
from dice_embeddings_b200.data.synthetic import zipf_kg  # noqa: E402
from dice_embeddings_b200.models import initialize_model  # noqa: E402
from dice_embeddings_b200.ops.fused_step import FusedKvsAllEngine  # noqa: E402
from dice_embeddings_b200.parallel.sharded_engine import ShardedKvsAllEngine  # noqa: E402


def main():
    name = sys.argv[1] if len(sys.argv) > 1 else "ComplEx"
    optim = sys.argv[2] if len(sys.argv) > 2 else "SGD"
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    W = dist.get_world_size()
    NE, NR, D, B, steps = 1003, 17, 128, 256, 4
    lr = 50.0 if optim == "SGD" else 0.02
    tr = zipf_kg(NE, NR, 6000, seed=0)

    def make():
        torch.manual_seed(0)
        m, _ = initialize_model(dict(model=name, embedding_dim=D, num_entities=NE, num_relations=NR, optim=optim,
                                     learning_rate=lr, scoring_technique="KvsAll", p=0, q=1))
        m.to(dev)
        with torch.no_grad():
            m.entity_embeddings.weight.mul_(0.3)
            m.relation_embeddings.weight.mul_(0.3)
            if name == "Keci":
                m.q_coefficients.weight.fill_(0.5)
        return m

    g = torch.Generator().manual_seed(5)
    results = {}
    mm_used = None
    for comm in ("p2p", "p2p-unicast", "p2p-sparse", "nccl"):
        ds = KvsAll(tr, NE, NR, label_smoothing_rate=0.1).to(dev)
        model = make()
        eng = ShardedKvsAllEngine(model, ds, batch_size=B, lr=lr, device=dev, comm=comm.split("-")[0],
                                  label_mode="sparse" if comm.endswith("sparse") else None,
                                  multimem=False if comm.endswith("unicast") else None)
        if comm == "p2p":
            mm_used = eng.multimem
        g.manual_seed(5)
        losses = []
        for _ in range(steps):
            idx_all = torch.randperm(len(ds), generator=g)[: W * B]
            idx = idx_all[rank * B:(rank + 1) * B].to(dev)
            losses.append(float(eng.step((ds.train_data[idx], idx))))
        eng.sync_to_model()
        results[comm] = (losses, model.entity_embeddings.weight.detach().clone(),
                         model.relation_embeddings.weight.detach().clone())
    ok = True
    msg = []
    lp, ep, rp = results["p2p"]
    ln, en, rn = results["nccl"]
    for a, b in zip(lp, ln):
        ok &= abs(a - b) < 2e-3 * abs(b) + 1e-6
    d_e = (ep - en).abs().max().item() / en.abs().max().item()
    d_r = (rp - rn).abs().max().item() / rn.abs().max().item()
    ok &= d_e < 2e-2 and d_r < 2e-2
    msg.append(f"p2p vs nccl: losses {lp} / {ln}; rel diff E {d_e:.2e} R {d_r:.2e}")
    lu, eu, ru = results["p2p-unicast"]
    for a, b in zip(lu, lp):
        ok &= abs(a - b) < 2e-3 * abs(b) + 1e-6
    d_e = (eu - ep).abs().max().item() / ep.abs().max().item()
    d_r = (ru - rp).abs().max().item() / rp.abs().max().item()
    ok &= d_e < 2e-2 and d_r < 2e-2
    msg.append(f"multimem ({'on' if mm_used else 'unavailable: both runs unicast'}) vs unicast: losses {lp} / {lu}; "
               f"rel diff E {d_e:.2e} R {d_r:.2e}")
    lsp, esp, rsp = results["p2p-sparse"]
    for a, b in zip(lsp, lp):
        ok &= abs(a - b) < 2e-3 * abs(b) + 1e-6
    d_e = (esp - ep).abs().max().item() / ep.abs().max().item()
    d_r = (rsp - rp).abs().max().item() / rp.abs().max().item()
    ok &= d_e < 2e-2 and d_r < 2e-2
    msg.append(f"sparse labels vs label masks: losses {lsp} / {lp}; rel diff E {d_e:.2e} R {d_r:.2e}")
    if rank == 0:
        ds = KvsAll(tr, NE, NR, label_smoothing_rate=0.1).to(dev)
        model = make()
        eng = FusedKvsAllEngine(model, ds, batch_size=W * B, lr=lr, device=dev)
        g.manual_seed(5)
        ls = []
        for _ in range(steps):
            idx = torch.randperm(len(ds), generator=g)[: W * B].to(dev)
            ls.append(float(eng.step((ds.train_data[idx], idx))))
        eng.sync_to_model()
        es = model.entity_embeddings.weight.detach()
        d_s = (ep - es).abs().max().item() / es.abs().max().item()
        for a, b in zip(lp, ls):
            ok &= abs(a - b) < 2e-3 * abs(b) + 1e-6
        ok &= d_s < 2e-2
        msg.append(f"p2p vs single: losses {lp} / {ls}; rel diff E {d_s:.2e}")
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("\n".join(msg))
        print("SHARDED_OK" if int(flag) == 1 else "SHARDED_MISMATCH")
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
