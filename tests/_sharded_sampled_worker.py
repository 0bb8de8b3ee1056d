"""Worker for the multi-GPU tests (launched with torch.distributed.run): the row-sharded sampled-candidate step with
the row-wise sparse optimiser against PyTorch autograd on the concatenated batch, plus device-side corruption runs."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dice_embeddings_b200.data.datasets import OnevsSample  # noqa: E402
from dice_embeddings_b200.data.synthetic import zipf_kg  # noqa: E402
from dice_embeddings_b200.models import initialize_model  # noqa: E402
from dice_embeddings_b200.parallel.sharded_sampled import ShardedSampledEngine  # noqa: E402


def make(name, D, NE, NR, optim, lr, dev, scoring):
    torch.manual_seed(0)
    m, _ = initialize_model(dict(model=name, embedding_dim=D, num_entities=NE, num_relations=NR, optim=optim,
                                 learning_rate=lr, scoring_technique=scoring, p=0, q=1))
    return m.to(dev)


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    W = dist.get_world_size()
    NE, NR, D, B, C = 1003, 11, 64, 256, 21
    tr = zipf_kg(NE, NR, 8000, seed=2)
    ok, msg = True, []

    # ---- (1) given candidates, SGD: must equal autograd on the whole batch
    lr = 20.0
    for name in ("ComplEx", "QMult", "TransE"):
        ref = make(name, D, NE, NR, "SGD", lr, dev, "1vsSample")
        mdl = make(name, D, NE, NR, "SGD", lr, dev, "1vsSample")
        ds = OnevsSample(tr, NE, NR, neg_sample_ratio=C - 1, label_smoothing_rate=0.1).to(dev)
        g = torch.Generator(device=dev).manual_seed(4)
        torch.manual_seed(4)
        x, idx, y = (t.contiguous() for t in ds.make_batch(torch.arange(W * B, device=dev)))
        for t in (x, idx, y):   # the dataset draws negatives with the device generator: make all ranks agree
            dist.broadcast(t, src=0)
        opt = torch.optim.SGD(ref.parameters(), lr=lr)
        loss_ref = ref.training_step((x, idx, y))
        loss_ref.backward()
        opt.step()
        eng = ShardedSampledEngine(mdl, "1vsSample", batch_size=B, lr=lr, device=dev, use_graph=False)
        sl = slice(rank * B, (rank + 1) * B)
        loss = float(eng.step((x[sl], idx[sl], y[sl])))
        eng.sync_to_model()
        d_e = (mdl.entity_embeddings.weight - ref.entity_embeddings.weight).abs().max().item()
        d_r = (mdl.relation_embeddings.weight - ref.relation_embeddings.weight).abs().max().item()
        s_e = (ref.entity_embeddings.weight.grad * lr).abs().max().item()
        good = abs(loss - float(loss_ref)) < 1e-4 * abs(float(loss_ref)) and d_e < 1e-3 * s_e + 1e-7 and d_r < 1e-3 * s_e + 1e-6
        ok &= good
        msg.append(f"{name}: loss {loss:.6f} vs {float(loss_ref):.6f}, max diff E {d_e:.2e} R {d_r:.2e} (update scale {s_e:.2e})")
        del eng

    # ---- (2) device-side corruption, Adam with lazy moments, graph replay: the loss must go down, rows move sparsely
    for name, layout in (("ComplEx", "tails"), ("TransE", "flat")):
        mdl = make(name, D, NE, NR, "Adam", 0.05, dev, "NegSample")
        before = mdl.entity_embeddings.weight.detach().clone()
        eng = ShardedSampledEngine(mdl, "NegSample", batch_size=B, lr=0.05, neg_ratio=8, device=dev, layout=layout)
        pos = torch.as_tensor(tr).long().to(dev)
        g = torch.Generator().manual_seed(9)
        losses = []
        for _ in range(30):
            sel = torch.randint(0, pos.shape[0], (W * B,), generator=g)[rank * B:(rank + 1) * B].to(dev)
            losses.append(float(eng.step((pos[sel],))))
        eng.sync_to_model()
        moved = ((mdl.entity_embeddings.weight - before).abs().sum(1) > 0).float().mean().item()
        good = losses[-1] < 0.8 * losses[0] and 0.05 < moved <= 1.0
        ok &= good
        msg.append(f"{name}/{layout}: loss {losses[0]:.4f} -> {losses[-1]:.4f}, {moved:.2%} of the rows were updated")
        del eng

    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("\n".join(msg))
        print("SHARDED_SAMPLED_OK" if int(flag) == 1 else "SHARDED_SAMPLED_MISMATCH")
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
