"""Worker for the multi-GPU tests (launched with torch.distributed.run): (1) a sharded engine saves a checkpoint,
trains on, reloads it and must be back at the saved state; (2) filtered ranks and top-k computed over the
row-sharded table equal those computed against the whole table on one GPU."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dice_embeddings_b200.data.datasets import KvsAll  # noqa: E402
from dice_embeddings_b200.data.synthetic import zipf_kg  # noqa: E402
from dice_embeddings_b200.data.vocab import er_csr  # noqa: E402
from dice_embeddings_b200.evaluation.ranking import filter_csr  # noqa: E402
from dice_embeddings_b200.models import initialize_model  # noqa: E402
from dice_embeddings_b200.ops.eval_rank import FusedRanker, model_queries  # noqa: E402
from dice_embeddings_b200.parallel.sharded_engine import ShardedKvsAllEngine, take_shard  # noqa: E402


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    W = dist.get_world_size()
    NE, NR, D, B = 2003, 11, 128, 256
    tr = zipf_kg(NE, NR, 9000, seed=1)
    torch.manual_seed(0)
    model, _ = initialize_model(dict(model="ComplEx", embedding_dim=D, num_entities=NE, num_relations=NR, optim="Adam",
                                     learning_rate=0.05, scoring_technique="KvsAll"))
    model.to(dev)
    ds = KvsAll(tr, NE, NR, label_smoothing_rate=0.1).to(dev)
    eng = ShardedKvsAllEngine(model, ds, batch_size=B, lr=0.05, device=dev, comm="p2p")
    g = torch.Generator().manual_seed(3)

    def step():
        idx_all = torch.randperm(len(ds), generator=g)[: W * B]
        idx = idx_all[rank * B:(rank + 1) * B].to(dev)
        return float(eng.step((ds.train_data[idx], idx)))

    ok = True
    msg = []
    for _ in range(3):
        step()
    # every rank must use the same directory: rank 0 picks it
    box = [tempfile.mkdtemp(prefix="dice_ck_") if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    ck = box[0]
    eng.save_checkpoint(ck)
    saved = {k: v.clone() for k, v in (("E", eng.E), ("mE", eng.mE), ("vE", eng.vE), ("R", eng.R))}
    saved_step = int(eng.step_count.item())
    rng_state = g.get_state()
    after = [step() for _ in range(2)]
    eng.load_checkpoint(ck)
    for k, v in (("E", eng.E), ("mE", eng.mE), ("vE", eng.vE), ("R", eng.R)):
        ok &= bool(torch.equal(v, saved[k]))
    ok &= int(eng.step_count.item()) == saved_step
    g.set_state(rng_state)
    again = [step() for _ in range(2)]
    ok &= all(abs(a - b) < 1e-3 * abs(a) + 1e-7 for a, b in zip(after, again))
    msg.append(f"resume: losses after save {after}, after reload {again}")

    # ---- sharded ranking / top-k against the whole table
    eng.sync_to_model()
    csr = er_csr(tr, NR)
    test = torch.as_tensor(tr[:1500]).long().to(dev)
    q, _ = model_queries(model, test[:, :2])
    ptr, cols = filter_csr(csr, test[:, 0], test[:, 1])
    full = FusedRanker(model.entity_embeddings.weight)
    shard = FusedRanker(take_shard(model.entity_embeddings.weight.data, rank, W).contiguous(), y_offset=rank,
                        y_stride=W, group=dist.group.WORLD)
    r_full = full.ranks(q, test[:, 2], ptr, cols)
    for rep in range(3):       # back to back: the merge buffers are reused while a slower rank may still read them
        r_shard = shard.ranks(q, test[:, 2], ptr, cols)
        same = float((r_full == r_shard).float().mean())
        ok &= same > 0.995 and int((r_full - r_shard).abs().max()) <= 2
    s_full, i_full = full.topk(q[:300], 10)
    for rep in range(3):
        s_shard, i_shard = shard.topk(q[:300], 10)
        ok &= bool(torch.allclose(s_full, s_shard, atol=1e-3, rtol=1e-3))
        ok &= float((i_full == i_shard).float().mean()) > 0.98
    full.check()
    shard.check()
    msg.append(f"ranks equal on {same:.4f} of the queries; top-k index agreement "
               f"{float((i_full == i_shard).float().mean()):.4f}")
    # exact mode over shards: the ranks of an fp32 evaluation of the whole table
    full_x = FusedRanker(model.entity_embeddings.weight, exact=True)
    shard_x = FusedRanker(take_shard(model.entity_embeddings.weight.data, rank, W).contiguous(), y_offset=rank,
                          y_stride=W, group=dist.group.WORLD, exact=True)
    rx_full, rx_shard = full_x.ranks(q, test[:, 2], ptr, cols), shard_x.ranks(q, test[:, 2], ptr, cols)
    full_x.check()
    shard_x.check()
    s32 = q.float() @ model.entity_embeddings.weight.data.float().t()
    tgt = s32.gather(1, test[:, 2:3])
    keep = torch.ones_like(s32, dtype=torch.bool)
    for i in range(test.shape[0]):
        keep[i, cols[ptr[i]:ptr[i + 1]].long()] = False
    keep.scatter_(1, test[:, 2:3], False)
    oracle = 1 + ((s32 > tgt) & keep).sum(1)
    ok &= bool(torch.equal(rx_shard, rx_full)) and float((rx_shard == oracle).float().mean()) > 0.999
    msg.append(f"exact sharded ranks equal the single-table ones: {bool(torch.equal(rx_shard, rx_full))}; "
               f"agreement with the fp32 oracle {float((rx_shard == oracle).float().mean()):.4f}")

    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("\n".join(msg))
        print("SHARDED_EVAL_OK" if int(flag) == 1 else "SHARDED_EVAL_MISMATCH")
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
