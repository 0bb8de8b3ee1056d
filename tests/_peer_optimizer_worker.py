"""Worker (launched with torch.distributed.run): a replicated model trained with the peer all-reduce optimiser on
per-rank batch slices equals single-process autograd + torch.optim on the whole batch."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dice_embeddings_b200.models import initialize_model  # noqa: E402
from dice_embeddings_b200.parallel.peer_allreduce_optimizer import PeerAllReduceOptimizer  # noqa: E402


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    W = dist.get_world_size()
    ok, msg = True, []
    # small buckets: several bucket launches per step, queued from the autograd hooks while backward still runs;
    # ConEx has more than a dozen parameter tensors; the last case runs without the overlap (everything at step())
    for name, optim, lr, bucket, overlap in (("DistMult", "Adam", 0.01, 4 << 20, True), ("DualE", "SGD", 0.5, 2048, True),
                                             ("Shallom", "Adopt", 0.01, 4096, True), ("ConEx", "AdamW", 0.01, 8192, True),
                                             ("ConEx", "Adam", 0.01, 1 << 20, False)):
        torch.manual_seed(0)
        args = dict(model=name, embedding_dim=32, num_entities=300, num_relations=7, optim=optim, learning_rate=lr,
                    scoring_technique="NegSample" if name != "Shallom" else "KvsAll", num_of_output_channels=2,
                    kernel_size=3)
        ref, _ = initialize_model(dict(args))
        mdl, _ = initialize_model(dict(args))
        mdl.load_state_dict(ref.state_dict())
        ref, mdl = ref.to(dev), mdl.to(dev)
        g = torch.Generator().manual_seed(1)
        B = 64 * W
        opt_ref = ref.configure_optimizers()
        popt = PeerAllReduceOptimizer(mdl, lr=lr, device=dev, bucket_bytes=bucket, overlap=overlap)
        if name == "ConEx":   # batch statistics differ between a whole batch and its slices: compare without them
            for mod in list(ref.modules()) + list(mdl.modules()):
                if isinstance(mod, torch.nn.modules.batchnorm._BatchNorm):
                    mod.eval()
        for _ in range(4):
            if name == "Shallom":
                x = torch.stack((torch.randint(0, 300, (B,), generator=g), torch.randint(0, 300, (B,), generator=g)), 1).to(dev)
                y = (torch.rand(B, 7, generator=g) < 0.3).float().to(dev)
            else:
                x = torch.stack((torch.randint(0, 300, (B,), generator=g), torch.randint(0, 7, (B,), generator=g),
                                 torch.randint(0, 300, (B,), generator=g)), 1).to(dev)
                y = (torch.rand(B, generator=g) < 0.5).float().to(dev)
            opt_ref.zero_grad()
            ref.training_step((x, y)).backward()
            opt_ref.step()
            sl = slice(rank * 64, (rank + 1) * 64)
            popt.zero_grad()
            mdl.training_step((x[sl], y[sl])).backward()
            popt.step()
        popt.check()
        worst = 0.0
        for (n, a), (_, b) in zip(ref.named_parameters(), mdl.named_parameters()):
            worst = max(worst, float((a - b).abs().max() / a.abs().max().clamp_min(1e-9)))
        good = worst < 2e-4
        ok &= good
        msg.append(f"{name}/{optim}: {len(popt.buckets)} buckets, overlap {overlap}, multimem {popt.multimem}: "
                   f"max relative parameter difference {worst:.2e}")
        del popt
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("\n".join(msg))
        print("PEER_OPT_OK" if int(flag) == 1 else "PEER_OPT_MISMATCH")
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
