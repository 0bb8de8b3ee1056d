"""Training on a knowledge graph that does not fit in memory.

1. ``index_triple_file`` streams the text file once through the native indexer: only the vocabularies are held in
   memory, the id triples go to ``memory_map_train_set.npy`` in the run folder (raw int32, memory-mapped afterwards).
2. Batches of positive triples are drawn straight from the memory map; the negatives are drawn on the device.
3. The model trains with the sampled-candidate step (fused kernels on a B200, plain PyTorch elsewhere) and is stored in
   the usual run-folder layout, so ``KGE(path=...)`` loads it.

    python examples/train_kge_on_kg_larger_than_memory.py --path_dataset dbpedia.nt --out Experiments/dbpedia \
        --embedding_dim 32 --batch_size 50000 --neg_ratio 100 --num_steps 1000

(The reference's example of the same name does step 1 with polars joins over batches and CSV chunks, and step 2 with a
multinomial draw per item on the host.)
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout

import torch

from dice_embeddings_b200.data import ingest
from dice_embeddings_b200.models import initialize_model


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--path_dataset", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--model", default="Keci")
    ap.add_argument("--embedding_dim", type=int, default=32)
    ap.add_argument("--batch_size", type=int, default=50_000)
    ap.add_argument("--neg_ratio", type=int, default=100)
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--num_steps", type=int, default=100)
    ap.add_argument("--read_only_few", type=int, default=None)
    a = ap.parse_args()

    t0 = time.time()
    if not os.path.isfile(os.path.join(a.out, "memory_map_details.json")):
        d = ingest.index_triple_file(a.path_dataset, a.out, max_rows=a.read_only_few)
        print(f"indexed {d['shape'][0]} triples, {d['num_entities']} entities, {d['num_relations']} relations "
              f"with the {d['indexer']} indexer in {time.time() - t0:.1f} s")
    d = json.load(open(os.path.join(a.out, "memory_map_details.json")))
    triples = ingest.open_triples(a.out)
    dev = torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
    args = dict(model=a.model, embedding_dim=a.embedding_dim, num_entities=d["num_entities"],
                num_relations=d["num_relations"], optim="SGD", learning_rate=a.lr, scoring_technique="NegSample",
                neg_ratio=a.neg_ratio, p=0, q=1)
    with torch.device(dev):
        model, _ = initialize_model(args)
    print(f"parameters: {sum(p.numel() for p in model.parameters()):,}")
    engine = None
    if dev.type == "cuda":
        from dice_embeddings_b200.ops.sampled_step import SampledEngine, sampled_model_code
        if sampled_model_code(model) is not None and torch.cuda.get_device_capability(dev)[0] == 10:
            engine = SampledEngine(model, "NegSample", lr=a.lr, device=dev, neg_ratio=a.neg_ratio)
    opt = None if engine is not None else model.configure_optimizers()
    batches = ingest.MemmapTriples(triples, a.batch_size)
    step = 0
    while step < a.num_steps:
        for pos in batches:
            t1 = time.time()
            pos = pos.to(dev, non_blocking=True)
            if engine is not None:
                loss = float(engine.step((pos,)))
            else:
                n = pos.shape[0]
                corrupt = pos.repeat(a.neg_ratio, 1)
                corrupt[:, 2] = torch.randint(0, d["num_entities"], (corrupt.shape[0],), device=dev)
                x = torch.cat([pos, corrupt])
                y = torch.cat([torch.ones(n, device=dev), torch.zeros(corrupt.shape[0], device=dev)])
                opt.zero_grad(set_to_none=True)
                loss_t = model.training_step((x, y))
                loss_t.backward()
                opt.step()
                loss = float(loss_t)
            print(f"step {step} | loss {loss:.5f} | {time.time() - t1:.3f} s")
            step += 1
            if step >= a.num_steps:
                break
    if engine is not None:
        engine.sync_to_model()
    torch.save(model.state_dict(), os.path.join(a.out, "model.pt"))
    json.dump(dict(args, full_storage_path=a.out), open(os.path.join(a.out, "configuration.json"), "w"), indent=3)
    json.dump({"num_train_triples": d["shape"][0], "num_entities": d["num_entities"],
               "num_relations": d["num_relations"]}, open(os.path.join(a.out, "report.json"), "w"), indent=3)


if __name__ == "__main__":
    main()
