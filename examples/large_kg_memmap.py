"""Training on a triple file that is indexed once and then memory-mapped: ``--reuse_existing_run_dir`` keeps the run
directory, so a second start skips reading and indexing and maps ``memory_map_train_set.npy`` instead.

    python examples/large_kg_memmap.py --path_single_kg big.tsv --out Experiments/big
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout
import argparse

from dice_embeddings_b200 import Execute, Namespace

ap = argparse.ArgumentParser()
ap.add_argument("--path_single_kg", required=True)
ap.add_argument("--out", required=True)
a = ap.parse_args()
common = dict(path_single_kg=a.path_single_kg, path_to_store_single_run=a.out, model="DistMult", embedding_dim=64,
              scoring_technique="1vsSample", neg_ratio=64, batch_size=8192, eval_model=None, backend="pandas",
              trainer="torchCPUTrainer")
Execute(Namespace(num_epochs=1, **common)).start()                                   # reads, indexes, writes the map
Execute(Namespace(num_epochs=5, reuse_existing_run_dir=True, **common)).start()      # maps the indexed triples
