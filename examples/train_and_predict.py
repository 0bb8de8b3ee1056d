"""Train a model on a folder with train.txt / valid.txt / test.txt, reload it and ask for completions.

    python examples/train_and_predict.py --dataset_dir KGs/UMLS --model Keci
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout
import argparse

from dice_embeddings_b200 import Execute, KGE, Namespace

ap = argparse.ArgumentParser()
ap.add_argument("--dataset_dir", required=True)
ap.add_argument("--model", default="Keci")
ap.add_argument("--gpu", type=int, default=None, help="CUDA device index; omit for CPU")
a = ap.parse_args()

args = Namespace(dataset_dir=a.dataset_dir, model=a.model, scoring_technique="KvsAll", embedding_dim=64, num_epochs=100,
                 batch_size=1024, lr=0.1, eval_model="train_val_test", gpus=a.gpu, trainer="torchCPUTrainer")
report = Execute(args).start()
print({k: report[k] for k in ("Train", "Val", "Test") if k in report})

kge = KGE(path=report["path_experiment_folder"])
h, r = next(iter(kge.entity_to_idx)), next(iter(kge.relation_to_idx))
print(f"top-5 tails for ({h}, {r}, ?):", kge.predict_topk(h=[h], r=[r], topk=5)[0])
print("score of one triple:", float(kge.triple_score(h=[h], r=[r], t=[h])))
