"""Regress numeric attributes of entities from frozen embeddings.

    python examples/literal_prediction.py --run Experiments/<run> --train literals/train.txt --test literals/test.txt

The literal files hold one ``entity<TAB>attribute<TAB>value`` row per line.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout
import argparse

from dice_embeddings_b200 import KGE
from dice_embeddings_b200.evaluation.literal_prediction import evaluate_literal_prediction

ap = argparse.ArgumentParser()
ap.add_argument("--run", required=True)
ap.add_argument("--train", required=True)
ap.add_argument("--test", required=True)
a = ap.parse_args()

kge = KGE(path=a.run)
kge.train_literals(train_file_path=a.train, num_epochs=200, lit_lr=0.01, batch_size=512)
print(evaluate_literal_prediction(kge, eval_file_path=a.test, return_attr_error_metrics=True))
