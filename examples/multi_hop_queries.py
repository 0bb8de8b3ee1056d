"""Sample multi-hop queries from a KG, answer them with a trained model and report filtered MRR / Hits per query type.

    python examples/multi_hop_queries.py --dataset_dir KGs/UMLS --run Experiments/<run>
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout
import argparse

from dice_embeddings_b200 import KGE, QueryGenerator, evaluate

ap = argparse.ArgumentParser()
ap.add_argument("--dataset_dir", required=True)
ap.add_argument("--run", required=True, help="directory of a trained run")
ap.add_argument("--per_type", type=int, default=50)
a = ap.parse_args()

kge = KGE(path=a.run)
rel2id = {r: i for i, r in enumerate(sorted(r for r in kge.relation_to_idx if not r.endswith("_inverse")))}
qg = QueryGenerator(f"{a.dataset_dir}/train.txt", f"{a.dataset_dir}/valid.txt", f"{a.dataset_dir}/test.txt",
                    ent2id=dict(kge.entity_to_idx), rel2id=rel2id, seed=1)
for qtype in ("1p", "2p", "3p", "2i", "3i", "ip", "pi", "2in", "3in", "inp", "pin", "pni", "2u", "up"):
    queries, easy, _, hard = qg.get_queries(qtype, a.per_type)
    scores = {q: kge.answer_multi_hop_query(query_type=qtype, query=q, tnorm="prod", only_scores=True) for q in queries}
    mrr, h1, h3, h10 = evaluate(kge.entity_to_idx, scores, easy, hard)
    print(f"{qtype:4s} n={len(queries):3d}  MRR {mrr:.3f}  H@1 {h1:.3f}  H@3 {h3:.3f}  H@10 {h10:.3f}")
