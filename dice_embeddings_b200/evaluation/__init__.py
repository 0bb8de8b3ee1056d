from .evaluator import Evaluator
from .ranking import (ALL_HITS_RANGE, filtered_rank_from_scores, head_and_tail_ranks, metrics_from_ranks,
                      relation_ranks, tail_ranks)
from .link_prediction import (evaluate_bpe_lp, evaluate_link_prediction_performance,
                              evaluate_link_prediction_performance_with_bpe,
                              evaluate_link_prediction_performance_with_bpe_reciprocals,
                              evaluate_link_prediction_performance_with_reciprocals, evaluate_lp,
                              evaluate_lp_bpe_k_vs_all)
from .ensemble import evaluate_ensemble_link_prediction_performance
from .literal_prediction import evaluate_literal_prediction

__all__ = ["Evaluator", "evaluate_lp", "evaluate_link_prediction_performance",
           "evaluate_link_prediction_performance_with_reciprocals", "evaluate_link_prediction_performance_with_bpe",
           "evaluate_link_prediction_performance_with_bpe_reciprocals", "evaluate_bpe_lp", "evaluate_lp_bpe_k_vs_all",
           "evaluate_ensemble_link_prediction_performance", "evaluate_literal_prediction", "metrics_from_ranks",
           "tail_ranks", "relation_ranks", "head_and_tail_ranks", "filtered_rank_from_scores", "ALL_HITS_RANGE"]
