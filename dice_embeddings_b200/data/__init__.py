from .kg import KG
from .datasets import construct_dataset
from .vocab import PairCSR, get_er_vocab, get_re_vocab, get_ee_vocab

__all__ = ["KG", "construct_dataset", "PairCSR", "get_er_vocab", "get_re_vocab", "get_ee_vocab"]
