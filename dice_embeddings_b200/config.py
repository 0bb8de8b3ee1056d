"""Configuration objects.

Two sets of defaults exist, exactly as in the reference: the Python-API defaults
(``Namespace``; reference ``dicee/config.py:9-191``) and the command-line defaults
(``cli.build_parser``; reference ``dicee/scripts/run.py:5-166``).  Both end up in the same
flat attribute bag which is serialised wholesale as ``configuration.json``
(reference ``dicee/executer.py:134-136``), so every key name below is part of the
on-disk contract.
"""
from __future__ import annotations

import argparse
from typing import Any, Dict, Iterator, Tuple

# key -> Python-API default (reference dicee/config.py).
_API_DEFAULTS: Dict[str, Any] = dict(
    dataset_dir=None,
    save_embeddings_as_csv=False,
    storage_path="Experiments",
    path_to_store_single_run=None,
    path_single_kg=None,
    sparql_endpoint=None,
    model="Keci",
    optim="Adam",
    embedding_dim=64,
    num_epochs=150,
    batch_size=1024,
    lr=0.1,
    add_noise_rate=None,
    gpus=None,
    callbacks=None,          # replaced by a fresh dict per instance
    backend="pandas",
    separator=r"\s+",
    trainer="torchCPUTrainer",
    scoring_technique="KvsAll",
    neg_ratio=0,
    weight_decay=0.0,
    normalization="None",
    init_param=None,
    gradient_accumulation_steps=0,
    num_folds_for_cv=0,
    eval_model="train_val_test",
    save_model_at_every_epoch=None,
    label_smoothing_rate=0.0,
    num_core=0,
    random_seed=0,
    sample_triples_ratio=None,
    read_only_few=None,
    pykeen_model_kwargs=None,  # fresh dict per instance
    kernel_size=3,
    num_of_output_channels=32,
    p=0,
    q=1,
    r=0,
    degree=0,
    input_dropout_rate=0.0,
    hidden_dropout_rate=0.0,
    feature_map_dropout_rate=0.0,
    byte_pair_encoding=False,
    adaptive_swa=False,
    swa=False,
    swag=False,
    ema=False,
    twa=False,
    block_size=None,
    continual_learning=None,
    auto_batch_finding=False,
    eval_every_n_epochs=0,
    save_every_n_epochs=False,
    eval_at_epochs=None,
    n_epochs_eval_model="val_test",
    adaptive_lr=None,        # fresh dict per instance
    swa_start_epoch=None,
    swa_c_epochs=1,
    reuse_existing_run_dir=False,
    # --- additions of this framework (absent from the reference) -------------------
    # compute dtype of the fused sm_100a scoring kernels ("bf16") or "fp32" for the generic path
    compute_dtype="fp32",
    # "auto": fused CUDA kernels when a GPU and a supported model are present, else PyTorch ops
    kernel_backend="auto",
    # communication style of the sharded trainer: "p2p" (peer loads/stores inside the kernels)
    # or "nccl" (library collectives; the comparison pipeline)
    comm="p2p",
)

_DICT_KEYS = ("callbacks", "pykeen_model_kwargs", "adaptive_lr")


class Namespace(argparse.Namespace):
    """Attribute bag with the Python-API defaults of the reference.

    ``Namespace(model="ComplEx", embedding_dim=32)`` overrides single fields; iteration
    yields ``(key, value)`` pairs (reference ``dicee/config.py:188-191``).
    """

    def __init__(self, **kwargs: Any):
        super().__init__()
        for k, v in _API_DEFAULTS.items():
            setattr(self, k, {} if k in _DICT_KEYS else v)
        for k, v in kwargs.items():
            setattr(self, k, v)

    def __iter__(self) -> Iterator[Tuple[str, Any]]:
        for k, v in self.__dict__.items():
            yield k, v


def namespace_from_dict(d: Dict[str, Any]) -> Namespace:
    """Rebuild a :class:`Namespace` from a loaded ``configuration.json`` (unknown keys kept)."""
    ns = Namespace()
    for k, v in d.items():
        setattr(ns, k, v)
    return ns


_SCORING_WITH_RECIPROCALS = ("AllvsAll", "1vsSample", "KvsAll", "1vsAll", "KvsSample")
_EVAL_CHOICES = (None, "None", "train", "val", "test", "train_val", "train_test", "val_test", "train_val_test")


def sanity_check_args(args) -> None:
    """Range / combination checks (reference ``dicee/sanity_checkers.py:83-116``)."""
    assert args.embedding_dim > 0, "embedding_dim must be positive"
    assert args.num_epochs >= 0
    assert args.batch_size is None or args.batch_size > 0
    if args.scoring_technique == "NegSample":
        assert args.neg_ratio is not None and args.neg_ratio >= 0
    sources = [getattr(args, "dataset_dir", None), getattr(args, "path_single_kg", None),
               getattr(args, "sparql_endpoint", None)]
    if getattr(args, "continual_learning", None) is None and not getattr(args, "_allow_no_source", False):
        if sum(s is not None for s in sources) == 0:
            raise RuntimeError("One of --dataset_dir, --path_single_kg or --sparql_endpoint must be given.")
    multi_gpu_trainer = args.trainer in ("torchDDP", "TP")
    if multi_gpu_trainer and getattr(args, "adaptive_lr", None):
        raise ValueError("adaptive_lr (LR scheduling with snapshot ensembles) is not available with multi-GPU trainers")
    if multi_gpu_trainer and (getattr(args, "twa", False) or getattr(args, "swag", False)):
        raise ValueError("TWA/SWAG are not available with the TP/torchDDP trainers")


def preprocess_args(args):
    """Derive the secondary fields every later stage expects.

    Mirrors reference ``dicee/static_preprocess_funcs.py:34-72``: ``max_epochs``,
    ``learning_rate``, the reciprocal flag, ``'None'`` strings → ``None``, Shallom→KvsAll,
    BytE→byte-pair encoding.
    """
    for k, v in _API_DEFAULTS.items():  # tolerate SimpleNamespace / argparse inputs missing new keys
        if not hasattr(args, k):
            setattr(args, k, {} if k in _DICT_KEYS else v)
    for k in _DICT_KEYS:
        if getattr(args, k) is None:
            setattr(args, k, {})
    args.max_epochs = args.num_epochs
    args.min_epochs = args.num_epochs
    assert args.weight_decay >= 0.0
    args.learning_rate = args.lr
    args.deterministic = True
    assert args.init_param in ("xavier_normal", None, "None")
    if args.init_param == "None":
        args.init_param = None
    args.check_val_every_n_epoch = 10 ** 6
    assert args.add_noise_rate is None or isinstance(args.add_noise_rate, float)
    args.logger = False
    assert args.eval_model in _EVAL_CHOICES, f"Unexpected input for eval_model ***\t{args.eval_model}\t***"
    if args.eval_model == "None":
        args.eval_model = None
    if args.scoring_technique in _SCORING_WITH_RECIPROCALS:
        args.apply_reciprical_or_noise = True
    elif args.scoring_technique in ("NegSample", "Sentence"):
        args.apply_reciprical_or_noise = False
    else:
        raise KeyError(f"Unexpected input for scoring_technique \t{args.scoring_technique}")
    if args.sample_triples_ratio is not None:
        assert 1.0 >= args.sample_triples_ratio >= 0.0
    assert args.backend in ("pandas", "polars", "rdflib")
    sanity_check_args(args)
    if args.model == "Shallom":
        args.scoring_technique = "KvsAll"
    if args.normalization == "None":
        args.normalization = None
    assert args.normalization in (None, "LayerNorm", "BatchNorm1d")
    if args.model == "BytE" and getattr(args, "block_size", None) is None:
        args.block_size = 8   # default of the command line (reference ``scripts/run.py:118``); the Python API leaves None
    if args.model == "BytE":
        args.byte_pair_encoding = True
    return args
