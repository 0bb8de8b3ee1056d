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


def is_sparql_endpoint_alive(sparql_endpoint: str = None) -> bool:
    """One tiny COUNT query; ``False`` without an endpoint, an ``AssertionError`` when the endpoint does not answer
    (reference ``dicee/sanity_checkers.py:7-15``)."""
    if not sparql_endpoint:
        return False
    import requests
    query = "SELECT (COUNT(*) as ?num_triples) WHERE {  ?s ?p ?o .} "
    response = requests.post(sparql_endpoint, data={"query": query})
    assert response.ok, f"SPARQL endpoint {sparql_endpoint} answered {getattr(response, 'status_code', '?')}"
    return True


def validate_knowledge_graph(args) -> None:
    """Exactly one source of triples is kept, in the reference's order of precedence: a live SPARQL endpoint, then a
    single file, then a dataset folder, which must exist and contain a ``train*`` file
    (reference ``dicee/sanity_checkers.py:18-80``)."""
    import glob
    import os
    endpoint = getattr(args, "sparql_endpoint", None)
    single = getattr(args, "path_single_kg", None)
    folder = getattr(args, "dataset_dir", None)
    if is_sparql_endpoint_alive(endpoint):
        args.dataset_dir = None
        args.path_single_kg = None
    elif single is not None:
        if not os.path.isfile(single):
            raise ValueError(f"--path_single_kg **{single}** does not lead to a file")
        args.dataset_dir = None
        args.sparql_endpoint = None
    elif folder:
        if not isinstance(folder, str):
            raise AssertionError(f"The dataset_dir must be a string. ***{folder}***")
        if not (os.path.isdir(folder) or os.path.isfile(folder)):
            raise AssertionError(f"The dataset_dir does not lead to a directory ***{folder}***")
        if not glob.glob(folder + "/train*"):
            raise ValueError(f"---dataset_dir **{folder}** must lead to a **folder** containing at least train.txt**. "
                             f"Use --path_single_kg **folder/dataset.format**, if you have a single file.")
        args.sparql_endpoint = None
        args.path_single_kg = None
    else:
        raise RuntimeError("One of the following arguments must be given: "
                           f"--dataset_dir:{folder},\t--path_single_kg:{single},\t--sparql_endpoint:{endpoint}.")


def sanity_check_callback_args(args) -> None:
    """Trainer / callback combinations (reference ``dicee/sanity_checkers.py:92-116``): training on several GPUs needs
    an explicit run folder (every rank must agree on it) and excludes the LR-schedule / TWA / SWAG callbacks."""
    import os
    gpu_count = 0
    try:
        import torch
        gpu_count = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:   # noqa: BLE001 - the checks must not depend on a working CUDA runtime
        pass
    launched = int(os.environ.get("WORLD_SIZE", "1")) > 1
    multi = args.trainer in ("torchDDP", "Sharded") or (args.trainer == "PL" and gpu_count >= 2 and launched)
    if multi and launched and getattr(args, "path_to_store_single_run", None) is None:
        raise NotImplementedError("Path to store experiments must be provided for Multi-GPU training "
                                  "(--path_to_store_single_run).")
    if any([getattr(args, "swa", False), getattr(args, "swag", False), getattr(args, "ema", False),
            getattr(args, "twa", False)]):
        args.swa_start_epoch = getattr(args, "swa_start_epoch", None) or 1
        assert args.swa_start_epoch > 0, "SWA Start Epoch must be greater than 0"


def dataset_sanity_checking(train_set, num_entities: int, num_relations: int) -> None:
    """Indexed triples must be a non-empty ``[n, 3]`` integer array whose ids fit the vocabularies
    (reference ``dicee/read_preprocess_save_load_kg/util.py:515-545``)."""
    import numpy as np
    assert isinstance(train_set, np.ndarray), "the training set must be a numpy array"
    assert train_set.ndim == 2 and train_set.shape[1] == 3, f"expected [n, 3] triples, got {train_set.shape}"
    if train_set.shape[0] == 0:
        raise AssertionError("Size of the training dataset must be greater than 0.")
    max_e = int(max(train_set[:, 0].max(), train_set[:, 2].max()))
    if max_e >= num_entities:
        raise AssertionError(f"Entity Indexing Error:\nMax ID of a subject or object entity in train set: {max_e} "
                             f"is not below num_entities: {num_entities}")
    max_r = int(train_set[:, 1].max())
    if max_r >= num_relations:
        raise AssertionError(f"Relation Indexing Error:\nMax ID of a relation in train set: {max_r} "
                             f"is not below num_relations: {num_relations}")
    assert np.issubdtype(train_set.dtype, np.integer), "triples must be stored as integers"


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
    if getattr(args, "continual_learning", None) is None and not getattr(args, "_allow_no_source", False):
        validate_knowledge_graph(args)
    sanity_check_callback_args(args)


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
