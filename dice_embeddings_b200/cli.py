"""Command line front-end with the flag set of the reference ``dicee`` script.

Every flag, choice list and CLI default follows reference ``dicee/scripts/run.py:5-166``;
three flags are additions of this framework (``--compute_dtype``, ``--kernel_backend``,
``--comm``).  ``main`` dispatches to :class:`Execute` or :class:`ContinuousExecute`
(reference ``dicee/scripts/run.py:168-174``).
"""
from __future__ import annotations

import argparse
from typing import Optional
import json

MODEL_CHOICES = [
    "ComplEx", "Keci", "CKeci", "ConEx", "AConEx", "ConvQ", "AConvQ", "ConvO", "AConvO", "QMult",
    "OMult", "Shallom", "DistMult", "TransE", "DualE", "BytE", "CoKE", "Pyke",
    "Pykeen_MuRE", "Pykeen_QuatE", "Pykeen_DistMult", "Pykeen_BoxE", "Pykeen_CP",
    "Pykeen_HolE", "Pykeen_ProjE", "Pykeen_RotatE", "Pykeen_TransE", "Pykeen_TransF", "Pykeen_TransH",
    "Pykeen_TransR", "Pykeen_TuckER", "Pykeen_ComplEx", "LFMult", "DeCaL",
]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(add_help=True, description="B200-native knowledge graph embedding framework")
    a = p.add_argument
    # knowledge graph
    a("--dataset_dir", type=str, default=None, help="Folder with train.txt and optionally valid.txt / test.txt")
    a("--sparql_endpoint", type=str, default=None, help="Endpoint of a triple store")
    a("--path_single_kg", type=str, default=None, help="Path of a single file holding the whole KG")
    # storage
    a("--path_to_store_single_run", type=str, default=None, help="Exact directory of this run")
    a("--storage_path", type=str, default="Experiments", help="Parent directory of time-stamped run folders")
    a("--save_embeddings_as_csv", action="store_true")
    a("--backend", type=str, default="pandas", choices=["pandas", "polars", "rdflib"])
    a("--separator", type=str, default=r"\s+")
    a("--reuse_existing_run_dir", action="store_true")
    # model
    a("--model", type=str, default="Keci", choices=MODEL_CHOICES)
    a("--optim", type=str, default="Adopt", choices=["Adam", "AdamW", "SGD", "NAdam", "Adagrad", "ASGD", "Adopt"])
    a("--embedding_dim", type=int, default=32)
    a("--num_epochs", type=int, default=10)
    a("--batch_size", type=int, default=32)
    a("--lr", type=float, default=0.1)
    a("--callbacks", type=json.loads, default={})
    a("--trainer", type=str, default="PL", choices=["torchCPUTrainer", "PL", "torchDDP", "TP", "Sharded"])
    a("--scoring_technique", default="NegSample",
      choices=["AllvsAll", "KvsAll", "1vsAll", "NegSample", "1vsSample", "KvsSample"])
    a("--neg_ratio", type=int, default=2)
    a("--weight_decay", type=float, default=0.0)
    a("--input_dropout_rate", type=float, default=0.0)
    a("--hidden_dropout_rate", type=float, default=0.0)
    a("--feature_map_dropout_rate", type=float, default=0.0)
    a("--normalization", type=str, default="None", choices=["LayerNorm", "BatchNorm1d", "None", None])
    a("--init_param", type=str, default=None, choices=["xavier_normal", None])
    a("--gradient_accumulation_steps", type=int, default=0)
    a("--label_smoothing_rate", type=float, default=0.0)
    a("--kernel_size", type=int, default=3)
    a("--num_of_output_channels", type=int, default=2)
    a("--num_core", type=int, default=0)
    a("--random_seed", type=int, default=1)
    a("--p", type=int, default=0)
    a("--q", type=int, default=1)
    a("--r", type=int, default=0)
    a("--pykeen_model_kwargs", type=json.loads, default={})
    # evaluation
    a("--num_folds_for_cv", type=int, default=0)
    a("--eval_model", type=str, default="train_val_test",
      choices=["None", "train", "train_val", "train_val_test", "test"])
    a("--save_model_at_every_epoch", type=int, default=None)
    # continual learning and sub-sampling
    a("--continual_learning", type=str, default=None)
    a("--sample_triples_ratio", type=float, default=None)
    a("--read_only_few", type=int, default=None)
    a("--add_noise_rate", type=float, default=0.0)
    a("--block_size", type=int, default=8)
    a("--byte_pair_encoding", action="store_true")
    a("--adaptive_swa", action="store_true")
    a("--swa", action="store_true")
    a("--swag", action="store_true")
    a("--ema", action="store_true")
    a("--twa", action="store_true")
    a("--auto_batch_finding", action="store_true")
    a("--degree", type=int, default=0)
    a("--adaptive_lr", type=json.loads, default={})
    a("--swa_start_epoch", type=int, default=None)
    a("--swa_c_epochs", type=int, default=1)
    a("--eval_every_n_epochs", type=int, default=0)
    a("--save_every_n_epochs", action="store_true")
    a("--eval_at_epochs", type=int, nargs="+", default=None)
    a("--n_epochs_eval_model", type=str, default="val_test",
      choices=["None", "train", "train_val", "train_val_test", "val_test", "val", "train_test", "test"])
    # additions of this framework
    a("--compute_dtype", type=str, default="fp32", choices=["fp32", "bf16"])
    a("--kernel_backend", type=str, default="auto", choices=["auto", "cuda", "torch"])
    a("--comm", type=str, default="p2p", choices=["p2p", "nccl"])
    a("--gpus", type=int, default=None, help="Index of the single CUDA device used by torchCPUTrainer")
    return p


def get_default_arguments(description=None):
    """Parse ``description`` (a list of strings) or ``sys.argv`` into a namespace."""
    parser = build_parser()
    if description is None:
        return parser.parse_args()
    return parser.parse_args(description)


def _relaunch_on_all_gpus(args, argv) -> Optional[int]:
    """``--trainer PL`` is the reference's command-line default and means "all visible GPUs, data parallel" there
    (Lightning starts one process per device; ``dicee/trainer/dice_trainer.py:75-92``).  The counterpart here: when
    several GPUs are visible and the process was not started by ``torchrun``, the command re-launches itself under
    ``torch.distributed.run`` with one rank per GPU and the data-parallel trainer (``torchDDP``, which picks the
    row-sharded engine when the model is covered).  ``DICE_B200_SINGLE_PROCESS=1`` keeps the single-device run."""
    import os
    import subprocess
    import sys
    if args.trainer != "PL" or "RANK" in os.environ or os.environ.get("DICE_B200_SINGLE_PROCESS") == "1":
        return None
    try:
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:   # noqa: BLE001
        n = 0
    if n < 2:
        return None
    if args.path_to_store_single_run is None:   # every rank has to agree on the run folder
        import datetime
        args_dir = os.path.join(args.storage_path, datetime.datetime.now().strftime("%Y-%m-%d %H-%M-%S.%f"))
        extra = ["--path_to_store_single_run", args_dir]
    else:
        extra = []
    raw = list(sys.argv[1:] if argv is None else argv)
    out, skip = [], False
    for tok in raw:                              # replace the trainer flag
        if skip:
            skip = False
            continue
        if tok == "--trainer":
            skip = True
            continue
        if tok.startswith("--trainer="):
            continue
        out.append(tok)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
           f"--nproc-per-node={n}", "-m", "dice_embeddings_b200", *out, "--trainer", "torchDDP", *extra]
    print(f"--trainer PL with {n} visible GPUs: starting one rank per GPU\n  " + " ".join(cmd))
    return subprocess.call(cmd)


def main(argv=None):
    from .executor import ContinuousExecute, Execute
    args = get_default_arguments(argv)
    rc = _relaunch_on_all_gpus(args, argv)
    if rc is not None:
        if rc != 0:
            raise SystemExit(rc)
        return None
    if args.continual_learning:
        return ContinuousExecute(args).continual_start()
    return Execute(args).start()


if __name__ == "__main__":
    main()
