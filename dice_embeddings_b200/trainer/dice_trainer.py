"""Trainer factory: picks the trainer for ``--trainer``, assembles the callbacks, builds the dataset of the
scoring technique and runs training or k-fold cross-validation
(reference ``dicee/trainer/dice_trainer.py:48-412``).

Trainer names map as follows:

========================  ==========================================================================
``torchCPUTrainer``       :class:`TorchTrainer` on CPU (or on ``cuda:<gpus>`` when ``args.gpus`` is set)
``PL``                    one GPU or none: :class:`TorchTrainer` (``cuda:0`` / CPU).  Several GPUs: the command line
                          re-launches itself with one rank per GPU under ``torch.distributed.run`` and the
                          ``torchDDP`` trainer (``cli._relaunch_on_all_gpus``); under ``torchrun`` the name is
                          an alias of ``torchDDP``.  The reference delegates to PyTorch-Lightning, which starts
                          DDP on several GPUs (``:75-92``); Lightning is not a dependency here
``torchDDP``              :class:`TorchDDPTrainer` — one process per device under ``torchrun``
``TP``                    :class:`TensorParallel` — embedding-dimension split over the local devices
``Sharded``               :class:`ShardedTrainer` — row-sharded entity table with fused kernels
anything else / ``None``  :class:`TorchTrainer` (reference ``:93-95``)
========================  ==========================================================================
"""
from __future__ import annotations

import copy
import os
from typing import List, Tuple, Union

import numpy as np
import pandas as pd
import torch

from ..data.datasets import construct_dataset
from ..data.kg import KG
from ..io.checkpoint import select_model
from ..models import EnsembleKGE
from .base import BatchLoader
from .torch_trainer import TorchTrainer


def initialize_trainer(args, callbacks: List):
    name = getattr(args, "trainer", None)
    if name == "TP":
        from .tensor_parallel import TensorParallel
        return TensorParallel(args, callbacks=callbacks)
    if name == "torchDDP" or (name == "PL" and int(os.environ.get("WORLD_SIZE", "1")) > 1):
        from .ddp import TorchDDPTrainer
        return TorchDDPTrainer(args, callbacks=callbacks)
    if name == "Sharded":
        from .sharded import ShardedTrainer
        return ShardedTrainer(args, callbacks=callbacks)
    return TorchTrainer(args, callbacks=callbacks)


def get_callbacks(args) -> List:
    """Callback list from the flags (reference ``dice_trainer.py:100-180``)."""
    from . import callbacks as cb
    from . import weight_averaging as wa
    out = [cb.PrintCallback(), cb.AccumulateEpochLossCallback(path=args.full_storage_path)]
    if getattr(args, "swa", False):
        out.append(wa.SWA(swa_start_epoch=args.swa_start_epoch, lr_init=args.lr, max_epochs=args.num_epochs,
                          swa_c_epochs=args.swa_c_epochs))
    elif getattr(args, "swag", False):
        out.append(wa.SWAG(swa_start_epoch=args.swa_start_epoch, lr_init=args.lr, max_epochs=args.num_epochs,
                           swa_c_epochs=args.swa_c_epochs))
    elif getattr(args, "ema", False):
        out.append(wa.EMA(ema_start_epoch=args.swa_start_epoch, max_epochs=args.num_epochs,
                          ema_c_epochs=args.swa_c_epochs))
    elif getattr(args, "twa", False):
        out.append(wa.TWA(twa_start_epoch=args.swa_start_epoch, lr_init=args.lr, max_epochs=args.num_epochs,
                          twa_c_epochs=args.swa_c_epochs))
    elif getattr(args, "adaptive_swa", False):
        out.append(wa.ASWA(num_epochs=args.num_epochs, path=args.full_storage_path))
    elif getattr(args, "adaptive_lr", None):
        out.append(cb.LRScheduler(adaptive_lr_config=args.adaptive_lr, total_epochs=args.num_epochs,
                                  experiment_dir=args.full_storage_path, eta_max=args.lr))
    if (getattr(args, "eval_every_n_epochs", 0) or 0) > 0 or getattr(args, "eval_at_epochs", None) is not None:
        out.append(cb.PeriodicEvalCallback(experiment_path=args.full_storage_path, max_epochs=args.num_epochs,
                                           eval_every_n_epoch=args.eval_every_n_epochs,
                                           eval_at_epochs=args.eval_at_epochs,
                                           save_model_every_n_epoch=args.save_every_n_epochs,
                                           n_epochs_eval_model=args.n_epochs_eval_model))
    extra = getattr(args, "callbacks", None)
    if isinstance(extra, list) or not extra:
        return out
    for k, v in extra.items():
        if k == "Perturb":
            out.append(cb.Perturb(**v))
        elif k == "KronE":
            out.append(cb.KronE())
        elif k == "Eval":
            out.append(cb.Eval(path=args.full_storage_path, epoch_ratio=v.get("epoch_ratio")))
        elif k == "PPE":
            out.append(cb.PPE(num_epochs=args.num_epochs, path=args.full_storage_path, **v))
        elif k == "KGESave":
            out.append(cb.KGESaveCallback(path=args.full_storage_path, max_epochs=args.num_epochs, **v))
        else:
            raise RuntimeError(f"Incorrect callback:{k}")
    return out


class DICE_Trainer:
    def __init__(self, args, is_continual_training: bool, storage_path, evaluator=None):
        self.report = dict()
        self.args = args
        self.trainer = None
        self.is_continual_training = is_continual_training
        self.storage_path = storage_path
        self.evaluator = evaluator
        self.form_of_labelling = None

    # ------------------------------------------------------------------ pieces
    def initialize_trainer(self, callbacks: List):
        return initialize_trainer(self.args, callbacks)

    def initialize_or_load_model(self):
        tp_devices = getattr(self.trainer, "devices", None) if getattr(self.args, "trainer", None) == "TP" else None
        model, form = select_model(vars(self.args), self.is_continual_training, self.storage_path,
                                   tp_devices=tp_devices)
        self.report["form_of_labelling"] = form
        assert form in ("EntityPrediction", "RelationPrediction")
        return model, form

    def init_dataloader(self, dataset) -> BatchLoader:
        rank = getattr(self.trainer, "global_rank", 0)
        world = getattr(self.trainer, "world_size", 1)
        return BatchLoader(dataset, batch_size=self.args.batch_size, shuffle=True,
                           seed=getattr(self.args, "random_seed", 0) or 0, rank=rank, world_size=world,
                           num_workers=getattr(self.args, "num_core", 0) or 0)

    def init_dataset(self):
        ds = self.trainer.dataset
        a = self.args
        common = dict(form_of_labelling=self.trainer.form_of_labelling, scoring_technique=a.scoring_technique,
                      neg_ratio=a.neg_ratio, label_smoothing_rate=a.label_smoothing_rate,
                      byte_pair_encoding=a.byte_pair_encoding, block_size=a.block_size)
        if isinstance(ds, KG):
            if ds.path_for_serialization and isinstance(ds.train_set, np.ndarray) and ds.train_set.ndim == 2 \
                    and not a.byte_pair_encoding:
                mm = os.path.join(ds.path_for_serialization, "memory_map_train_set.npy")
                if not os.path.exists(mm):
                    m = np.memmap(mm, dtype=ds.train_set.dtype, mode="w+", shape=ds.train_set.shape)
                    m[:] = ds.train_set[:]
                    m.flush()
                    del m
            return construct_dataset(train_set=ds.train_set, valid_set=ds.valid_set, test_set=ds.test_set,
                                     train_target_indices=ds.train_target_indices, target_dim=ds.target_dim,
                                     ordered_bpe_entities=ds.ordered_bpe_entities, entity_to_idx=ds.entity_to_idx,
                                     relation_to_idx=ds.relation_to_idx, **common)
        assert isinstance(ds, np.ndarray), f"Train dataset must be a KG or an index array, not {type(ds)}"
        # ranks other than 0 (and continual training) only have the memory-mapped triples
        return construct_dataset(train_set=np.asarray(ds), valid_set=None, test_set=None, train_target_indices=None,
                                 target_dim=None, ordered_bpe_entities=None,
                                 entity_to_idx=range(int(a.num_entities)), relation_to_idx=range(int(a.num_relations)),
                                 **common)

    # ------------------------------------------------------------------ entry points
    def _prepare(self, knowledge_graph):
        self.trainer = self.initialize_trainer(callbacks=get_callbacks(self.args))
        model, form = self.initialize_or_load_model()
        self.trainer.evaluator = self.evaluator
        self.trainer.dataset = knowledge_graph
        self.trainer.form_of_labelling = form
        return model, form

    def continual_start(self, knowledge_graph):
        model, form = self._prepare(knowledge_graph)
        self.trainer.fit(model, train_dataloaders=self.init_dataloader(self.init_dataset()))
        return model, form

    def start(self, knowledge_graph: Union[KG, np.ndarray]) -> Tuple[object, str]:
        if getattr(self.args, "num_folds_for_cv", 0) == 0:
            model, form = self._prepare(knowledge_graph)
            out = self.trainer.fit(model, train_dataloaders=self.init_dataloader(self.init_dataset()))
            if isinstance(out, EnsembleKGE):
                model = out
            return model, form
        return self.k_fold_cross_validation(knowledge_graph)

    def k_fold_cross_validation(self, dataset) -> Tuple[object, str]:
        """Train one model per fold on ``train_set`` and rank the held-out fold; the per-fold metrics become the
        evaluator's report (reference ``dice_trainer.py:359-412``)."""
        k = self.args.num_folds_for_cv
        n = len(dataset.train_set)
        perm = np.random.RandomState(1).permutation(n)
        folds = np.array_split(perm, k)
        rows = []
        model, form = None, None
        for i in range(k):
            test_idx = folds[i]
            train_idx = np.concatenate([folds[j] for j in range(k) if j != i])
            args = copy.copy(self.args)
            trainer = initialize_trainer(args, get_callbacks(args))
            self.trainer = trainer
            model, form = select_model(vars(args), self.is_continual_training, self.storage_path)
            trainer.evaluator, trainer.dataset, trainer.form_of_labelling = self.evaluator, dataset, form
            ds = construct_dataset(train_set=dataset.train_set[train_idx], entity_to_idx=dataset.entity_to_idx,
                                   relation_to_idx=dataset.relation_to_idx, form_of_labelling=form,
                                   scoring_technique=args.scoring_technique, neg_ratio=args.neg_ratio,
                                   label_smoothing_rate=args.label_smoothing_rate)
            trainer.fit(model, train_dataloaders=self.init_dataloader(ds))
            res = self.evaluator.eval_with_data(dataset=dataset, trained_model=model,
                                                triple_idx=dataset.train_set[test_idx], form_of_labelling=form)
            rows.append([res["MRR"], res["H@1"], res["H@3"], res["H@10"]])
        df = pd.DataFrame(rows, columns=["MRR", "H@1", "H@3", "H@10"])
        self.evaluator.report = df.to_dict()
        print(df)
        print(df.describe())
        return model, form
