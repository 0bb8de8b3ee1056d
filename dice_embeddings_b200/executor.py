"""Experiment orchestration: ``Execute(args).start()`` and ``ContinuousExecute(args).continual_start()``.

Life-cycle and artefacts follow the reference (``dicee/executer.py:39-440``): create the run directory and
``configuration.json`` (rank 0), read / index the KG and write the memory-mapped train triples, barrier, other
ranks map the triples, train, then rank 0 stores ``model.pt``, ``report.json`` and runs the evaluation.  The
process group is created for the ``torchDDP`` and ``Sharded`` trainers; its backend is NCCL on GPUs and Gloo
otherwise, so the multi-process code paths also run on CPU-only machines.
"""
from __future__ import annotations

import datetime
import json
import os
import random
import shutil
import time
from types import SimpleNamespace
from typing import Dict, Optional

import numpy as np
import torch
import torch.distributed as dist

from .config import preprocess_args
from .data.kg import KG
from .evaluation.evaluator import Evaluator
from .io.checkpoint import create_experiment_folder, load_json, store, write_json
from .trainer.dice_trainer import DICE_Trainer

_DISTRIBUTED_TRAINERS = ("torchDDP", "Sharded")


def seed_everything(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def read_or_load_kg(args, cls=KG):
    """Build the KG from its source and serialise it into the run directory
    (reference ``dicee/static_funcs.py:459-480``)."""
    return cls(dataset_dir=args.dataset_dir, byte_pair_encoding=args.byte_pair_encoding,
               padding=bool(args.byte_pair_encoding and args.model != "BytE"),
               add_noise_rate=args.add_noise_rate, sparql_endpoint=args.sparql_endpoint,
               path_single_kg=args.path_single_kg, add_reciprocal=args.apply_reciprical_or_noise,
               eval_model=args.eval_model, read_only_few=args.read_only_few,
               sample_triples_ratio=args.sample_triples_ratio, path_for_serialization=args.full_storage_path,
               backend=args.backend, training_technique=args.scoring_technique, separator=args.separator)


class Execute:
    def __init__(self, args, continuous_training: bool = False):
        trainer = getattr(args, "trainer", None)
        launched = "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1
        # "PL" started under torchrun with several ranks is data parallel, as with the reference's Lightning trainer
        self.distributed = (trainer in _DISTRIBUTED_TRAINERS and ("RANK" in os.environ or dist.is_initialized())) \
            or (trainer == "PL" and launched)
        self._setup_distributed_training()
        self.args = preprocess_args(args)
        seed_everything(args.random_seed)
        self.is_continual_training = continuous_training
        if self.rank == 0:
            self.setup_executor()
        self.trainer: Optional[DICE_Trainer] = None
        self.trained_model = None
        self.knowledge_graph: Optional[KG] = None
        self.report: Dict = {}
        self.evaluator: Optional[Evaluator] = None
        self.start_time: Optional[float] = None

    # ------------------------------------------------------------------ distributed plumbing
    def _setup_distributed_training(self) -> None:
        if self.distributed:
            if not dist.is_initialized():
                backend = "nccl" if torch.cuda.is_available() else "gloo"
                dist.init_process_group(backend=backend, init_method="env://")
            self.rank = dist.get_rank()
            self.world_size = dist.get_world_size()
            self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
            if torch.cuda.is_available():
                torch.cuda.set_device(self.local_rank)
        else:
            self.rank, self.world_size, self.local_rank = 0, 1, 0

    def is_rank_zero(self) -> bool:
        return self.rank == 0

    def cleanup(self):
        if self.distributed and dist.is_initialized():
            dist.destroy_process_group()

    # ------------------------------------------------------------------ run directory
    def setup_executor(self) -> None:
        if self.is_continual_training:
            return
        a = self.args
        if a.path_to_store_single_run is not None:
            path = a.path_to_store_single_run
            if os.path.exists(path):
                if not getattr(a, "reuse_existing_run_dir", False):
                    shutil.rmtree(path)
                    os.makedirs(path, exist_ok=False)
            else:
                os.makedirs(path, exist_ok=False)
            a.full_storage_path = path
        else:
            a.full_storage_path = create_experiment_folder(folder_name=a.storage_path)
            a.path_to_store_single_run = a.full_storage_path
        write_json({k: v for k, v in vars(a).items() if not k.startswith("_")},
                   os.path.join(a.full_storage_path, "configuration.json"), indent=3)

    def _memmap_paths(self):
        base = self.args.path_to_store_single_run
        return os.path.join(base, "memory_map_train_set.npy"), os.path.join(base, "memory_map_details.json")

    def create_and_store_kg(self) -> None:
        if not self.is_rank_zero():
            return
        mm, details = self._memmap_paths()
        if os.path.exists(mm) and os.path.exists(details) and self.distributed:
            return  # a previous run of the same directory already indexed the graph
        self.knowledge_graph = read_or_load_kg(self.args, cls=KG)
        kg = self.knowledge_graph
        a = self.args
        a.num_entities, a.num_relations = kg.num_entities, kg.num_relations
        a.num_tokens = kg.num_tokens
        a.max_length_subword_tokens = kg.max_length_subword_tokens
        a.ordered_bpe_entities = kg.ordered_bpe_entities
        self.report["num_train_triples"] = len(kg.train_set)
        self.report["num_entities"] = kg.num_entities
        self.report["num_relations"] = kg.num_relations
        self.report["max_length_subword_tokens"] = kg.max_length_subword_tokens
        self.report["runtime_kg_loading"] = time.time() - self.start_time
        ts = np.asarray(kg.train_set)
        write_json({"shape": tuple(ts.shape), "dtype": ts.dtype.str, "num_entities": kg.num_entities,
                    "num_relations": kg.num_relations}, details, indent=4)
        m = np.memmap(mm, dtype=ts.dtype, mode="w+", shape=ts.shape)
        m[:] = ts[:]
        m.flush()
        del m

    def load_from_memmap(self) -> None:
        mm, details = self._memmap_paths()
        d = load_json(details)
        self.knowledge_graph = np.memmap(mm, mode="r", dtype=d["dtype"], shape=tuple(d["shape"]))
        a = self.args
        a.num_entities, a.num_relations = d["num_entities"], d["num_relations"]
        a.num_tokens = a.max_length_subword_tokens = a.ordered_bpe_entities = None
        if not getattr(a, "full_storage_path", None):
            a.full_storage_path = a.path_to_store_single_run

    # ------------------------------------------------------------------ end of run
    def save_trained_model(self) -> None:
        self.trained_model.eval()
        self.trained_model.to("cpu")
        self.report.update(self.trained_model.mem_of_model())
        store(trained_model=self.trained_model, model_name="model", full_storage_path=self.args.full_storage_path,
              save_embeddings_as_csv=self.args.save_embeddings_as_csv)
        self.report["path_experiment_folder"] = self.args.full_storage_path
        self.report["num_entities"] = self.args.num_entities
        self.report["num_relations"] = self.args.num_relations

    def write_report(self) -> None:
        self.report["Runtime"] = time.time() - self.start_time
        write_json(self.report, os.path.join(self.args.full_storage_path, "report.json"), indent=4)

    def end(self, form_of_labelling: str) -> Optional[dict]:
        if not self.is_rank_zero():
            return None
        self.save_trained_model()
        self.write_report()
        if self.args.eval_model is None or self.knowledge_graph is None or isinstance(self.knowledge_graph, np.memmap):
            return {**self.report}
        # the model was stored from the host; the evaluation goes back to the device it was trained on, where the
        # ranking runs on the tensor cores (the reference evaluates on the CPU, dicee/executer.py:256-257)
        dev = getattr(getattr(self.trainer, "trainer", None), "device", None)
        if dev is not None and getattr(dev, "type", "cpu") == "cuda":
            self.trained_model.to(dev)
        self.evaluator.eval(dataset=self.knowledge_graph, trained_model=self.trained_model,
                            form_of_labelling=form_of_labelling)
        if hasattr(self.knowledge_graph, "wait_for_vocab_pickles"):
            self.knowledge_graph.wait_for_vocab_pickles()   # the run folder is complete when start() returns
        self.write_report()
        return {**self.report, **self.evaluator.report}

    def start(self) -> Optional[dict]:
        self.start_time = time.time()
        print(f"Start time:{datetime.datetime.now()}")
        self.create_and_store_kg()
        if self.distributed and dist.is_initialized():
            dist.barrier()
        if self.knowledge_graph is None:
            self.load_from_memmap()
        self.evaluator = Evaluator(args=self.args)
        if not getattr(self.args, "full_storage_path", None):
            self.args.full_storage_path = self.args.path_to_store_single_run
        self.trainer = DICE_Trainer(args=self.args, is_continual_training=self.is_continual_training,
                                    storage_path=self.args.full_storage_path, evaluator=self.evaluator)
        self.trained_model, form_of_labelling = self.trainer.start(knowledge_graph=self.knowledge_graph)
        return self.end(form_of_labelling)


class ContinuousExecute(Execute):
    """Resume training of a stored run for ``args.num_epochs`` more epochs.

    Only the weights are restored; optimiser state is fresh, as in the reference (``executer.py:361-440``)."""

    def __init__(self, args):
        path = args.continual_learning
        assert os.path.exists(path), f"Path doesn't exist {path}"
        assert os.path.isfile(os.path.join(path, "configuration.json"))
        prev = load_json(os.path.join(path, "configuration.json"))
        new = vars(args)
        prev["num_epochs"] = new["num_epochs"]
        prev["continual_learning"] = new["continual_learning"]
        try:
            rep = load_json(os.path.join(path, "report.json"))
            prev["num_entities"], prev["num_relations"] = rep["num_entities"], rep["num_relations"]
        except AssertionError:
            print("Couldn't find report.json.")
        prev["full_storage_path"] = path
        prev["path_to_store_single_run"] = path
        prev["_allow_no_source"] = True
        super().__init__(SimpleNamespace(**prev), continuous_training=True)

    def continual_start(self) -> dict:
        self.start_time = time.time()
        a = self.args
        self.trainer = DICE_Trainer(args=a, is_continual_training=True, storage_path=a.continual_learning)
        details = load_json(os.path.join(a.continual_learning, "memory_map_details.json"))
        kg = np.memmap(os.path.join(a.continual_learning, "memory_map_train_set.npy"), mode="r",
                       dtype=details["dtype"], shape=tuple(details["shape"]))
        a.num_entities, a.num_relations = details["num_entities"], details["num_relations"]
        a.num_tokens = a.max_length_subword_tokens = a.ordered_bpe_entities = None
        self.trained_model, form = self.trainer.continual_start(kg)
        self.save_trained_model()
        if a.eval_model is None:
            return self.report
        self.evaluator = Evaluator(args=a, is_continual_training=True)
        self.evaluator.dummy_eval(self.trained_model, form)
        return {**self.report, **self.evaluator.report}
