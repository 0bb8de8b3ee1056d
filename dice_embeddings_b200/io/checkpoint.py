"""Run-directory layout: writing and reading trained models.

The directory contract is the reference's (``dicee/static_funcs.py:246-299, 395-428``):

* ``model.pt`` — ``state_dict`` of CPU tensors; ``model_partial_{i}.pt`` for the replicas of an
  :class:`EnsembleKGE`;
* ``configuration.json`` — the argument namespace; ``report.json`` — carries ``num_entities`` /
  ``num_relations``, which model re-construction reads;
* ``entity_to_idx.csv`` / ``relation_to_idx.csv`` — pandas layout (index column + ``entity`` / ``relation``);
* optional ``{Model}_entity_embeddings.csv`` / ``{Model}_relation_embeddings.csv`` indexed by the strings.

A folder produced by the reference loads here and vice versa.
"""
from __future__ import annotations

import datetime
import json
import os
import pickle
from typing import Dict, List, Optional, Tuple

import numpy as np
import pandas as pd
import torch

from ..models import BaseKGE, EnsembleKGE, initialize_model


def load_json(path: str) -> Dict:
    assert os.path.isfile(path), f"{path} is not found"
    with open(path, "r") as f:
        return json.load(f)


def save_pickle(*, data=None, file_path: str) -> None:
    if data is not None:
        with open(file_path, "wb") as f:
            pickle.dump(data, f)


def load_pickle(file_path: str):
    with open(file_path, "rb") as f:
        return pickle.load(f)


def create_experiment_folder(folder_name: str = "Experiments") -> str:
    """``<cwd>/<folder_name>/<timestamp>`` (colons replaced), created."""
    path = os.path.join(os.getcwd(), folder_name, str(datetime.datetime.now()).replace(":", "-"))
    os.makedirs(path)
    return path


def _json_default(o):
    if isinstance(o, (np.integer,)):
        return int(o)
    if isinstance(o, (np.floating,)):
        return float(o)
    if isinstance(o, np.ndarray):
        return o.tolist()
    if isinstance(o, (set, tuple)):
        return list(o)
    return str(o)


def write_json(obj: Dict, path: str, indent: int = 4) -> None:
    with open(path, "w") as f:
        json.dump(obj, f, indent=indent, default=_json_default)


def save_checkpoint_model(model, path: str) -> None:
    """``state_dict`` → ``path``; replicas of an ensemble go to ``…/model_partial_{i}.pt``."""
    if isinstance(model, EnsembleKGE):
        for i, part in enumerate(model):
            torch.save(_cpu_state(part), path.replace("model.pt", f"model_partial_{i}.pt"))
    elif isinstance(model, torch.nn.Module):
        torch.save(_cpu_state(model), path)
    else:
        torch.save(_cpu_state(model.model), path)


def _cpu_state(module: torch.nn.Module) -> Dict[str, torch.Tensor]:
    return {k: v.detach().to("cpu") for k, v in module.state_dict().items()}


def save_embeddings(embeddings: np.ndarray, indexes: List, path: str) -> None:
    pd.DataFrame(embeddings, index=indexes).to_csv(path)


def store(trained_model, model_name: str = "model", full_storage_path: str = None,
          save_embeddings_as_csv: bool = False) -> None:
    """Write the weights and optionally the embedding CSVs of a trained model."""
    assert full_storage_path is not None and len(model_name) > 1
    save_checkpoint_model(model=trained_model, path=os.path.join(full_storage_path, f"{model_name}.pt"))
    if not save_embeddings_as_csv:
        return
    ent, rel = trained_model.get_embeddings()
    entity = pd.read_csv(os.path.join(full_storage_path, "entity_to_idx.csv"), index_col=0)["entity"]
    save_embeddings(ent.cpu().numpy(), indexes=entity.to_list(),
                    path=os.path.join(full_storage_path, trained_model.name + "_entity_embeddings.csv"))
    if rel is not None:
        relations = pd.read_csv(os.path.join(full_storage_path, "relation_to_idx.csv"), index_col=0)["relation"]
        save_embeddings(rel.cpu().numpy(), indexes=relations.to_list(),
                        path=os.path.join(full_storage_path, trained_model.name + "_relation_embeddings.csv"))


def read_index_csv(path: str, column: str) -> Dict[str, int]:
    """``{string: id}`` from either the pandas layout (index column first) or the polars layout
    (``index,entity`` header)."""
    df = pd.read_csv(path, dtype=str, keep_default_na=False)
    if column not in df.columns:
        column = df.columns[-1]
    idx_col = [c for c in df.columns if c != column]
    ids = df[idx_col[0]].astype(int).tolist() if idx_col else list(range(len(df)))
    return {s: i for s, i in zip(df[column].tolist(), ids)}


def _configs_for_model(path: str, weights: Dict[str, torch.Tensor]) -> Dict:
    configs = load_json(os.path.join(path, "configuration.json"))
    report = load_json(os.path.join(path, "report.json")) if os.path.isfile(os.path.join(path, "report.json")) else {}
    if configs.get("byte_pair_encoding", None) and configs.get("model") != "BytE":
        configs["ordered_bpe_entities"] = load_pickle(os.path.join(path, "ordered_bpe_entities.p"))
        configs["num_tokens"] = weights["token_embeddings.weight"].shape[0]
        configs["max_length_subword_tokens"] = report.get("max_length_subword_tokens")
    elif configs.get("byte_pair_encoding", None):
        configs["num_tokens"] = weights["lm_head.weight"].shape[0]
    else:
        configs["num_entities"] = report.get("num_entities", configs.get("num_entities"))
        configs["num_relations"] = report.get("num_relations", configs.get("num_relations"))
        if configs["num_entities"] is None and "entity_embeddings.weight" in weights:
            configs["num_entities"] = weights["entity_embeddings.weight"].shape[0]
            configs["num_relations"] = weights["relation_embeddings.weight"].shape[0]
    if configs.get("normalization") == "None":
        configs["normalization"] = None
    return configs


def load_model(path_of_experiment_folder: str, model_name: str = "model.pt", verbose: int = 0
               ) -> Tuple[BaseKGE, Optional[Tuple[dict, dict]]]:
    """Rebuild the module from ``configuration.json`` + ``report.json``, load the weights, freeze, ``eval()``.
    Returns ``(model, (entity_to_idx, relation_to_idx))`` (``None`` mappings for byte-pair-encoded runs)."""
    p = path_of_experiment_folder
    weights = torch.load(os.path.join(p, model_name), map_location="cpu", weights_only=False)
    if isinstance(weights, torch.nn.Module):
        weights = weights.state_dict()
    weights = {k.replace("_orig_mod.", ""): v for k, v in weights.items()}
    configs = _configs_for_model(p, weights)
    model, _ = initialize_model(configs, verbose)
    model.load_state_dict(weights)
    for prm in model.parameters():
        prm.requires_grad = False
    model.eval()
    if configs.get("byte_pair_encoding", None):
        return model, None
    return model, (read_index_csv(os.path.join(p, "entity_to_idx.csv"), "entity"),
                   read_index_csv(os.path.join(p, "relation_to_idx.csv"), "relation"))


def load_model_ensemble(path_of_experiment_folder: str) -> Tuple[BaseKGE, Tuple[dict, dict]]:
    """Average the parameters of all ``model*.pt`` checkpoints of a folder into one model
    (reference ``dicee/static_funcs.py:302-365``)."""
    p = path_of_experiment_folder
    files = sorted(f for f in os.listdir(p) if f.startswith("model") and f.endswith(".pt"))
    assert files, f"No model checkpoint under {p}"
    states = [torch.load(os.path.join(p, f), map_location="cpu", weights_only=False) for f in files]
    avg = {k: torch.stack([s[k].float() for s in states]).mean(0).to(states[0][k].dtype) if states[0][k].is_floating_point()
           else states[0][k] for k in states[0]}
    configs = _configs_for_model(p, avg)
    model, _ = initialize_model(configs)
    model.load_state_dict(avg)
    for prm in model.parameters():
        prm.requires_grad = False
    model.eval()
    return model, (read_index_csv(os.path.join(p, "entity_to_idx.csv"), "entity"),
                   read_index_csv(os.path.join(p, "relation_to_idx.csv"), "relation"))


def select_model(args: dict, is_continual_training: bool = False, storage_path: Optional[str] = None,
                 tp_devices=None):
    """New model (an :class:`EnsembleKGE` for ``trainer == 'TP'``) or, for continual training, the stored
    weights with gradients re-enabled (reference ``dicee/static_funcs.py:197-244``)."""
    if is_continual_training:
        files = [f for f in os.listdir(storage_path) if os.path.isfile(os.path.join(storage_path, f))]
        n_part = len([f for f in files if "partial" in f])
        if n_part >= 1:
            models, form = [], None
            for i in range(n_part):
                m, form = initialize_model(args)
                m.load_state_dict(torch.load(os.path.join(storage_path, f"model_partial_{i}.pt"), map_location="cpu",
                                             weights_only=False))
                for prm in m.parameters():
                    prm.requires_grad = True
                m.train()
                models.append(m)
            return EnsembleKGE(pretrained_models=models, devices=tp_devices), form
        model, form = initialize_model(args)
        model.load_state_dict(torch.load(os.path.join(storage_path, "model.pt"), map_location="cpu",
                                         weights_only=False))
        for name, prm in model.named_parameters():
            prm.requires_grad = not (args.get("model") == "CKeci" and "coefficients" in name)
        model.train()
        return model, form
    if args.get("trainer") == "TP":
        n = len(tp_devices) if tp_devices is not None else max(torch.cuda.device_count(), 1)
        models, form = [], None
        for i in range(n):
            a = dict(args)
            a["random_seed"] = i
            torch.manual_seed(i)
            m, form = initialize_model(a)
            models.append(m)
        return EnsembleKGE(models=models, devices=tp_devices), form
    return initialize_model(args)


def write_csv_from_model_parallel(path: str) -> None:
    """Concatenate the embedding tables of ``model_partial_*.pt`` along dim 1 and write the two CSVs
    (reference ``dicee/static_funcs.py:798-818``)."""
    parts = sorted(f for f in os.listdir(path) if f.startswith("model_partial_") and f.endswith(".pt"))
    assert parts
    ents, rels = [], []
    for f in parts:
        sd = {k.replace("_orig_mod.", ""): v for k, v in torch.load(os.path.join(path, f), map_location="cpu").items()}
        ents.append(sd["entity_embeddings.weight"])
        rels.append(sd["relation_embeddings.weight"])
    e2i = read_index_csv(os.path.join(path, "entity_to_idx.csv"), "entity")
    r2i = read_index_csv(os.path.join(path, "relation_to_idx.csv"), "relation")
    save_embeddings(torch.cat(ents, 1).numpy(), list(e2i.keys()), os.path.join(path, "entity_embeddings.csv"))
    save_embeddings(torch.cat(rels, 1).numpy(), list(r2i.keys()), os.path.join(path, "relation_embeddings.csv"))


def from_pretrained_model_write_embeddings_into_csv(path: str) -> None:
    """Export ``{Model}_entity_embeddings.csv`` / ``…_relation_embeddings.csv`` of a stored run
    (reference ``dicee/static_funcs.py:821-858``)."""
    config = load_json(os.path.join(path, "configuration.json"))
    if config.get("trainer") == "TP":
        return write_csv_from_model_parallel(path)
    model, (e2i, r2i) = load_model(path)
    ent, rel = model.get_embeddings()
    save_embeddings(ent.numpy(), list(e2i.keys()), os.path.join(path, f"{model.name}_entity_embeddings.csv"))
    if rel is not None:
        save_embeddings(rel.numpy(), list(r2i.keys()), os.path.join(path, f"{model.name}_relation_embeddings.csv"))
