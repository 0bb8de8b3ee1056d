"""Sharded training checkpoints for row-sharded entity tables, with export to / import from the single-file layout.

The reference only stores the final ``model.pt`` (weights) and cannot resume an optimiser
(``dicee/static_funcs.py:408-428``; ``dicee/trainer/torch_trainer_ddp.py:96-97``).  A 10 M x 256 table with Adam
moments is ~30 GB, so here every rank writes its own rows:

``<dir>/manifest.json``          world size, table shape, sharding rule, step, optimiser constants, sampler counters
``<dir>/shard_00003.pt``         rows ``3, 3 + W, 3 + 2 W, ...`` of the entity table and of its two moment tables
``<dir>/replicated.pt``          relation table, coefficients and their moments (written by rank 0)

``load_shard`` re-shards on the fly when the world size changed between save and resume; ``export_model_pt``
assembles the reference's ``model.pt`` (``state_dict`` keys of the model) and ``import_model_pt`` goes back.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

MANIFEST = "manifest.json"
FORMAT_VERSION = 1


def shard_file(directory: str, rank: int) -> str:
    return os.path.join(directory, f"shard_{rank:05d}.pt")


def shard_rows(n: int, rank: int, world: int) -> int:
    return (n - rank + world - 1) // world if rank < n else 0


def save_shard(directory: str, rank: int, world: int, num_entities: int, tables: Dict[str, torch.Tensor],
               replicated: Optional[Dict[str, torch.Tensor]] = None, step: int = 0,
               extra: Optional[Dict] = None) -> None:
    """``tables``: name -> this rank's rows (``[>= shard_rows, D]``; padding rows are dropped).  Rank 0 also writes
    ``replicated`` and the manifest; callers synchronise the ranks around the call."""
    os.makedirs(directory, exist_ok=True)
    rows = shard_rows(num_entities, rank, world)
    payload = {k: v[:rows].detach().to("cpu", copy=True) for k, v in tables.items()}
    tmp = shard_file(directory, rank) + ".tmp"
    torch.save({"rank": rank, "world": world, "tables": payload}, tmp)
    os.replace(tmp, shard_file(directory, rank))
    if rank == 0:
        if replicated is not None:
            tmp = os.path.join(directory, "replicated.pt.tmp")
            torch.save({k: v.detach().to("cpu", copy=True) for k, v in replicated.items()}, tmp)
            os.replace(tmp, os.path.join(directory, "replicated.pt"))
        dim = int(next(iter(tables.values())).shape[1])
        man = {"format": FORMAT_VERSION, "world": world, "num_entities": int(num_entities), "dim": dim,
               "sharding": "cyclic: entity e -> shard e % world, row e // world", "tables": sorted(tables),
               "step": int(step), "extra": extra or {}}
        tmp = os.path.join(directory, MANIFEST + ".tmp")
        with open(tmp, "w") as f:
            json.dump(man, f, indent=2)
        os.replace(tmp, os.path.join(directory, MANIFEST))


def read_manifest(directory: str) -> Dict:
    with open(os.path.join(directory, MANIFEST)) as f:
        man = json.load(f)
    if man.get("format") != FORMAT_VERSION:
        raise ValueError(f"unsupported sharded checkpoint format {man.get('format')}")
    missing = [r for r in range(man["world"]) if not os.path.isfile(shard_file(directory, r))]
    if missing:
        raise FileNotFoundError(f"sharded checkpoint {directory} lacks shards {missing}")
    return man


def load_shard(directory: str, rank: int, world: int, device="cpu") -> Dict[str, torch.Tensor]:
    """This rank's rows of every table under the *current* world size (may differ from the saved one)."""
    man = read_manifest(directory)
    n, w_old = man["num_entities"], man["world"]
    if w_old == world:
        blob = torch.load(shard_file(directory, rank), map_location="cpu", weights_only=False)
        return {k: v.to(device) for k, v in blob["tables"].items()}
    mine = torch.arange(rank, n, world)                      # global ids this rank owns now
    out = {k: torch.empty(mine.numel(), man["dim"]) for k in man["tables"]}
    for old in range(w_old):
        sel = (mine % w_old) == old
        if not bool(sel.any()):
            continue
        blob = torch.load(shard_file(directory, old), map_location="cpu", weights_only=False)["tables"]
        for k in out:
            out[k][sel] = blob[k][mine[sel] // w_old].float()
    return {k: v.to(device) for k, v in out.items()}


def load_replicated(directory: str, device="cpu") -> Dict[str, torch.Tensor]:
    p = os.path.join(directory, "replicated.pt")
    if not os.path.isfile(p):
        return {}
    return {k: v.to(device) for k, v in torch.load(p, map_location="cpu", weights_only=False).items()}


def assemble_table(directory: str, name: str = "E") -> torch.Tensor:
    """Full ``[num_entities, D]`` table from all shards (host memory)."""
    man = read_manifest(directory)
    n, w = man["num_entities"], man["world"]
    full = torch.empty(n, man["dim"])
    for r in range(w):
        full[r::w] = torch.load(shard_file(directory, r), map_location="cpu", weights_only=False)["tables"][name].float()
    return full


def export_model_pt(directory: str, out_path: str, entity_key: str = "entity_embeddings.weight",
                    rename: Optional[Dict[str, str]] = None) -> Dict[str, torch.Tensor]:
    """Write a ``state_dict`` in the single-file layout: the assembled entity table under ``entity_key`` plus the
    replicated parameters whose names are model keys (optimiser moments are left out)."""
    sd = {entity_key: assemble_table(directory, "E")}
    for k, v in load_replicated(directory).items():
        if k.startswith(("m_", "v_")):
            continue
        sd[(rename or {}).get(k, k)] = v
    torch.save(sd, out_path)
    return sd


def import_model_pt(model_pt: str, directory: str, world: int, entity_key: str = "entity_embeddings.weight") -> None:
    """Split a single-file checkpoint into ``world`` shards with zero optimiser moments (start of a sharded run
    from a model trained elsewhere)."""
    sd = torch.load(model_pt, map_location="cpu", weights_only=False)
    E = sd[entity_key].float()
    rep = {k: v for k, v in sd.items() if k != entity_key}
    for r in range(world):
        rows = E[r::world]
        save_shard(directory, r, world, E.shape[0], {"E": rows, "mE": torch.zeros_like(rows), "vE": torch.zeros_like(rows)},
                   replicated=rep if r == 0 else None, step=0)
