"""Small helpers that user code imports from the package root in the reference
(``from dicee import timeit, load_numpy, evaluate, ...``; ``dicee/static_funcs.py``)."""
from __future__ import annotations

import functools
import os
import re
import time
from typing import Callable, Dict, Iterable, Tuple

import numpy as np
import torch


def timeit(func: Callable) -> Callable:
    """Print wall-clock seconds and resident memory after each call (reference ``static_funcs.py:129-146``)."""
    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        t0 = time.perf_counter()
        out = func(*args, **kwargs)
        dt = time.perf_counter() - t0
        try:
            import psutil
            mem = psutil.Process(os.getpid()).memory_info().rss / 1e6
            print(f"{func.__name__} took {dt:.4f} s | current memory usage {mem:.1f} MB")
        except Exception:
            print(f"{func.__name__} took {dt:.4f} s")
        return out
    return wrapper


def save_numpy_ndarray(*, data: np.ndarray, file_path: str) -> None:
    with open(file_path, "wb") as f:
        np.save(f, data)


@timeit
def load_numpy(path: str) -> np.ndarray:
    with open(path, "rb") as f:
        return np.load(f)


def numpy_data_type_changer(train_set: np.ndarray, num: int) -> np.ndarray:
    """Smallest signed integer dtype that holds ``num`` (reference ``static_funcs.py:373-392``)."""
    for dt in (np.int8, np.int16, np.int32):
        if np.iinfo(dt).max > num:
            return train_set.astype(dt)
    return train_set.astype(np.int64)


def load_term_mapping(file_path: str):
    """``entity_to_idx`` / ``relation_to_idx`` from ``<file_path>.csv`` or a pickle (older runs)."""
    import pandas as pd
    if os.path.isfile(file_path + ".csv"):
        return pd.read_csv(file_path + ".csv", index_col=0)
    if os.path.isfile(file_path + ".p"):
        import pickle
        with open(file_path + ".p", "rb") as f:
            return pickle.load(f)
    raise FileNotFoundError(file_path)


def vocab_to_parquet(vocab_to_idx, name: str, path_for_serialization: str, print_into: str = "") -> None:
    import pandas as pd
    if print_into:
        print(print_into)
    pd.DataFrame({"term": list(vocab_to_idx.keys()), "idx": list(vocab_to_idx.values())}).to_parquet(
        os.path.join(path_for_serialization, name), compression="gzip")


def create_recipriocal_triples(df):
    """Append ``(o, p_inverse, s)`` for every ``(s, p, o)`` row of a three-column frame
    (reference ``static_funcs.py:56-72``; the spelling of the name is the reference's)."""
    import pandas as pd
    inv = pd.DataFrame({"subject": df["object"], "relation": df["relation"].astype(str) + "_inverse",
                        "object": df["subject"]})
    return pd.concat([df, inv], ignore_index=True)


def exponential_function(x: np.ndarray, lam: float, ascending_order: bool = True) -> torch.Tensor:
    """Normalised exponentially decaying weights (ensemble coefficients)."""
    w = np.exp(-lam * np.asarray(x, dtype=np.float64))
    w = w / w.sum()
    return torch.tensor((w[::-1] if ascending_order else w).copy(), dtype=torch.float32)


def continual_training_setup_executor(executor) -> None:
    """Storage path of a continued run: reuse the given folder (reference ``static_funcs.py:642-658``)."""
    if executor.is_continual_training:
        executor.args.full_storage_path = getattr(executor.args, "continual_learning", None) or \
            executor.args.full_storage_path
    os.makedirs(executor.args.full_storage_path, exist_ok=True)


def evaluate(entity_to_idx: Dict[str, int], scores: Dict, easy_answers: Dict, hard_answers: Dict
             ) -> Tuple[float, float, float, float]:
    """Filtered MRR / H@1 / H@3 / H@10 of multi-hop query answers: every hard answer is ranked against all
    entities with the other (easy and hard) answers removed (reference ``static_funcs.py:677-734``).

    ``scores[query]`` holds one score per entity in the order of ``entity_to_idx``; the per-query work is one
    ``argsort`` plus vector arithmetic instead of the reference's Python loops over the sorted list."""
    names = list(entity_to_idx.keys())
    pos = {e: i for i, e in enumerate(names)}
    tot = np.zeros(4)
    for query, s in scores.items():
        s = torch.as_tensor(s).detach().float().cpu().numpy().ravel()
        order = np.argsort(-s, kind="stable")
        rank_of = np.empty(len(order), dtype=np.int64)
        rank_of[order] = np.arange(len(order))
        easy = [pos[e] for e in easy_answers[query] if e in pos]
        hard = [pos[e] for e in hard_answers[query] if e in pos]
        if not hard:
            continue
        all_r = np.sort(rank_of[np.asarray(easy + hard, dtype=np.int64)])
        hard_r = rank_of[np.asarray(hard, dtype=np.int64)]
        before = np.searchsorted(all_r, hard_r, side="left")   # answers ranked ahead of each hard answer
        r = hard_r - before + 1.0
        tot += (np.mean(1.0 / r), np.mean(r <= 1), np.mean(r <= 3), np.mean(r <= 10))
    n = max(len(scores), 1)
    return tuple(float(v) for v in tot / n)


def download_file(url: str, destination_folder: str = ".") -> None:
    import requests
    from urllib.parse import urlparse
    r = requests.get(url, stream=True, timeout=120)
    if r.status_code != 200:
        print(f"Failed to download: {url}")
        return
    name = os.path.join(destination_folder, os.path.basename(urlparse(url).path))
    with open(name, "wb") as f:
        for chunk in r.iter_content(chunk_size=1 << 16):
            if chunk:
                f.write(chunk)
    print(f"Downloaded: {name}")


def download_files_from_url(base_url: str, destination_folder: str = ".") -> None:
    """Fetch every file linked from a directory listing page (no HTML parser dependency)."""
    import requests
    r = requests.get(base_url, timeout=60)
    if r.status_code != 200:
        print("ERROR:", r.status_code)
        return
    hrefs: Iterable[str] = {h for h in re.findall(r'href="([^"]+)"', r.text) if len(h) > 3 and "." in h
                            and not h.startswith("?") and not h.endswith("/")}
    for h in sorted(hrefs):
        download_file(base_url.rstrip("/") + "/" + h, destination_folder)


def download_pretrained_model(url: str) -> str:
    assert url[-1] != "/"
    dir_name = url[url.rfind("/") + 1:]
    if os.path.exists(dir_name):
        print("Path exists", dir_name)
    else:
        os.mkdir(dir_name)
        download_files_from_url(f"https://files.dice-research.org/projects/DiceEmbeddings/{dir_name}", dir_name)
    return dir_name
