"""Summarise a directory of runs: ``python -m dice_embeddings_b200.scripts.analyse_experiments --dir Experiments
--features model trainMRR testMRR``.

Joins ``configuration.json``, ``report.json`` (``Runtime``, ``NumParam``) and ``eval_report.json`` of every run
folder into one row, sorts by test MRR, prints the table and its LaTeX form and writes ``summary.csv`` into the
directory (reference ``dicee/analyse_experiments.py:117-170``)."""
from __future__ import annotations

import argparse
import json
import os
from typing import List, Optional

import pandas as pd


def collect(directory: str) -> pd.DataFrame:
    rows = []
    for name in sorted(os.listdir(directory)):
        full = os.path.join(directory, name)
        paths = [os.path.join(full, f) for f in ("configuration.json", "report.json", "eval_report.json")]
        if not os.path.isdir(full) or not all(os.path.isfile(p) for p in paths):
            continue
        config, report, evals = (json.load(open(p)) for p in paths)
        row = dict(config)
        row.update({k: report[k] for k in ("Runtime", "NumParam") if k in report})
        for split, prefix in (("Train", "train"), ("Val", "val"), ("Test", "test")):
            for k, v in (evals.get(split) or {}).items():
                row[f"{prefix}{k}"] = v
        row["full_storage_path"] = full
        rows.append(row)
    df = pd.DataFrame(rows)
    if "testMRR" in df.columns:
        df = df.sort_values(by=["testMRR"], ascending=False)
    return df


def analyse(directory: str, features: Optional[List[str]] = None) -> pd.DataFrame:
    df = collect(directory)
    pd.set_option("display.precision", 3)
    view = df
    if features:
        cols = [c for c in features if c in df.columns]
        view = df[cols] if cols else df
    print(view)
    try:
        print(view.to_latex(index=False, float_format="%.3f"))
    except Exception:  # LaTeX export needs jinja2
        pass
    path = os.path.join(directory, "summary.csv")
    df.to_csv(path, index=False)
    print(f"Saved in {path}")
    return df


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--dir", type=str, required=True, help="Directory containing run folders")
    p.add_argument("--features", nargs="+", default=[])
    a = p.parse_args(argv)
    analyse(a.dir, a.features)


if __name__ == "__main__":
    main()
