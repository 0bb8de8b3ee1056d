"""Per-attribute MAE / RMSE of a trained literal regressor (reference
``dicee/evaluation/literal_prediction.py:14-121``); writes ``lit_predictions.csv`` and ``lit_eval_results.csv``."""
from __future__ import annotations

import os
from typing import Optional

import numpy as np
import pandas as pd


def evaluate_literal_prediction(kge_model, eval_file_path: str = None, store_lit_preds: bool = True,
                                eval_literals: bool = True, loader_backend: str = "pandas",
                                return_attr_error_metrics: bool = False) -> Optional[pd.DataFrame]:
    if getattr(kge_model, "literal_model", None) is None:
        raise RuntimeError("Literal model is not trained or loaded.")
    df = kge_model.literal_dataset.load_and_validate_literal_data(file_path=eval_file_path,
                                                                  loader_backend=loader_backend)
    df = df[df["head"].isin(kge_model.entity_to_idx.keys())
            & df["attribute"].isin(kge_model.data_property_to_idx.keys())].copy()
    assert len(df) > 0, "No valid (entity, attribute) pair in the evaluation file"
    df["predictions"] = kge_model.predict_literals(entity=df["head"].to_list(), attribute=df["attribute"].to_list())
    if store_lit_preds:
        df[["head", "attribute", "predictions"]].to_csv(os.path.join(kge_model.path, "lit_predictions.csv"), index=False)
    if not eval_literals:
        return None
    err = df["value"].astype(float) - df["predictions"].astype(float)
    g = pd.DataFrame({"attribute": df["attribute"], "ae": err.abs(), "se": err ** 2}).groupby("attribute")
    metrics = pd.DataFrame({"MAE": g["ae"].mean(), "RMSE": np.sqrt(g["se"].mean())}).reset_index()
    metrics.to_csv(os.path.join(kge_model.path, "lit_eval_results.csv"), index=False)
    print("Literal-Prediction evaluation results on Test Set")
    print(metrics)
    return metrics if return_attr_error_metrics else None
