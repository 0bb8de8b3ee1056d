"""Model zoo and registry (reference ``dicee/static_funcs.py:33-54``: name → class and form of labelling)."""
from .base import BaseKGE, IdentityClass
from .real import DistMult, TransE, Shallom, Pyke
from .hypercomplex import ComplEx, QMult, OMult, DualE
from .clifford import Keci, CKeci, DeCaL
from .conv import ConEx, AConEx, ConvQ, AConvQ, ConvO, AConvO
from .transformers import CoKE, BytE, Block, GPTConfig, CoKEConfig
from .function_space import FMult, GFMult, FMult2, LFMult1, LFMult
from .literal import LiteralEmbeddings
from .ensemble import EnsembleKGE
from .pykeen import PykeenKGE

MODEL_REGISTRY = {
    "Shallom": (Shallom, "RelationPrediction"),
    "ConEx": (ConEx, "EntityPrediction"),
    "AConEx": (AConEx, "EntityPrediction"),
    "QMult": (QMult, "EntityPrediction"),
    "OMult": (OMult, "EntityPrediction"),
    "ConvQ": (ConvQ, "EntityPrediction"),
    "AConvQ": (AConvQ, "EntityPrediction"),
    "ConvO": (ConvO, "EntityPrediction"),
    "AConvO": (AConvO, "EntityPrediction"),
    "ComplEx": (ComplEx, "EntityPrediction"),
    "DistMult": (DistMult, "EntityPrediction"),
    "TransE": (TransE, "EntityPrediction"),
    "Pyke": (Pyke, "EntityPrediction"),
    "Keci": (Keci, "EntityPrediction"),
    "CKeci": (CKeci, "EntityPrediction"),
    "BytE": (BytE, "EntityPrediction"),
    "LFMult": (LFMult, "EntityPrediction"),
    "LFMult1": (LFMult1, "EntityPrediction"),
    "FMult": (FMult, "EntityPrediction"),
    "FMult2": (FMult2, "EntityPrediction"),
    "GFMult": (GFMult, "EntityPrediction"),
    "DeCaL": (DeCaL, "EntityPrediction"),
    "DualE": (DualE, "EntityPrediction"),
    "CoKE": (CoKE, "EntityPrediction"),
}


def initialize_model(args: dict, verbose: int = 0):
    """Instantiate ``args['model']`` → ``(model, form_of_labelling)``
    (reference ``dicee/static_funcs.py:483-509``)."""
    name = args["model"]
    if "pykeen" in name.lower():
        return PykeenKGE(args=args), "EntityPrediction"
    if name not in MODEL_REGISTRY:
        raise ValueError(f"--model_name: {name} is not found.")
    cls, form = MODEL_REGISTRY[name]
    return cls(args=args), form


intialize_model = initialize_model  # spelling used by the reference API
