"""B200-native knowledge-graph-embedding framework with the CLI, Python API and checkpoint layout of ``dicee``."""
from .config import Namespace
from .executor import ContinuousExecute, Execute
from .kge import KGE
from .data.kg import KG
from .models import *  # noqa: F401,F403
from .models import MODEL_REGISTRY, initialize_model, intialize_model
from .evaluation import Evaluator
from .trainer import DICE_Trainer

__version__ = "0.1.0"
__all__ = ["Namespace", "Execute", "ContinuousExecute", "KGE", "KG", "Evaluator", "DICE_Trainer", "MODEL_REGISTRY",
           "initialize_model", "intialize_model"]
