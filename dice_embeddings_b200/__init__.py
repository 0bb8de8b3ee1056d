"""B200-native knowledge-graph-embedding framework with the CLI, Python API and checkpoint layout of ``dicee``."""
from .config import Namespace
from .executor import ContinuousExecute, Execute
from .kge import KGE
from .data.kg import KG
from .models import *  # noqa: F401,F403
from .models import MODEL_REGISTRY, initialize_model, intialize_model
from .evaluation import Evaluator
from .trainer import DICE_Trainer
from .data.query_generator import QueryGenerator
from .data.datasets import *  # noqa: F401,F403
from .io.checkpoint import (create_experiment_folder, load_json, load_model, load_model_ensemble, load_pickle,  # noqa: F401
                            save_checkpoint_model, save_embeddings, save_pickle, select_model, store,
                            write_csv_from_model_parallel, from_pretrained_model_write_embeddings_into_csv)
from .data.vocab import get_ee_vocab, get_er_vocab, get_re_vocab  # noqa: F401
from .utils import *  # noqa: F401,F403

__version__ = "0.1.0"
__all__ = ["QueryGenerator", "Namespace", "Execute", "ContinuousExecute", "KGE", "KG", "Evaluator", "DICE_Trainer", "MODEL_REGISTRY",
           "initialize_model", "intialize_model"]
