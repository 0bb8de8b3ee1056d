from .base import AbstractCallback, AbstractTrainer, BatchLoader
from .torch_trainer import TorchTrainer
from .dice_trainer import DICE_Trainer, get_callbacks, initialize_trainer

__all__ = ["AbstractCallback", "AbstractTrainer", "BatchLoader", "TorchTrainer", "DICE_Trainer", "get_callbacks",
           "initialize_trainer"]
