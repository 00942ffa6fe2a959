"""Core layer: configuration, instantiation, typed modules, ModelPT, .nemo files, optimizers, trainer."""
from .config import DictConfig, ListConfig, OmegaConf, hydra_runner, open_dict  # noqa: F401
from .modelpt import ModelPT  # noqa: F401
from .module import AccessMixin, Loss, NeuralModule  # noqa: F401
from .neural_types import NeuralType, typecheck  # noqa: F401
from .save_restore import SaveRestoreConnector  # noqa: F401
from .trainer import Callback, Trainer  # noqa: F401
