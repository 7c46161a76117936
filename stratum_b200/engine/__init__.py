from .model import (Model, config_from_dir, expected_tensors, load_model, model_from_tensors,
                    random_model_on_device)
from .step import Engine, StepBatch, StepEntry, StepError

__all__ = ["Model", "config_from_dir", "expected_tensors", "load_model", "model_from_tensors",
           "random_model_on_device", "Engine", "StepBatch", "StepEntry", "StepError"]
