from .context import StepContext
from .engine import Engine, SequenceStep, StepError, require_cuda
from .model import DecoderModel
from .workspace import Workspace

__all__ = ["StepContext", "Engine", "SequenceStep", "StepError", "require_cuda", "DecoderModel",
           "Workspace"]
