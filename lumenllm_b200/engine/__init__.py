from .engine import Engine, StepEntry, StepError
from .model import DecoderModel, expected_tensors
from .context import EntryView, StepContext

__all__ = ["Engine", "StepEntry", "StepError", "DecoderModel", "expected_tensors", "EntryView",
           "StepContext"]
