from .engine import Engine, StepEntry, StepError
from .model import DecoderModel, expected_tensors
from .context import EntryView, StepContext
from .generate import GenerateOutput, GenerateRequest, GenerationError, generate, plan_batches
from .api import BuiltEngine, EngineConfig, build

__all__ = ["Engine", "StepEntry", "StepError", "DecoderModel", "expected_tensors", "EntryView",
           "StepContext", "GenerateOutput", "GenerateRequest", "GenerationError", "generate",
           "plan_batches", "BuiltEngine", "EngineConfig", "build"]
