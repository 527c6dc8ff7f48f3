"""The engine: model, step function, decode graphs, generation loop, trace replay."""
from .engine import DTYPES, Engine, StepContext, StepError
from .model import CausalLM, optional_duplicates_of_spec, tensor_needs_of_spec
from .workspace import Workspace

__all__ = ["DTYPES", "Engine", "StepContext", "StepError", "CausalLM", "optional_duplicates_of_spec",
           "tensor_needs_of_spec", "Workspace"]
