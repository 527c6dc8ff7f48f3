"""A B200-native (sm_100a) model library with generation of its own, for Qwen3 dense.

From a model folder (config.json + safetensors) or seeded random weights to the next token on
one GPU: typed configuration and architecture registry, weights by tensor name, layers composed
from registered parts, a paged cache with a slot per sequence, one step function, a generation
loop with greedy / temperature / nucleus sampling, trace replay, and hand-written CUDA kernels.
"""
from .config import ConfigError, Qwen3Config, config_from_folder, register_architecture
from .api import GenerateResult, Model
from .engine import Engine, StepError
from .sampling import SamplingParams
from .weights import RandomInit, WeightsError, write_model_folder

__version__ = "0.1.0"

__all__ = ["ConfigError", "Qwen3Config", "config_from_folder", "register_architecture", "Engine", "StepError", "Model", "GenerateResult", "SamplingParams",
           "RandomInit", "WeightsError", "write_model_folder"]
