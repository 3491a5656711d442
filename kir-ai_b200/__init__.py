"""kirai_b200: a small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

Configuration and registry (``config``, ``registry``), weights (``weights``),
model parts (``parts``) and plans (``models``), the paged cache (``cache``), the
step function, scheduler and engine (``engine``), sampling (``sampling``) and
the CUDA kernels with their bindings (``csrc``).
"""
from . import registry  # registers the built-in architectures
from .engine.engine import Engine, GenerationOutput
from .registry import load_config, register_architecture, registered_architectures
from .sampling.params import SamplingParams

__all__ = ["registry", "load_config", "register_architecture", "registered_architectures", "Engine",
           "GenerationOutput", "SamplingParams"]
__version__ = "0.1.0"
