"""cosmos_b200: a Blackwell-native (B200, sm_100a) training and inference framework with the capabilities of
NVIDIA Cosmos 3 (Generator + Reasoner towers of one Mixture-of-Transformers model).

The heavy modules are imported on first use, so `import cosmos_b200` stays cheap:

    cosmos_b200.Cosmos3OmniPipeline                      pipeline class (`from_pretrained`, `__call__`, `step`)
    cosmos_b200.UniPCMultistepScheduler                  scheduler handle of the pipeline
    cosmos_b200.Cosmos3ReasonerForConditionalGeneration  Reasoner class in the transformers style
    cosmos_b200.ops                                      fused ops on the sm_100a kernel library
"""
from __future__ import annotations

__version__ = "0.1.0"

_LAZY = {
    "Cosmos3OmniPipeline": ("cosmos_b200.pipeline", "Cosmos3OmniPipeline"),
    "UniPCMultistepScheduler": ("cosmos_b200.pipeline", "UniPCMultistepScheduler"),
    "Cosmos3Output": ("cosmos_b200.pipeline", "Cosmos3Output"),
    "Cosmos3ReasonerForConditionalGeneration": ("cosmos_b200.hf", "Cosmos3ReasonerForConditionalGeneration"),
    "Cosmos3ReasonerConfig": ("cosmos_b200.hf", "Cosmos3ReasonerConfig"),
    "MoTConfig": ("cosmos_b200.config", "MoTConfig"),
    "SamplingConfig": ("cosmos_b200.config", "SamplingConfig"),
    "DecodingConfig": ("cosmos_b200.config", "DecodingConfig"),
    "ParallelConfig": ("cosmos_b200.config", "ParallelConfig"),
}
__all__ = ["__version__", *_LAZY]


def __getattr__(name: str):
    if name in _LAZY:
        import importlib

        module, attr = _LAZY[name]
        value = getattr(importlib.import_module(module), attr)
        globals()[name] = value
        return value
    raise AttributeError(f"module 'cosmos_b200' has no attribute '{name}'")


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
