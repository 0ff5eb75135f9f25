"""atom_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a), in the manner of
ROCm/ATOM.  ``from atom_b200 import LLMEngine, SamplingParams`` mirrors the reference's
``from atom import LLMEngine, SamplingParams`` (atom/__init__.py:4-29)."""

__version__ = "0.1.0"


def __getattr__(name):
    # Lazy, so that importing the package for its configuration or cache manager does not
    # pull in the device code (the reference imports LLMEngine lazily too, atom/__init__.py:24-29).
    if name == "LLMEngine":
        from .engine.llm_engine import LLMEngine
        return LLMEngine
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    raise AttributeError(name)
