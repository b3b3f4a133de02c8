"""nnis_b200: a small Llama generation library for one B200 (sm_100a).

Layout: ``config`` (typed configuration, registry), ``weights`` (safetensors
by name, random-weights mode), ``parts`` (norm, position encoding, attention,
feed-forward, block), ``cache`` (slots, paged keys and values, state),
``engine`` (model, step function, generation, replay), ``sampling``,
``csrc`` (CUDA kernels and their build), ``cli``.
"""
__version__ = "0.1.0"


def __getattr__(name):
    # the entry points import torch and the kernels; keep "import nnis_b200" light
    if name in ("LLM", "InferenceSession"):
        from .engine import api
        return getattr(api, name)
    if name in ("GenerationConfig", "GenerationRequest", "GenerationResult", "StreamControl"):
        from .engine import generate
        return getattr(generate, name)
    if name == "SamplingConfig":
        from .sampling import SamplingConfig
        return SamplingConfig
    if name in ("execute", "ProcessContractError"):
        from .cli import process
        return getattr(process, name)
    if name == "Engine":
        from .engine import Engine
        return Engine
    raise AttributeError(name)
