"""nnis_b200: a small Llama generation library for one B200 (sm_100a).

Layout: ``config`` (typed configuration, registry), ``weights`` (safetensors
by name, random-weights mode), ``parts`` (norm, position encoding, attention,
feed-forward, block), ``cache`` (slots, paged keys and values, state),
``engine`` (model, step function, generation, replay), ``sampling``,
``csrc`` (CUDA kernels and their build), ``cli``.
"""
__version__ = "0.1.0"
