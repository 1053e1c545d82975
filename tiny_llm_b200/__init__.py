"""tiny_llm_b200: a small, whole inference engine for the Llama dense decoder on one B200 (sm_100a).

config/    typed configuration and the architecture registry
weights/   safetensors by tensor name, random-weights mode
parts/     norm, position encoding, mixer, feed-forward, block, model: put together from specs
cache/     paged keys and values with block tables per request, layer groups, state slots
engine/    the step function, the scheduler and the generate loop
sampling/  greedy, temperature, top-k, top-p
ops/       Python face of the kernels; csrc/ holds their CUDA sources
"""
from . import config, weights, cache, parts, sampling, engine  # noqa: F401
from .engine import Pipeline
from .sampling import SamplingParams

__version__ = "0.1.0"
