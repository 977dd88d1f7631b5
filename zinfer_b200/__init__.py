"""zinfer_b200: a small, whole inference engine for one B200, for the Qwen3 dense
architecture, in the manner of NeoZedAtlas/Zinfer.

From a model folder (config.json + model.safetensors) and token ids to generated
token ids: typed configuration and registry (``config``), weights by name
(``weights``), layers put together from parts (``parts``), a paged cache manager
(``cache``), one step function with a scheduler above it (``engine``), sampling
(``sampling``) and hand-written sm_100a kernels (``csrc``, through ``ops``).
"""
from . import config  # registers the architectures
from . import parts   # registers the parts

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "SamplingParams", "generate"):
        from .engine import api
        return getattr(api, name)
    raise AttributeError(name)
