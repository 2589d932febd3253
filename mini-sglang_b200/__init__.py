"""A small, whole inference engine for the Qwen3 dense decoder on one B200 (sm_100a).

Model folder (config.json + model.safetensors) -> generated tokens: typed configuration and
architecture registry (`config`), weights by tensor name (`weights`), layers assembled from
parts (`parts`), a paged cache manager (`cache`), one step function, a scheduler and the entry
points (`engine`), sampling (`sampling`), and the CUDA kernels (`csrc`, bound in `ops`).
"""

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "EngineArgs"):
        from . import engine as _e
        return getattr(_e, name)
    if name == "SamplingParams":
        from .sampling import SamplingParams
        return SamplingParams
    raise AttributeError(name)
