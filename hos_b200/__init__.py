"""hos_b200: a small Gemma-2 generation library for one B200 GPU.

    from hos_b200 import Engine
    eng = Engine("/path/to/model_folder")             # config.json + model.safetensors
    ids = eng.generate([2, 651, 1234], max_tokens=32)   # greedy by default
"""
from .errors import (CacheError, ExtensionMissingError, FormatError, HosError, IoError,  # noqa: F401
                     KernelError, MissingMetaError, MissingTensorError, SpecError,
                     UnsupportedArchError, WeightMismatchError)

__version__ = "0.2.0"


def version() -> str:
    return __version__


def __getattr__(name):
    # the engine pulls in torch and the kernels: loaded on first use
    if name in ("Engine", "Runner"):
        from . import engine
        return getattr(engine, name)
    if name in ("SamplingParams",):
        from . import sampling
        return getattr(sampling, name)
    raise AttributeError(name)
