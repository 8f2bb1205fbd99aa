"""ferrotorch_b200 -- a Blackwell-native deep-learning framework with the capability set of
ferrotorch (ferrotorch/src/lib.rs:59-177 is the reference's umbrella crate).

PyTorch is the tensor / autograd / module layer; this package adds hand-written sm_100a
kernels (``ops``), layers built on them (``nn``), flat-arena fused optimizers (``optim``),
the parallel runtime (``parallel``), model families (``models``), a trace-and-fuse JIT
(``jit``), checkpoint formats (``serialize``), a training loop (``train``) and a profiler
(``profiler``).
"""
__version__ = "0.1.0"

from . import _native  # noqa: F401
from . import ops  # noqa: F401
from . import autograd, core  # noqa: F401,E402

_SUBMODULES = ("nn", "optim", "data", "train", "vision", "jit", "serialize", "parallel", "models", "profiler", "hub",
               "cuda", "distributions", "utils", "tensor_ops")
# module names of the reference's umbrella crate (ferrotorch/src/lib.rs:72-177) that live elsewhere here
_ALIASES = {"gpu": "cuda", "distributed": "parallel", "llama": "models.llama_api", "ml": "utils.ml", "tokenize": "utils.text",
            "grammar": "utils.grammar", "jit_script": "jit", "prelude": "prelude", "bert": "models.pretrained",
            "whisper": "models.pretrained", "graph": "models.pretrained", "rl": "models.pretrained",
            "diffusion": "models.diffusion", "cubecl": "utils.portable_kernels"}
__all__ = ["ops", "autograd", "core", "__version__", *_SUBMODULES, *_ALIASES]


def __getattr__(name):
    """``import ferrotorch_b200 as ft; ft.nn.Linear`` -- sub-packages load on first use, like the
    umbrella crate's re-exports (ferrotorch/src/lib.rs:59-177) without its compile-time cost."""
    if name in _SUBMODULES:
        import importlib

        return importlib.import_module("." + name, __name__)
    if name in _ALIASES:
        import importlib

        return importlib.import_module("." + _ALIASES[name], __name__)
    if not name.startswith("_"):
        # the flat tensor API of the reference's core crate: its own spellings first, torch's second
        import importlib

        import torch

        ops_mod = importlib.import_module(".tensor_ops", __name__)
        try:
            return getattr(ops_mod, name)
        except AttributeError:
            pass
        from .ops import ptq

        more = importlib.import_module(".tensor_ops_more", __name__)
        for home in (more, core, autograd, ptq, torch, torch.linalg, torch.special, torch.nn.functional, torch.signal.windows,
                     torch.fft):
            if hasattr(home, name):
                return getattr(home, name)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
