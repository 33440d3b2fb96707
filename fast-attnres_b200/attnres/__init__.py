"""AttnRes read for B200: BF16 values, sliced tail keys, sm_100a CUDA kernels.

Drop-in for the public surface of the reference package
(src/attnres/__init__.py:8-15): ``attnres``, ``LearnedQuery``, ``__version__``.
"""

__version__ = "0.1.0"

from .api import attnres
from .modules import LearnedQuery

__all__ = [
    "LearnedQuery",
    "__version__",
    "attnres",
]
