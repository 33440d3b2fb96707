"""AttnRes read for B200: BF16 storage, sliced tail keys, hand-written sm_100a kernels.

The importable surface is the reference package's (src/attnres/__init__.py:8-15):
``attnres``, ``LearnedQuery`` and ``__version__``; ``python -m attnres.info`` reports the
state of the CUDA library.  ``attnres.accumulate`` and ``attnres.parallel`` are additions.
"""
from . import api as _api
from . import modules as _modules

# The version of the reference API this package is a drop-in for (tests/test_info.py:16 of the
# reference pins it).
__version__ = "2.0.1"
attnres = _api.attnres
LearnedQuery = _modules.LearnedQuery

__all__ = ["LearnedQuery", "__version__", "attnres"]
