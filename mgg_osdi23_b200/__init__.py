"""B200-native implementation of MGG's multi-GPU neighbor-aggregation path.

``api``      the reference's operator surface (split_CSR, build_part, mgg_SAG_np_div, ...)
``drivers``  the 2-layer GCN / 5-layer GIN / single-aggregation orchestration of the reference's
             ``main()`` functions
``symmem``   symmetric buffers (peer-readable embedding shards)
``graphgen`` seeded synthetic graphs of the benchmark shapes
``graphio``  the reference's binary CSR files

Importing the package loads ``libmggb200.so``; it raises if the library has not been built.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from .api import *  # noqa: F401,F403
from ._lib import MggbError  # noqa: F401

__version__ = "0.1.0"
