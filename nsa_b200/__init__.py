"""nsa_b200: Native Sparse Attention on B200 (sm_100a) behind the Python API of the `nsa` package.

`import nsa_b200 as nsa` gives the same surface as the reference package: ``nsa.selection_attention``
(nsa/__init__.py:1), ``nsa.nsa.NSAAttention``, ``nsa.compression_kv``, ``nsa.triton_attention`` and
``nsa.selection_attn``.  All compute runs in hand-written CUDA kernels reached through the C ABI of
``include/nsa_b200.h``; there is no Triton, no backend dispatch and no CPU fallback.
"""
from .selection_attn import parallel_nsa as selection_attention  # noqa: F401
from . import compression_kv, selection_attn, triton_attention  # noqa: F401
from . import nsa  # noqa: F401
from .nsa import NSAAttention  # noqa: F401
