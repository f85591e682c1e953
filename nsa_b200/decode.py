"""Decode step of NSAAttention: one new query token per sequence against that sequence's whole K/V cache.

The reference has no decode entry point (its module assumes len(q) == len(k), nsa/nsa.py:97); this evaluates
the same forward (nsa/nsa.py:94-135) for the single row t = L-1 of every sequence of a packed batch.
"""
import ctypes

import torch

from . import _lib
from .compression_kv import _CompressOne


def compress_cache(module, k, v, cu_seqlens_k):
    """Compressed K/V of a packed cache: k, v [sum L,Hkv,D] -> ck, cv [sum Tc,Hkv,D], cu_c (host list).
    Tc = (L-block)//stride + 1 per sequence, the module's Conv1d rule (nsa/compression_kv.py:298-307)."""
    cu = [int(c) for c in (cu_seqlens_k.tolist() if torch.is_tensor(cu_seqlens_k) else cu_seqlens_k)]
    block, stride = module.compression_block, module.compression_stride
    cu_c = [0]
    for i in range(len(cu) - 1):
        L = cu[i + 1] - cu[i]
        cu_c.append(cu_c[-1] + ((L - block) // stride + 1 if L >= block else 0))
    D = k.shape[-1]
    ws = []
    for conv in (module.compressor.compressor_k, module.compressor.compressor_v):
        ws.append((conv.weight.permute(2, 1, 0).reshape(block * D, D), conv.bias))
    ck = _CompressOne.apply(k, ws[0][0], ws[0][1], cu, cu_c, block, stride)
    cv = _CompressOne.apply(v, ws[1][0], ws[1][1], cu, cu_c, block, stride)
    return ck, cv, cu, cu_c


@torch.no_grad()
def nsa_decode(module, q, k, v, cu_seqlens_k, cache=None):
    """q [nseq,Hq,D] (the newest token of every sequence), k, v [sum L,Hkv,D] packed with cu_seqlens_k.
    Returns o [nseq,Hq,D].  ``cache`` = (ck, cv, cu, cu_c) from ``compress_cache`` skips the re-compression."""
    q = _lib.require(q, "q")
    k = _lib.require(k, "k")
    v = _lib.require(v, "v")
    nseq, Hq, D = q.shape
    Hkv = k.shape[1]
    ck, cv, cu, cu_c = cache if cache is not None else compress_cache(module, k, v, cu_seqlens_k)
    scale = module.softmax_scale
    if scale is None or scale is True:
        scale = 1.0 if scale is True else D ** -0.5
    gates = module.gating(q)
    g_slc, g_swa, g_cmp = (g.contiguous() for g in gates.unbind(-1))
    o, o_cmp, o_slc, o_swa = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty(3, nseq, Hq, dtype=torch.float32, device=q.device)
    n_sel = module.selected_block_count
    idx = torch.empty(nseq, Hkv, n_sel, dtype=torch.int32, device=q.device)
    arr = ctypes.c_int32 * (nseq + 1)
    P = _lib.ptr
    _lib.check(_lib.lib().nsa_decode_fwd(P(q), P(k), P(v), P(ck), P(cv), ctypes.cast(arr(*cu), ctypes.c_void_p),
                                         ctypes.cast(arr(*cu_c), ctypes.c_void_p), P(g_slc), P(g_swa), P(g_cmp), P(o),
                                         P(o_cmp), P(o_slc), P(o_swa), P(lse), P(idx), nseq, Hq, Hkv, D,
                                         module.compression_block, module.compression_stride,
                                         module.selection_block_size, n_sel, module.sliding_window, float(scale),
                                         _lib.stream()), "nsa_decode_fwd")
    return o
