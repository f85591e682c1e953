"""Decode step of NSAAttention: one new query token per sequence against that sequence's whole K/V cache.

The reference has no decode entry point (its module assumes len(q) == len(k), nsa/nsa.py:97); this evaluates
the same forward (nsa/nsa.py:94-135) for the single row t = L-1 of every sequence of a packed batch, all sequences
in one kernel launch (nsa_decode_fwd).  The compressed K/V are a cache: ``compress_cache`` builds it once,
``extend_compress_cache`` appends only the compressed positions that new tokens complete.
"""
import torch

from . import _lib
from .compression_kv import _CompressOne


class CompressedCache:
    """Compressed K/V of a packed cache plus the (host and device) length tables the decode kernel needs.

    ck, cv [sum Tc,Hkv,D]; cu, cu_c: host lists [nseq+1] (cumulative lengths of k/v and of ck/cv); the device copies and
    the longest-first launch order are built once here so that a decode step issues no host-to-device copy."""

    def __init__(self, ck, cv, cu, cu_c):
        self.ck, self.cv, self.cu, self.cu_c = ck, cv, list(cu), list(cu_c)
        dev = ck.device
        n = len(self.cu) - 1
        self.cu_dev = torch.tensor(self.cu, dtype=torch.int32, device=dev)
        self.cu_c_dev = torch.tensor(self.cu_c, dtype=torch.int32, device=dev)
        lens = [self.cu[i + 1] - self.cu[i] for i in range(n)]
        self.order_dev = torch.tensor(sorted(range(n), key=lambda i: -lens[i]), dtype=torch.int32, device=dev)
        self.max_tc = max([self.cu_c[i + 1] - self.cu_c[i] for i in range(n)] + [0])

    def workspace(self, nbytes):
        """Scratch of the decode kernels (per-warp partial results), kept with the cache so a step allocates nothing."""
        ws = getattr(self, "_ws", None)
        if ws is None or ws.numel() < nbytes:
            ws = self._ws = torch.empty(nbytes, dtype=torch.uint8, device=self.ck.device)
        return ws

    def __iter__(self):   # (ck, cv, cu, cu_c), the tuple earlier callers unpack
        return iter((self.ck, self.cv, self.cu, self.cu_c))


def _lengths(cu_seqlens_k):
    return [int(c) for c in (cu_seqlens_k.tolist() if torch.is_tensor(cu_seqlens_k) else cu_seqlens_k)]


def _weights(module, D):
    block = module.compression_block
    return [(conv.weight.permute(2, 1, 0).reshape(block * D, D), conv.bias)
            for conv in (module.compressor.compressor_k, module.compressor.compressor_v)]


def compress_cache(module, k, v, cu_seqlens_k):
    """Compressed K/V of a packed cache: k, v [sum L,Hkv,D] -> CompressedCache (ck, cv [sum Tc,Hkv,D]).
    Tc = (L-block)//stride + 1 per sequence, the module's Conv1d rule (nsa/compression_kv.py:298-307)."""
    cu = _lengths(cu_seqlens_k)
    block, stride = module.compression_block, module.compression_stride
    cu_c = [0]
    for i in range(len(cu) - 1):
        L = cu[i + 1] - cu[i]
        cu_c.append(cu_c[-1] + ((L - block) // stride + 1 if L >= block else 0))
    (wk, bk), (wv, bv) = _weights(module, k.shape[-1])
    ck = _CompressOne.apply(k, wk, bk, cu, cu_c, block, stride)
    cv = _CompressOne.apply(v, wv, bv, cu, cu_c, block, stride)
    return CompressedCache(ck, cv, cu, cu_c)


@torch.no_grad()
def extend_compress_cache(module, cache, k, v, cu_seqlens_k):
    """The cache after tokens were appended to the sequences: k, v [sum L',Hkv,D] are the grown packed K/V with lengths
    L' >= L.  Only the compressed positions that the new tokens complete are computed (each is one [block x D] window
    times the Conv1d weight, the same contraction as nsa/compression_kv.py:298-307); the existing entries are copied."""
    cu_new = _lengths(cu_seqlens_k)
    block, stride = module.compression_block, module.compression_stride
    n = len(cu_new) - 1
    if n != len(cache.cu) - 1:
        raise ValueError("the number of sequences changed")
    D, H = k.shape[-1], k.shape[1]
    old_tc = [cache.cu_c[i + 1] - cache.cu_c[i] for i in range(n)]
    cu_c = [0]
    rows = []               # start rows (in the packed k/v) of the windows of the new compressed positions
    for i in range(n):
        L = cu_new[i + 1] - cu_new[i]
        if L < cache.cu[i + 1] - cache.cu[i]:
            raise ValueError("sequence %d became shorter" % i)
        tc = (L - block) // stride + 1 if L >= block else 0
        cu_c.append(cu_c[-1] + tc)
        rows += [cu_new[i] + j * stride for j in range(old_tc[i], tc)]
    ck = torch.empty(cu_c[-1], H, D, dtype=cache.ck.dtype, device=k.device)
    cv = torch.empty_like(ck)
    for i in range(n):      # old entries keep their values
        ck[cu_c[i]:cu_c[i] + old_tc[i]] = cache.ck[cache.cu_c[i]:cache.cu_c[i + 1]]
        cv[cu_c[i]:cu_c[i] + old_tc[i]] = cache.cv[cache.cu_c[i]:cache.cu_c[i + 1]]
    if rows:
        nw = len(rows)
        gather = (torch.tensor(rows, device=k.device).unsqueeze(1) + torch.arange(block, device=k.device)).reshape(-1)
        win_cu = [block * j for j in range(nw + 1)]          # nw windows of exactly one block: one output each
        out_cu = list(range(nw + 1))
        (wk, bk), (wv, bv) = _weights(module, D)
        new_k = _CompressOne.apply(k[gather].contiguous(), wk, bk, win_cu, out_cu, block, stride)
        new_v = _CompressOne.apply(v[gather].contiguous(), wv, bv, win_cu, out_cu, block, stride)
        dst, pos = [], 0
        for i in range(n):
            cnt = (cu_c[i + 1] - cu_c[i]) - old_tc[i]
            dst += list(range(cu_c[i] + old_tc[i], cu_c[i + 1]))
            pos += cnt
        dst = torch.tensor(dst, device=k.device)
        ck[dst] = new_k
        cv[dst] = new_v
    return CompressedCache(ck, cv, cu_new, cu_c)


@torch.no_grad()
def nsa_decode(module, q, k, v, cu_seqlens_k, cache=None, return_parts=False):
    """q [nseq,Hq,D] (the newest token of every sequence), k, v [sum L,Hkv,D] packed with cu_seqlens_k.
    Returns o [nseq,Hq,D].  ``cache`` = a CompressedCache from ``compress_cache`` / ``extend_compress_cache`` skips the
    re-compression.  With ``return_parts`` also returns (o_cmp, o_slc, o_swa, lse [3,nseq,Hq], idx [nseq,Hkv,n])."""
    q = _lib.require(q, "q")
    k = _lib.require(k, "k")
    v = _lib.require(v, "v")
    nseq, Hq, D = q.shape
    Hkv = k.shape[1]
    if cache is None:
        cache = compress_cache(module, k, v, cu_seqlens_k)
    scale = module.softmax_scale
    if scale is None or scale is True:
        scale = 1.0 if scale is True else D ** -0.5
    w_gate = _lib.require(module.gating.weight.detach(), "gating.weight")
    b_gate = _lib.require(module.gating.bias.detach(), "gating.bias") if module.gating.bias is not None else None
    o = torch.empty_like(q)
    n_sel = module.selected_block_count
    idx = torch.empty(nseq, Hkv, n_sel, dtype=torch.int32, device=q.device)
    o_cmp = o_slc = o_swa = lse = None
    if return_parts:
        o_cmp, o_slc, o_swa = (torch.empty_like(q) for _ in range(3))
        lse = torch.empty(3, nseq, Hq, dtype=torch.float32, device=q.device)
    P, L = _lib.ptr, _lib.lib()
    ws_bytes = L.nsa_decode_workspace_bytes(nseq, Hkv)
    ws = cache.workspace(ws_bytes)
    _lib.check(L.nsa_decode_fwd(P(q), P(k), P(v), P(cache.ck), P(cache.cv), P(cache.cu_dev), P(cache.cu_c_dev),
                                         P(cache.order_dev), P(w_gate), P(b_gate), None, None, None, P(o), P(o_cmp), P(o_slc),
                                         P(o_swa), P(lse), P(idx), P(ws), ws_bytes, nseq, k.shape[0], cache.ck.shape[0],
                                         cache.max_tc, Hq, Hkv, D, module.compression_block, module.compression_stride,
                                         module.selection_block_size, n_sel, module.sliding_window, float(scale),
                                         _lib.stream()), "nsa_decode_fwd")
    if return_parts:
        return o, (o_cmp, o_slc, o_swa, lse, idx)
    return o
