"""Selected-block + sliding-window attention with the reference's API (nsa/selection_attn.py)."""
from typing import Optional, Union

import torch

from . import _lib


class ParallelNSAFunction(torch.autograd.Function):
    """Drop-in for ``ParallelNSAFunction`` (nsa/selection_attn.py:679-737):
    apply(q, k, v, block_indices, block_counts, block_size, window_size, scale, offsets) -> (o_slc, o_swa)."""

    @staticmethod
    def forward(ctx, q, k, v, block_indices, block_counts, block_size, window_size, scale, offsets):
        if offsets is not None:
            raise NotImplementedError("variable-length sequences (cu_seqlens) are not supported by this operator yet")
        q = _lib.require(q, "q")
        k = _lib.require(k, "k")
        v = _lib.require(v, "v")
        B, T, Hq, D = q.shape
        Hkv = k.shape[2]
        if block_indices.dtype not in (torch.int32, torch.int64):
            raise TypeError("block_indices must be int32 or int64")
        idx = block_indices.contiguous()
        S = idx.shape[-1]
        counts = None
        if torch.is_tensor(block_counts):
            counts = block_counts.to(torch.int32).contiguous()
        o_slc = torch.empty_like(q)
        lse_slc = torch.empty(B, T, Hq, dtype=torch.float32, device=q.device)
        o_swa = torch.empty_like(q) if window_size > 0 else None
        lse_swa = torch.empty_like(lse_slc) if window_size > 0 else None
        _lib.check(_lib.lib().nsa_sel_swa_fwd(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(idx), 1 if idx.dtype == torch.int64 else 0, _lib.ptr(counts),
            _lib.ptr(o_slc), _lib.ptr(lse_slc), _lib.ptr(o_swa), _lib.ptr(lse_swa), None, None, None, None, None,
            B, T, Hq, Hkv, D, S, block_size, window_size, float(scale), _lib.stream()), "nsa_sel_swa_fwd")
        ctx.save_for_backward(q, k, v, o_slc, lse_slc, o_swa, lse_swa, idx, counts)
        ctx.meta = (block_size, window_size, float(scale))
        return o_slc, o_swa

    @staticmethod
    def backward(ctx, do_slc, do_swa):
        q, k, v, o_slc, lse_slc, o_swa, lse_swa, idx, counts = ctx.saved_tensors
        block_size, window_size, scale = ctx.meta
        B, T, Hq, D = q.shape
        Hkv, S = k.shape[2], idx.shape[-1]
        L = _lib.lib()
        rows = B * T * Hq

        def delta_of(o, do):
            d = torch.empty(B, T, Hq, dtype=torch.float32, device=q.device)
            _lib.check(L.nsa_rowdot(_lib.ptr(o), _lib.ptr(do), None, _lib.ptr(d), None, rows, D, _lib.stream()),
                       "nsa_rowdot")
            return d

        do_slc = _lib.require(do_slc, "do_slc") if do_slc is not None else torch.zeros_like(q)
        delta_slc = delta_of(o_slc, do_slc)
        delta_swa = None
        if window_size > 0:
            do_swa = _lib.require(do_swa, "do_swa") if do_swa is not None else torch.zeros_like(q)
            delta_swa = delta_of(o_swa, do_swa)
        else:
            do_swa = None
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ws_bytes = L.nsa_sel_swa_bwd_workspace_bytes(B, T, Hkv, S, block_size)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        _lib.check(L.nsa_sel_swa_bwd(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(idx), 1 if idx.dtype == torch.int64 else 0, _lib.ptr(counts),
            _lib.ptr(do_slc), _lib.ptr(lse_slc), _lib.ptr(delta_slc), None,
            _lib.ptr(do_swa), _lib.ptr(lse_swa), _lib.ptr(delta_swa), None,
            _lib.ptr(dq), 0, _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(ws), ws_bytes,
            B, T, Hq, Hkv, D, S, block_size, window_size, scale, _lib.stream()), "nsa_sel_swa_bwd")
        return dq, dk, dv, None, None, None, None, None, None


def parallel_nsa(q: torch.Tensor,
                 k: torch.Tensor,
                 v: torch.Tensor,
                 g_slc: torch.Tensor,
                 g_swa: torch.Tensor,
                 block_indices: torch.LongTensor,
                 block_counts: Optional[Union[torch.LongTensor, int]] = None,
                 block_size: int = 64,
                 window_size: int = 0,
                 scale: Optional[float] = None,
                 cu_seqlens: Optional[torch.LongTensor] = None,
                 head_first: bool = False) -> torch.Tensor:
    """Drop-in for ``parallel_nsa`` (nsa/selection_attn.py:740-814), exported as ``selection_attention``.

    q [B,T,HQ,K]; k,v [B,T,H,K]; g_slc,g_swa [B,T,HQ]; block_indices [B,T,H,S]; block_counts an int, a
    [B,T,H] tensor or None.  Returns o_slc*g_slc (+ o_swa*g_swa when window_size > 0), shape [B,T,HQ,K].
    ``head_first=True`` takes/returns the [B,H,T,...] layouts.
    """
    if scale is None:
        scale = k.shape[-1] ** -0.5
    if cu_seqlens is not None:
        assert q.shape[0] == 1, "batch size must be 1 when cu_seqlens are provided"
    if head_first:
        q, k, v, block_indices = (x.transpose(1, 2) for x in (q, k, v, block_indices))
        g_slc, g_swa = g_slc.transpose(1, 2), g_swa.transpose(1, 2)
        if isinstance(block_counts, torch.Tensor):
            block_counts = block_counts.transpose(1, 2)
    assert q.shape[2] % (k.shape[2] * 16) == 0, "Group size must be a multiple of 16 in NSA"
    if isinstance(block_counts, int):
        block_indices = block_indices[:, :, :, :block_counts]
        block_counts = None
    o_slc, o_swa = ParallelNSAFunction.apply(q, k, v, block_indices, block_counts, block_size, window_size, scale,
                                             cu_seqlens)
    if window_size > 0:
        o = torch.addcmul(o_slc * g_slc.unsqueeze(-1), o_swa, g_swa.unsqueeze(-1))
    else:
        o = o_slc * g_slc.unsqueeze(-1)
    if head_first:
        o = o.transpose(1, 2)
    return o
