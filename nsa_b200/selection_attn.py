"""Selected-block + sliding-window attention with the reference's API (nsa/selection_attn.py)."""
from typing import Optional, Union

import torch

from . import _lib


def _sequences(offsets, T):
    """[(start, end)] of the packed sequences: one host read of cu_seqlens, or the whole tensor when there are none."""
    if offsets is None:
        return None
    cu = [int(c) for c in (offsets.tolist() if torch.is_tensor(offsets) else offsets)]
    if cu[0] != 0 or cu[-1] != T or any(b <= a for a, b in zip(cu[:-1], cu[1:])):
        raise ValueError("cu_seqlens must start at 0, end at the token count %d and increase: %s" % (T, cu))
    return list(zip(cu[:-1], cu[1:]))


class ParallelNSAFunction(torch.autograd.Function):
    """Drop-in for ``ParallelNSAFunction`` (nsa/selection_attn.py:679-737):
    apply(q, k, v, block_indices, block_counts, block_size, window_size, scale, offsets) -> (o_slc, o_swa).

    With ``offsets`` (= cu_seqlens, batch size 1) the tokens are packed sequences of different lengths; block indices
    and the causal / window masks are relative to each sequence's own start, as in the reference's varlen indexing
    (nsa/selection_attn.py:419-425).  Each sequence is one launch chain on its slice of the packed tensors."""

    @staticmethod
    def forward(ctx, q, k, v, block_indices, block_counts, block_size, window_size, scale, offsets):
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
        seqs = _sequences(offsets, T)
        if seqs is not None and B != 1:
            raise ValueError("batch size must be 1 when cu_seqlens are provided")
        o_slc = torch.empty_like(q)
        lse_slc = torch.empty(B, T, Hq, dtype=torch.float32, device=q.device)
        o_swa = torch.empty_like(q) if window_size > 0 else None
        lse_swa = torch.empty_like(lse_slc) if window_size > 0 else None
        P, i64 = _lib.ptr, 1 if idx.dtype == torch.int64 else 0
        for a, b in (seqs or [(0, T)]):
            sl = slice(a, b)
            fws_bytes = _lib.sel_swa_fwd_workspace_bytes(B, b - a, b - a, Hq, Hkv, D, S, block_size)
            fws = torch.empty(fws_bytes, dtype=torch.uint8, device=q.device) if fws_bytes else None
            _lib.check(_lib.lib().nsa_sel_swa_fwd_ws(
                P(q[:, sl]), P(k[:, sl]), P(v[:, sl]), P(idx[:, sl]), i64, P(counts[:, sl]) if counts is not None else None,
                P(o_slc[:, sl]), P(lse_slc[:, sl]), P(o_swa[:, sl]) if o_swa is not None else None,
                P(lse_swa[:, sl]) if lse_swa is not None else None, None, None, None, None, None, P(fws), fws_bytes,
                B, b - a, Hq, Hkv, D, S, block_size, window_size, float(scale), b - a, 0, _lib.stream()), "nsa_sel_swa_fwd")
        ctx.save_for_backward(q, k, v, o_slc, lse_slc, o_swa, lse_swa, idx, counts)
        ctx.meta = (block_size, window_size, float(scale), seqs)
        return o_slc, o_swa

    @staticmethod
    def backward(ctx, do_slc, do_swa):
        q, k, v, o_slc, lse_slc, o_swa, lse_swa, idx, counts = ctx.saved_tensors
        block_size, window_size, scale, seqs = ctx.meta
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
        P, i64 = _lib.ptr, 1 if idx.dtype == torch.int64 else 0
        opt = lambda t, sl: P(t[:, sl]) if t is not None else None
        for a, b in (seqs or [(0, T)]):
            sl = slice(a, b)
            ws_bytes = _lib.sel_swa_bwd_workspace_bytes(B, b - a, b - a, Hq, Hkv, D, S, block_size)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
            _lib.check(L.nsa_sel_swa_bwd(
                P(q[:, sl]), P(k[:, sl]), P(v[:, sl]), P(idx[:, sl]), i64, opt(counts, sl),
                P(do_slc[:, sl]), P(lse_slc[:, sl]), P(delta_slc[:, sl]), None,
                opt(do_swa, sl), opt(lse_swa, sl), opt(delta_swa, sl), None,
                P(dq[:, sl]), 0, P(dk[:, sl]), P(dv[:, sl]), P(ws), ws_bytes,
                B, b - a, Hq, Hkv, D, S, block_size, window_size, scale, _lib.stream()), "nsa_sel_swa_bwd")
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
