"""Compressed attention + block selection with the reference's API (nsa/triton_attention.py).

The module keeps the reference's file name so ``from nsa.triton_attention import flash_attn_func`` still
resolves, although nothing here is Triton: ``_attention`` launches ``nsa_cmp_attn_fwd`` / ``nsa_cmp_attn_bwd``.
"""
import math

import torch

from . import _lib


class _attention(torch.autograd.Function):
    """Drop-in for ``_attention`` (nsa/triton_attention.py:419-546).

    forward(q, k, v, block_stride, block_size, causal, sm_scale, pool_num_kv_head, pool_kernel_size,
            pool_stride, pool_padding, select_block_count) -> (o, indices)
    q [B,T,Hq,D]; k,v = compressed keys/values [B,Tc,Hk,D].  Hk may be the number of KV heads (compact
    form: every group of Hq/Hk query heads shares one compressed head) or Hq with each group's heads
    holding identical copies (the reference's repeated form, checked).  indices [B,T,Hkv,n] int64 are the
    top-n pooled blocks of softmax(q.k^T) summed per KV group; no gradient flows through them
    (nsa/triton_attention.py:545).
    """

    @staticmethod
    def forward(ctx, q, k, v, block_stride, block_size, causal, sm_scale, pool_num_kv_head=0, pool_kernel_size=0,
                pool_stride=0, pool_padding=0, select_block_count=0):
        q = _lib.require(q, "q")
        k = _lib.require(k, "k")
        v = _lib.require(v, "v")
        B, T, Hq, D = q.shape
        Tc, Hk = k.shape[1], k.shape[2]
        if k.shape != v.shape or k.shape[0] != B or k.shape[3] != D:
            raise ValueError("k and v must both be [B, Tc, Hk, D]")
        if sm_scale is None:
            sm_scale = 1.0 / math.sqrt(D)
        repeated = 1
        if pool_num_kv_head and Hk == Hq and Hq // pool_num_kv_head > 1:
            # the reference passes K/V repeated to Hq heads (nsa/compression_kv.py:308-310)
            G = Hq // pool_num_kv_head
            kg, vg = k.view(B, Tc, pool_num_kv_head, G, D), v.view(B, Tc, pool_num_kv_head, G, D)
            if not (torch.equal(kg, kg[:, :, :, :1].expand_as(kg)) and torch.equal(vg, vg[:, :, :, :1].expand_as(vg))):
                raise NotImplementedError(
                    "compressed K/V with Hq distinct heads: only group-shared compressed heads are supported")
            k, v = kg[:, :, :, 0].contiguous(), vg[:, :, :, 0].contiguous()
            Hk, repeated = pool_num_kv_head, G
        n_sel = int(select_block_count) if pool_num_kv_head else 0
        L = _lib.lib()
        o = torch.empty_like(q)
        lse = torch.empty(B, T, Hq, dtype=torch.float32, device=q.device)
        idx = None
        if n_sel > 0:
            if pool_num_kv_head != Hk:
                raise ValueError("pool_num_kv_head must equal the number of compressed KV heads")
            n_pool = L.nsa_pool_out_len(Tc, pool_kernel_size, pool_stride, pool_padding)
            if n_sel > n_pool:
                raise RuntimeError("selected index k out of range: %d blocks requested, %d exist" % (n_sel, n_pool))
            idx = torch.empty(B, T, Hq // 16, n_sel, dtype=torch.int32, device=q.device)
        _lib.check(L.nsa_cmp_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(idx),
                                      None, B, T, Tc, Hq, Hk, D, block_size, block_stride, 1 if causal else 0,
                                      float(sm_scale), n_sel, pool_kernel_size, pool_stride, pool_padding,
                                      _lib.stream()), "nsa_cmp_attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (float(sm_scale), bool(causal), block_stride, block_size, repeated)
        indices = idx.long() if idx is not None else None
        if indices is not None:
            ctx.mark_non_differentiable(indices)
        return o, indices

    @staticmethod
    def backward(ctx, do, dind):
        q, k, v, o, lse = ctx.saved_tensors
        sm_scale, causal, block_stride, block_size, repeated = ctx.meta
        do = _lib.require(do, "do")
        B, T, Hq, D = q.shape
        Tc, Hk = k.shape[1], k.shape[2]
        L = _lib.lib()
        delta = torch.empty(B, T, Hq, dtype=torch.float32, device=q.device)
        _lib.check(L.nsa_rowdot(_lib.ptr(o), _lib.ptr(do), None, _lib.ptr(delta), None, B * T * Hq, D, _lib.stream()),
                   "nsa_rowdot")
        dq = torch.empty_like(q)
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        ws_bytes = L.nsa_cmp_attn_bwd_workspace_bytes(B, T, Tc, Hk, D)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        _lib.check(L.nsa_cmp_attn_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(lse), _lib.ptr(do), _lib.ptr(delta),
                                      None, _lib.ptr(dq), 0, _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(ws), ws_bytes, B, T, Tc,
                                      Hq, Hk, D, block_size, block_stride, 1 if causal else 0, sm_scale, _lib.stream()),
                   "nsa_cmp_attn_bwd")
        if repeated > 1:
            # callers that passed repeated heads sum these copies again in the repeat's backward
            dk = (dk / repeated).repeat_interleave(repeated, dim=2)
            dv = (dv / repeated).repeat_interleave(repeated, dim=2)
        return dq, dk, dv, None, None, None, None, None, None, None, None, None


flash_attn_func = _attention.apply
