"""The NSAAttention module with the reference's constructor, parameters and forward signature
(nsa/nsa.py:15-135)."""
import torch
from torch import nn

from . import _lib
from .compression_kv import KVCompressor
from .selection_attn import ParallelNSAFunction
from .triton_attention import _attention


class _GatedCombine(torch.autograd.Function):
    """o = g_slc*o_slc + g_swa*o_swa + g_cmp*o_cmp in one pass (the mul + two addcmul of
    nsa/selection_attn.py:808-811 and nsa/nsa.py:133).  Gates [B,T,Hq], tensors [B,T,Hq,D]."""

    @staticmethod
    def forward(ctx, o_slc, g_slc, o_swa, g_swa, o_cmp, g_cmp):
        ts = [_lib.require(t, "combine operand") for t in (o_slc, g_slc, o_swa, g_swa, o_cmp, g_cmp)]
        o = torch.empty_like(ts[0])
        rows, D = o.numel() // o.shape[-1], o.shape[-1]
        _lib.check(_lib.lib().nsa_combine(*[_lib.ptr(t) for t in ts], _lib.ptr(o), rows, D, _lib.stream()), "nsa_combine")
        ctx.save_for_backward(*ts)
        return o

    @staticmethod
    def backward(ctx, do):
        o_slc, g_slc, o_swa, g_swa, o_cmp, g_cmp = ctx.saved_tensors
        do = _lib.require(do, "do")
        L = _lib.lib()
        rows, D = do.numel() // do.shape[-1], do.shape[-1]
        grads = []
        for o_x, g_x in ((o_slc, g_slc), (o_swa, g_swa), (o_cmp, g_cmp)):
            d_o = torch.empty_like(do)
            _lib.check(L.nsa_combine(_lib.ptr(do), _lib.ptr(g_x), None, None, None, None, _lib.ptr(d_o), rows, D,
                                     _lib.stream()), "nsa_combine")
            d_g = torch.empty_like(g_x)
            _lib.check(L.nsa_rowdot(_lib.ptr(o_x), _lib.ptr(do), None, None, _lib.ptr(d_g), rows, D, _lib.stream()),
                       "nsa_rowdot")
            grads += [d_o, d_g]
        return tuple(grads)


class NSAAttention(nn.Module):
    """Drop-in for ``nsa.nsa.NSAAttention``.

    Same constructor arguments and defaults, same sub-modules and parameter names (``compressor`` holding
    ``compressor_k`` / ``compressor_v`` Conv1d parameter sets, ``gating`` = Linear(head_dim, 3)), so a
    reference ``state_dict`` loads unchanged.  ``forward`` takes packed q [B*T,Hq,D], k,v [B*T,Hkv,D] and
    ``cu_seqlens`` of equal-length sequences (as the reference's reshape at nsa/nsa.py:97 assumes) and returns
    [B*T,Hq,D].  Gates are the raw linear outputs (no activation), as in the reference.
    """

    def __init__(
        self,
        head_dim: int,
        causal=False,
        softmax_scale=None,
        attention_dropout=0.0,
        deterministic=False,
        compression_stride=16,
        compression_block=32,
        selection_block=64,
        selected_block_count=16,
        sliding_window=512,
        device=None,
        dtype=None,
    ):
        super().__init__()
        if attention_dropout not in (0, 0.0, None):
            raise NotImplementedError("attention dropout is not part of the NSA path (the reference never applies it)")
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.drop_p = attention_dropout
        self.deterministic = deterministic
        self.sliding_window = sliding_window
        self.selected_block_count = selected_block_count
        self.selection_block_size = selection_block
        self.compression_stride = compression_stride
        self.compression_block = compression_block
        self.compressor = KVCompressor(compression_stride, compression_block, head_dim, device, dtype)
        self.pool_kernel_size = selection_block // compression_stride + 1
        self.pool_padding = compression_block // compression_stride - 2
        self.pool_stride = selection_block // compression_stride
        self.gating = nn.Linear(head_dim, 3, device=device, dtype=dtype)

    def forward(
        self,
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        cu_seqlens: torch.Tensor,
        max_seqlen=None,
        cu_seqlens_k: torch.Tensor = None,
        max_seqlen_k=None,
        causal: bool = None,
    ) -> torch.Tensor:
        causal = self.causal if causal is None else causal
        cu_seqlens_k = cu_seqlens if cu_seqlens_k is None else cu_seqlens_k
        bs = cu_seqlens_k.numel() - 1
        num_q_head, head_qk_dim = q.shape[1:]
        num_token, num_kv_head, head_v_dim = v.shape
        scale = self.softmax_scale
        if scale is None or scale is True:
            # the reference's own callers pass `True` here positionally (tests/test_nsa_module.py:25), which its
            # kernels read as 1.0; None selects D^-0.5 in both attention entry points
            scale = 1.0 if scale is True else head_qk_dim ** -0.5
        q4 = q.reshape(bs, -1, num_q_head, head_qk_dim)

        # compressed keys/values stay in the compact [B,Tc,Hkv,D] form (no repeat to Hq heads)
        ck, cv, _ = self.compressor(k, v, cu_seqlens_k, None)
        cmp_o, indices = _attention.apply(q4, ck, cv, self.compression_stride, self.compression_block, bool(causal),
                                          scale, num_kv_head, self.pool_kernel_size, self.pool_stride,
                                          self.pool_padding, self.selected_block_count)

        gating_score = self.gating(q4)                         # [B,T,Hq,3], no activation
        g_slc, g_swa, g_cmp = (g.contiguous() for g in gating_score.unbind(-1))
        k4 = k.reshape(bs, -1, num_kv_head, head_qk_dim)
        v4 = v.reshape(bs, -1, num_kv_head, head_v_dim)
        o_slc, o_swa = ParallelNSAFunction.apply(q4, k4, v4, indices, None, self.selection_block_size,
                                                 self.sliding_window, scale, None)
        if o_swa is None:
            o = o_slc * g_slc.unsqueeze(-1) + cmp_o * g_cmp.unsqueeze(-1)
        else:
            o = _GatedCombine.apply(o_slc, g_slc, o_swa, g_swa, cmp_o, g_cmp)
        return o.reshape(-1, *o.shape[-2:])
