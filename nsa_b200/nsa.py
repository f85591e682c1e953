"""The NSAAttention module with the reference's constructor, parameters and forward signature
(nsa/nsa.py:15-135)."""
import torch
from torch import nn

from . import _lib
from .compression_kv import KVCompressor


class _NSACore(torch.autograd.Function):
    """Everything of NSAAttention.forward between the compression and the output, as one autograd node:
    compressed attention + block selection, selected + sliding-window attention and the gated three-way sum
    (nsa/nsa.py:102-133).  Keeping the three branches in one node lets the backward feed dO and the gates straight
    to the kernels (no g*dO tensors are materialised, dQ is accumulated inside the kernels instead of by autograd)."""

    @staticmethod
    def forward(ctx, q, k, v, ck, cv, w_gate, b_gate, cfg):
        """q: [B,Tq,Hq,D] = the queries at sequence positions q0 .. q0+Tq-1; k, v: [B,T,Hkv,D] and ck, cv:
        [B,Tc,Hkv,D] cover the whole sequence; w_gate [3,D], b_gate [3]: the gate projection (rows: selected,
        window, compressed; nsa/nsa.py:59,117).  cfg[10] = q0 (0 and Tq == T for an unsharded call); an optional
        cfg[11] = True folds the gate projection and the backward's row pre-pass into the attention kernels (fewer
        launches; slower than the streaming kernels at large shapes, see NSAAttention.fuse_row_passes)."""
        (stride, block, causal, scale, pool_k, pool_s, pool_p, n_sel, sel_block, window, q0) = cfg[:11]
        fused = len(cfg) > 11 and bool(cfg[11])
        score_mode = int(cfg[12]) if len(cfg) > 12 else 0
        q, k, v, ck, cv = (_lib.require(t, n) for t, n in ((q, "q"), (k, "k"), (v, "v"), (ck, "ck"), (cv, "cv")))
        w_gate = _lib.require(w_gate, "gating.weight")
        b_gate = _lib.require(b_gate, "gating.bias") if b_gate is not None else None
        B, Tq, Hq, D = q.shape
        T, Hkv, Tc = k.shape[1], k.shape[2], ck.shape[1]
        L, P, S = _lib.lib(), _lib.ptr, _lib.stream
        dev = q.device
        g_slc, g_swa, g_cmp = (torch.empty(B, Tq, Hq, dtype=q.dtype, device=dev) for _ in range(3))
        n_pool = L.nsa_pool_out_len(Tc, pool_k, pool_s, pool_p)
        if n_sel > n_pool:
            raise RuntimeError("selected index k out of range: %d blocks requested, %d exist" % (n_sel, n_pool))
        o_cmp, o_slc, o = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        o_swa = torch.empty_like(q) if window > 0 else None
        lse_cmp, lse_slc = (torch.empty(B, Tq, Hq, dtype=torch.float32, device=dev) for _ in range(2))
        lse_swa = torch.empty_like(lse_slc) if window > 0 else None
        idx = torch.empty(B, Tq, Hkv, n_sel, dtype=torch.int32, device=dev)
        if fused:
            # compressed attention + block selection; the gate projection rides on the resident query tiles
            _lib.check(L.nsa_cmp_attn_fwd_gated(P(q), P(ck), P(cv), P(o_cmp), P(lse_cmp), P(idx), None, P(w_gate),
                                                P(b_gate), P(g_slc), P(g_swa), P(g_cmp), B, T, Tc, Hq, Hkv, D, block, stride,
                                                1 if causal else 0, scale, n_sel, pool_k, pool_s, pool_p, score_mode, Tq,
                                                q0, S()), "nsa_cmp_attn_fwd_gated")
        else:
            _lib.check(L.nsa_gate_fwd(P(q), P(w_gate), P(b_gate), P(g_slc), P(g_swa), P(g_cmp), B * Tq * Hq, D, S()),
                       "nsa_gate_fwd")
            _lib.check(L.nsa_cmp_attn_fwd_gated(P(q), P(ck), P(cv), P(o_cmp), P(lse_cmp), P(idx), None, None, None, None,
                                                None, None, B, T, Tc, Hq, Hkv, D, block, stride, 1 if causal else 0, scale,
                                                n_sel, pool_k, pool_s, pool_p, score_mode, Tq, q0, S()), "nsa_cmp_attn_fwd")
        fws_bytes = _lib.sel_swa_fwd_workspace_bytes(B, T, Tq, Hq, Hkv, D, n_sel, sel_block)
        fws = torch.empty(fws_bytes, dtype=torch.uint8, device=dev) if fws_bytes else None
        _lib.check(L.nsa_sel_swa_fwd_ws(P(q), P(k), P(v), P(idx), 0, None, P(o_slc), P(lse_slc), P(o_swa),
                                        P(lse_swa), P(g_slc), P(g_swa), P(o_cmp), P(g_cmp), P(o), P(fws), fws_bytes, B, T,
                                        Hq, Hkv, D, n_sel, sel_block, window, scale, Tq, q0, S()), "nsa_sel_swa_fwd")
        ctx.save_for_backward(q, k, v, ck, cv, g_slc, g_swa, g_cmp, o_slc, o_swa, o_cmp, lse_slc, lse_swa, lse_cmp, idx,
                              w_gate)
        ctx.cfg = cfg
        ctx.has_bias = b_gate is not None
        return o

    @staticmethod
    def backward(ctx, do):
        (q, k, v, ck, cv, g_slc, g_swa, g_cmp, o_slc, o_swa, o_cmp, lse_slc, lse_swa, lse_cmp, idx,
         w_gate) = ctx.saved_tensors
        (stride, block, causal, scale, pool_k, pool_s, pool_p, n_sel, sel_block, window, q0) = ctx.cfg[:11]
        fused = len(ctx.cfg) > 11 and bool(ctx.cfg[11])
        do = _lib.require(do, "do")
        B, Tq, Hq, D = q.shape
        T, Hkv, Tc = k.shape[1], k.shape[2], ck.shape[1]
        L, P, S = _lib.lib(), _lib.ptr, _lib.stream
        dev = q.device
        rows = B * Tq * Hq

        delta_slc, delta_cmp = (torch.empty(B, Tq, Hq, dtype=torch.float32, device=dev) for _ in range(2))
        delta_swa = torch.empty_like(delta_slc) if window > 0 else None
        dg_slc, dg_swa, dg_cmp = (torch.empty_like(g_slc) for _ in range(3))
        if window <= 0:
            dg_swa.zero_()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dck, dcv = torch.empty_like(ck), torch.empty_like(cv)
        ws_bytes = _lib.sel_swa_bwd_workspace_bytes(B, T, Tq, Hq, Hkv, D, n_sel, sel_block)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        ws2_bytes = L.nsa_cmp_attn_bwd_workspace_bytes(B, T, Tc, Hkv, D)
        ws2 = torch.empty(ws2_bytes, dtype=torch.uint8, device=dev)
        if fused:
            # delta = g * rowsum(o * dO) and the gate gradients rowsum(o * dO) are formed inside the dQ kernels while the
            # dO tile is resident (no separate pass over o_slc, o_swa, o_cmp and dO)
            _lib.check(L.nsa_sel_swa_bwd_fused(P(q), P(k), P(v), P(idx), 0, None, P(o_slc), P(o_swa), P(do), P(lse_slc),
                                               P(delta_slc), P(g_slc), P(dg_slc), P(lse_swa), P(delta_swa), P(g_swa),
                                               P(dg_swa) if window > 0 else None, P(dq), 0, P(dk), P(dv), P(ws), ws_bytes,
                                               B, T, Hq, Hkv, D, n_sel, sel_block, window, scale, Tq, q0, S()),
                       "nsa_sel_swa_bwd_fused")
            _lib.check(L.nsa_cmp_attn_bwd_fused(P(q), P(ck), P(cv), P(o_cmp), P(lse_cmp), P(do), P(delta_cmp), P(g_cmp),
                                                P(dg_cmp), P(dq), 1, P(dck), P(dcv), P(ws2), ws2_bytes, B, T, Tc, Hq, Hkv, D,
                                                block, stride, 1 if causal else 0, scale, Tq, q0, S()),
                       "nsa_cmp_attn_bwd_fused")
        else:
            # one streaming pass over dO: delta = g * rowsum(o * dO) and the gate gradients of all three branches
            _lib.check(L.nsa_rowdot3(P(o_slc), P(o_swa), P(o_cmp), P(do), P(g_slc), P(g_swa), P(g_cmp), P(delta_slc),
                                     P(delta_swa), P(delta_cmp), P(dg_slc), P(dg_swa), P(dg_cmp), rows, D, S()),
                       "nsa_rowdot3")
            _lib.check(L.nsa_sel_swa_bwd_sharded(P(q), P(k), P(v), P(idx), 0, None, P(do), P(lse_slc), P(delta_slc),
                                                 P(g_slc), P(do) if window > 0 else None, P(lse_swa), P(delta_swa), P(g_swa),
                                                 P(dq), 0, P(dk), P(dv), P(ws), ws_bytes, B, T, Hq, Hkv, D, n_sel, sel_block,
                                                 window, scale, Tq, q0, S()), "nsa_sel_swa_bwd")
            _lib.check(L.nsa_cmp_attn_bwd_sharded(P(q), P(ck), P(cv), P(lse_cmp), P(do), P(delta_cmp), P(g_cmp), P(dq), 1,
                                                  P(dck), P(dcv), P(ws2), ws2_bytes, B, T, Tc, Hq, Hkv, D, block, stride,
                                                  1 if causal else 0, scale, Tq, q0, S()), "nsa_cmp_attn_bwd")
        # gate projection backward: dq += dg . W in place (dq is complete here), dW and db by fixed-order reduction
        dw = torch.empty_like(w_gate)
        db = torch.empty(3, dtype=w_gate.dtype, device=dev) if ctx.has_bias else None
        ws_bytes = L.nsa_gate_bwd_workspace_bytes(rows, D)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        _lib.check(L.nsa_gate_bwd(P(q), P(dg_slc), P(dg_swa), P(dg_cmp), P(w_gate), P(dq), P(dw), P(db), P(ws), ws_bytes,
                                  rows, D, S()), "nsa_gate_bwd")
        return dq, dk, dv, dck, dcv, dw, db, None


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
        # Not a constructor argument (the signature stays the reference's).  True folds the gate projection into the
        # compressed-attention kernel and the backward's row pre-pass into the dQ kernels: three launches fewer per step,
        # which pays for small, launch-bound shapes; at the benchmark's shape the separate streaming kernels are faster
        # (they read rows fully coalesced; a thread-per-row epilogue does not), so the default is False.
        self.fuse_row_passes = False
        # Selection scores (also not a constructor argument).  "reference": what the reference's scoring does -- the
        # soft-max of the unscaled, unmasked q.ck over all compressed keys (nsa/torch_attention.py:121-125), so blocks in
        # a query's future can be selected and are then skipped.  "causal": the compressed branch's own attention
        # probabilities (scaled, causally masked), as in the NSA paper: every selected block is visible.
        self.score_mode = "reference"

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
        if bs > 1 and (max_seqlen is None or bs * int(max_seqlen) != num_token):
            # Sequences of different lengths (the reference's reshape at nsa/nsa.py:97 cannot take them): every sequence
            # is one equal-length call on its slice of the packed tensors.  Costs one host read of cu_seqlens.
            cu = [int(c) for c in cu_seqlens_k.tolist()]
            if any(b - a != cu[1] - cu[0] for a, b in zip(cu[:-1], cu[1:])):
                outs = []
                for a, b in zip(cu[:-1], cu[1:]):
                    one = torch.tensor([0, b - a], dtype=torch.int32, device=q.device)
                    outs.append(self.forward(q[a:b], k[a:b], v[a:b], one, b - a, None, None, causal))
                return torch.cat(outs, 0)
        scale = self.softmax_scale
        if scale is None or scale is True:
            # the reference's own callers pass `True` here positionally (tests/test_nsa_module.py:25), which its
            # kernels read as 1.0; None selects D^-0.5 in both attention entry points
            scale = 1.0 if scale is True else head_qk_dim ** -0.5
        q4 = q.reshape(bs, -1, num_q_head, head_qk_dim)

        # compressed keys/values stay in the compact [B,Tc,Hkv,D] form (no repeat to Hq heads)
        ck, cv, _ = self.compressor(k, v, cu_seqlens_k, None)
        k4 = k.reshape(bs, -1, num_kv_head, head_qk_dim)
        v4 = v.reshape(bs, -1, num_kv_head, head_v_dim)
        cfg = (self.compression_stride, self.compression_block, bool(causal), float(scale), self.pool_kernel_size,
               self.pool_stride, self.pool_padding, self.selected_block_count, self.selection_block_size,
               self.sliding_window, 0, self.fuse_row_passes, {"reference": 0, "causal": 1}[self.score_mode])
        # the gate projection (nn.Linear(head_dim, 3), no activation) runs inside the fused node
        o = _NSACore.apply(q4, k4, v4, ck, cv, self.gating.weight, self.gating.bias, cfg)
        return o.reshape(-1, *o.shape[-2:])
