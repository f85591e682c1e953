"""CPU oracle for the Native Sparse Attention path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 torch on the CPU, the algorithm of the
reference's naive torch paths.  It is the checker the CUDA kernels are compared
against; nothing in the shipped package imports it.  Only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may call it.

Parity pinning: every function below is checked in ``tests/test_oracle_golden.py``
against fixtures under ``tests/golden/`` that were produced by running the
reference's own functions (``nsa/torch_attention.py`` ``attention_ref`` /
``get_indices``, ``tests/test_parallel_nsa.py`` ``naive_nsa``,
``tests/test_compression_kv_bwd.py`` ``compute_reference_kv`` and the
``nn.Conv1d`` composition of ``nsa/compression_kv.py`` ``KVCompressor``) on
seeded inputs; the generating script is ``tests/golden/make_golden.py``.

Each function cites the reference lines it follows (paths relative to the
reference project root).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

# --------------------------------------------------------------------------
# compression
# --------------------------------------------------------------------------


def compressed_len_conv(T: int, block: int, stride: int) -> int:
    """Conv1d output length used by the module path: nsa/compression_kv.py:298-307."""
    return (T - block) // stride + 1 if T >= block else 0


def compressed_len_varlen(T: int, block: int, stride: int) -> int:
    """``calc_compressed_len`` of the functional path: nsa/compression_kv.py:9-10."""
    return max((T - block) // stride, 0)


def _windows(x: torch.Tensor, n_out: int, block: int, stride: int) -> torch.Tensor:
    """x [T,H,D] -> [n_out,H,block*D]: window i is rows stride*i .. stride*i+block-1, flattened
    (row-major over (in-block offset, channel)), as tests/test_compression_kv_bwd.py:40-52."""
    T, H, D = x.shape
    idx = (torch.arange(n_out).unsqueeze(1) * stride + torch.arange(block).unsqueeze(0))  # [n,block]
    w = x[idx.reshape(-1)].reshape(n_out, block, H, D).permute(0, 2, 1, 3)
    return w.reshape(n_out, H, block * D)


def compress_varlen(x: torch.Tensor, w: torch.Tensor, cu_seq_len, block: int, stride: int):
    """Functional-path compression.  x [tok,H,D]; w [block*D, D] (row j*D+c multiplies channel
    c of in-block offset j); no bias; per-sequence output length (L-block)//stride.
    Follows tests/test_compression_kv_bwd.py:28-59 (the reference's own loop oracle for
    nsa/compression_kv.py:21-57,178-217).  Returns (y [sum_out,H,D] fp32, cu_out list)."""
    cu = [int(c) for c in cu_seq_len]
    outs, cu_out = [], [0]
    for s in range(len(cu) - 1):
        xs = x[cu[s]:cu[s + 1]].float()
        n = compressed_len_varlen(xs.shape[0], block, stride)
        cu_out.append(cu_out[-1] + n)
        if n > 0:
            outs.append(_windows(xs, n, block, stride) @ w.float())
    y = torch.cat(outs, 0) if outs else x.new_zeros((0,) + tuple(x.shape[1:]), dtype=torch.float32)
    return y, cu_out


def compress_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                  block: int, stride: int) -> torch.Tensor:
    """Module-path compression (nn.Conv1d(D, D, block, stride) over the token axis per
    (batch, head)): nsa/compression_kv.py:298-307.  x [B,T,H,D]; weight [D_out, D_in, block];
    returns [B,Tc,H,D] fp32 with Tc=(T-block)//stride+1."""
    B, T, H, D = x.shape
    n = compressed_len_conv(T, block, stride)
    # conv weight W[o,c,j]  ->  matrix rows (j*D + c), columns o
    wm = weight.float().permute(2, 1, 0).reshape(block * D, D)
    ys = []
    for b in range(B):
        y = _windows(x[b].float(), n, block, stride) @ wm
        if bias is not None:
            y = y + bias.float()
        ys.append(y)
    return torch.stack(ys, 0)


# --------------------------------------------------------------------------
# compressed attention + block selection
# --------------------------------------------------------------------------


def pool_out_len(n: int, kernel: int, stride: int, pad: int) -> int:
    """Output length of avg_pool1d(..., ceil_mode=True) as torch computes it."""
    out = -(-(n + 2 * pad - kernel) // stride) + 1
    if (out - 1) * stride >= n + pad:
        out -= 1
    return out


def pooled_scores(q: torch.Tensor, ck: torch.Tensor, n_kv_head: int, kernel: int, stride: int,
                  pad: int) -> torch.Tensor:
    """Importance scores: softmax over ALL compressed positions of the UNSCALED, UNMASKED q.ck,
    summed over the query heads of each KV group, then average-pooled (ceil mode, pads counted
    in the divisor, the overhang of the last window not counted).
    nsa/torch_attention.py:121-125 (scores) and :51-62 (get_indices).
    q [B,T,Hq,D], ck [B,Tc,Hk,D] with Hk == Hq or Hk dividing Hq.  Returns [B,Hkv,T,NB] fp32."""
    B, T, Hq, D = q.shape
    Tc, Hk = ck.shape[1], ck.shape[2]
    ckr = ck.float().repeat_interleave(Hq // Hk, dim=2) if Hk != Hq else ck.float()
    qk = torch.einsum("bthd,bshd->bhts", q.float(), ckr)
    p = torch.softmax(qk, dim=-1)                                    # [B,Hq,T,Tc]
    p = p.reshape(B, n_kv_head, Hq // n_kv_head, T, Tc).sum(2)       # [B,Hkv,T,Tc]
    nb = pool_out_len(Tc, kernel, stride, pad)
    out = p.new_zeros(B, n_kv_head, T, nb)
    for blk in range(nb):
        lo = blk * stride - pad
        hi = min(lo + kernel, Tc + pad)
        div = hi - lo
        a, z = max(lo, 0), min(hi, Tc)
        out[..., blk] = p[..., a:z].sum(-1) / div
    return out


def pooled_scores_causal(q: torch.Tensor, ck: torch.Tensor, n_kv_head: int, kernel: int, stride: int, pad: int,
                         cstride: int, cblock: int, scale: Optional[float] = None) -> torch.Tensor:
    """Causal variant of the importance scores (no counterpart in the reference; the NSA paper's definition): the
    compressed branch's own attention probabilities -- softmax of the SCALED scores over the compressed positions
    visible to the query (t >= j*cstride + cblock; rows that see nothing score 0) -- summed over the query heads of
    each KV group and pooled exactly as ``pooled_scores`` does.  Returns [B,Hkv,T,NB] fp32."""
    B, T, Hq, D = q.shape
    Tc, Hk = ck.shape[1], ck.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    ckr = ck.float().repeat_interleave(Hq // Hk, dim=2) if Hk != Hq else ck.float()
    s = torch.einsum("bthd,bshd->bhts", q.float(), ckr) * scale
    masked = torch.arange(Tc).unsqueeze(0) * cstride + cblock > torch.arange(T).unsqueeze(1)
    s = s.masked_fill(masked, float("-inf"))
    ev = masked.all(-1).view(1, 1, T, 1)
    p = torch.softmax(s.masked_fill(ev, 0.0), dim=-1).masked_fill(ev, 0.0).masked_fill(masked, 0.0)
    p = p.reshape(B, n_kv_head, Hq // n_kv_head, T, Tc).sum(2)
    nb = pool_out_len(Tc, kernel, stride, pad)
    out = p.new_zeros(B, n_kv_head, T, nb)
    for blk in range(nb):
        lo = blk * stride - pad
        hi = min(lo + kernel, Tc + pad)
        out[..., blk] = p[..., max(lo, 0):min(hi, Tc)].sum(-1) / (hi - lo)
    return out


def topn_blocks(scores: torch.Tensor, n: int) -> torch.Tensor:
    """[B,Hkv,T,NB] -> [B,T,Hkv,n] int64; largest first, ties broken by the lower block index.
    (torch.topk at nsa/torch_attention.py:60 leaves the tie order unspecified; comparisons in
    the tests are on index sets with a score-gap waiver.)"""
    nb = scores.shape[-1]
    order = torch.argsort(-scores, dim=-1, stable=True)[..., :n]
    return order.transpose(1, 2).contiguous()


def cmp_attention(q: torch.Tensor, ck: torch.Tensor, cv: torch.Tensor, stride: int, block: int,
                  causal: bool = True, scale: Optional[float] = None, q_pos=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Compressed attention.  o = softmax(scale * q.ck^T + mask) . cv, where with ``causal`` the
    compressed position j is visible to query t iff t >= j*stride + block; rows with no visible
    position give 0.  nsa/torch_attention.py:66-163 with the mask of :42-43.
    Returns (o [B,T,Hq,D] fp32, lse [B,T,Hq] natural log of the scaled row sums; -inf if empty).
    ``q_pos`` (optional, [T]) gives the sequence positions of the query rows when q holds only some
    rows of the sequence (row-chunked checks at full size)."""
    B, T, Hq, D = q.shape
    Tc, Hk = ck.shape[1], ck.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    g = Hq // Hk
    ckr = ck.float().repeat_interleave(g, dim=2) if g > 1 else ck.float()
    cvr = cv.float().repeat_interleave(g, dim=2) if g > 1 else cv.float()
    s = torch.einsum("bthd,bshd->bhts", q.float(), ckr) * scale
    if causal:
        row = (torch.arange(T) if q_pos is None else q_pos).unsqueeze(1)
        col = torch.arange(Tc).unsqueeze(0)
        masked = col * stride + block > row
        s = s.masked_fill(masked, float("-inf"))
        empty = masked.all(-1)
    else:
        empty = torch.zeros(T, dtype=torch.bool)
    with torch.no_grad():
        lse = torch.logsumexp(s, dim=-1)                               # [B,Hq,T]
    ev = empty.view(1, 1, T, 1)
    p = torch.softmax(s.masked_fill(ev, 0.0), dim=-1).masked_fill(ev, 0.0)
    o = torch.einsum("bhts,bshd->bthd", p, cvr)
    return o, lse.permute(0, 2, 1).contiguous()


# --------------------------------------------------------------------------
# selected-block attention and sliding-window attention
# --------------------------------------------------------------------------


def selected_attention(q, k, v, block_indices, block_counts=None, block_size: int = 64,
                       scale: Optional[float] = None, chunk: int = 128, q_pos=None):
    """Attention of every query over the keys of its selected blocks.
    A key at position p of block b (p = b*block_size + r) takes part iff b >= 0, p <= t and the
    slot is below ``block_counts``; a query with no valid key gives 0 (the reference's NaN -> 0
    convention).  Follows naive_nsa, tests/test_parallel_nsa.py:81-144 and :207-212, and the
    skip rule of nsa/selection_attn.py:454,464.
    q [B,T,Hq,D]; k,v [B,T,Hkv,D]; block_indices [B,T,Hkv,S].  Returns (o fp32, lse fp32).
    ``q_pos`` (optional, [Tq]) gives the sequence positions of the query rows when q holds only a
    subset of the rows (row-sampled checks at full size); k,v always hold the whole sequence."""
    B, Tq, Hq, D = q.shape
    T = k.shape[1]
    if q_pos is None:
        q_pos = torch.arange(Tq)
    Hkv = k.shape[2]
    G = Hq // Hkv
    S = block_indices.shape[-1]
    if scale is None:
        scale = D ** -0.5
    qf, kf, vf = q.float(), k.float(), v.float()
    o = qf.new_zeros(B, Tq, Hq, v.shape[-1])
    lse = qf.new_full((B, Tq, Hq), float("-inf"))
    r = torch.arange(block_size)
    for b in range(B):
        for t0 in range(0, Tq, chunk):
            t1 = min(Tq, t0 + chunk)
            idx = block_indices[b, t0:t1].long()                                # [c,Hkv,S]
            pos = idx.unsqueeze(-1) * block_size + r                           # [c,Hkv,S,bs]
            tt = q_pos[t0:t1].view(-1, 1, 1, 1)
            bad = (idx.unsqueeze(-1) < 0) | (pos > tt)
            if block_counts is not None:
                if torch.is_tensor(block_counts):
                    cnt = block_counts[b, t0:t1].long().view(t1 - t0, Hkv, 1, 1)
                else:
                    cnt = int(block_counts)
                bad = bad | (torch.arange(S).view(1, 1, S, 1) >= cnt)
            pos = pos.clamp(0, T - 1).reshape(t1 - t0, Hkv, S * block_size)
            bad = bad.reshape(t1 - t0, Hkv, S * block_size)
            for h in range(Hkv):
                kk = kf[b, :, h][pos[:, h]]                                     # [c,N,D]
                vv = vf[b, :, h][pos[:, h]]
                qq = qf[b, t0:t1, h * G:(h + 1) * G] * scale                    # [c,G,D]
                s = torch.einsum("cgd,cnd->cgn", qq, kk)
                s = s.masked_fill(bad[:, h].unsqueeze(1), float("-inf"))
                empty = bad[:, h].all(-1).view(-1, 1, 1)
                with torch.no_grad():
                    l = torch.logsumexp(s, -1)
                # rows with no valid key: output 0, and no NaN in the gradient either
                p = torch.softmax(s.masked_fill(empty, 0.0), -1).masked_fill(empty, 0.0)
                o[b, t0:t1, h * G:(h + 1) * G] = torch.einsum("cgn,cnd->cgd", p, vv)
                lse[b, t0:t1, h * G:(h + 1) * G] = l
    return o, lse


def sliding_window_attention(q, k, v, window: int, scale: Optional[float] = None, chunk: int = 256, q0: int = 0):
    """Query t attends keys max(0, t-window+1) .. t.  tests/test_parallel_nsa.py:147-156 and
    nsa/selection_attn.py:484-511.  Returns (o fp32 [B,T,Hq,D], lse fp32 [B,T,Hq]).
    With ``q0`` the rows of q are the sequence positions q0 .. q0+T-1 (k, v hold the whole sequence)."""
    if q0:
        k0 = max(0, q0 - window + 1)
        n = q.shape[1]
        pad = q.new_zeros(q.shape[0], q0 - k0, q.shape[2], q.shape[3])
        o, lse = sliding_window_attention(torch.cat([pad, q], 1), k[:, k0:q0 + n], v[:, k0:q0 + n], window, scale, chunk)
        return o[:, q0 - k0:], lse[:, q0 - k0:]
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    if scale is None:
        scale = D ** -0.5
    qf, kf, vf = q.float(), k.float(), v.float()
    o = qf.new_zeros(B, T, Hq, v.shape[-1])
    lse = qf.new_zeros(B, T, Hq)
    for t0 in range(0, T, chunk):
        t1 = min(T, t0 + chunk)
        k0 = max(0, t0 - window + 1)
        row = torch.arange(t0, t1).unsqueeze(1)
        col = torch.arange(k0, t1).unsqueeze(0)
        bad = (col > row) | (col < row - window + 1)
        kk = kf[:, k0:t1].repeat_interleave(G, dim=2)
        vv = vf[:, k0:t1].repeat_interleave(G, dim=2)
        s = torch.einsum("bthd,bshd->bhts", qf[:, t0:t1] * scale, kk)
        s = s.masked_fill(bad, float("-inf"))
        lse[:, t0:t1] = torch.logsumexp(s, -1).permute(0, 2, 1)
        o[:, t0:t1] = torch.einsum("bhts,bshd->bthd", torch.softmax(s, -1), vv)
    return o, lse


def parallel_nsa(q, k, v, g_slc, g_swa, block_indices, block_counts=None, block_size=64,
                 window_size=0, scale=None):
    """o = o_slc * g_slc (+ o_swa * g_swa when window_size > 0): nsa/selection_attn.py:805-811."""
    if isinstance(block_counts, int):
        block_indices = block_indices[..., :block_counts]
        block_counts = None
    o_slc, _ = selected_attention(q, k, v, block_indices, block_counts, block_size, scale)
    o = o_slc * g_slc.float().unsqueeze(-1)
    if window_size > 0:
        o_swa, _ = sliding_window_attention(q, k, v, window_size, scale)
        o = o + o_swa * g_swa.float().unsqueeze(-1)
    return o


# --------------------------------------------------------------------------
# the whole module (nsa/nsa.py:63-135)
# --------------------------------------------------------------------------


def nsa_forward(q, k, v, wk, bk, wv, bv, wg, bg, *, stride=16, block=32, sel_block=64, n_sel=16,
                window=512, scale=None, causal=True, gate_sigmoid=False, return_parts=False):
    """End-to-end NSAAttention.forward on equal-length sequences.
    q [B,T,Hq,D]; k,v [B,T,Hkv,D]; wk/wv Conv1d weights [D,D,block] with biases; wg [3,D], bg [3].
    Gates are the raw linear outputs (nsa/nsa.py:117,124-125,133) unless ``gate_sigmoid``.
    Pool parameters as nsa/nsa.py:57-59."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    ck = compress_conv(k, wk, bk, block, stride)
    cv = compress_conv(v, wv, bv, block, stride)
    o_cmp, _ = cmp_attention(q, ck, cv, stride, block, causal, scale)
    pk, ps, pp = sel_block // stride + 1, sel_block // stride, block // stride - 2
    sc = pooled_scores(q, ck, Hkv, pk, ps, pp)
    idx = topn_blocks(sc, n_sel)
    gate = q.float() @ wg.float().t() + bg.float()
    if gate_sigmoid:
        gate = torch.sigmoid(gate)
    o_slc, _ = selected_attention(q, k, v, idx, None, sel_block, scale)
    o_swa, _ = sliding_window_attention(q, k, v, window, scale)
    o = o_slc * gate[..., 0:1] + o_swa * gate[..., 1:2] + o_cmp * gate[..., 2:3]
    if return_parts:
        return o, dict(ck=ck, cv=cv, o_cmp=o_cmp, scores=sc, indices=idx, gate=gate, o_slc=o_slc,
                       o_swa=o_swa)
    return o


def nsa_decode_row(q_row, k, v, wk, bk, wv, bv, wg, bg, *, stride=16, block=32, sel_block=64,
                   n_sel=16, window=512, scale=None, ck=None, cv=None, return_scores=False):
    """The module's output for the single query at position t = L-1 of one sequence, given that
    sequence's whole K/V.  q_row [Hq,D]; k,v [L,Hkv,D].  The same formulas as ``nsa_forward``
    evaluated for the last row only (the reference has no decode entry point; its module
    assumes len(q) == len(k), nsa/nsa.py:97)."""
    L, Hkv, D = k.shape
    Hq = q_row.shape[0]
    G = Hq // Hkv
    t = L - 1
    if scale is None:
        scale = D ** -0.5
    qf = q_row.float()
    if ck is None:   # (a caller may pass the compressed cache it wants the row evaluated on)
        ck = compress_conv(k.unsqueeze(0), wk, bk, block, stride)[0]       # [Tc,Hkv,D]
        cv = compress_conv(v.unsqueeze(0), wv, bv, block, stride)[0]
    ck, cv = ck.float(), cv.float()
    Tc = ck.shape[0]
    if Tc == 0:
        # shorter than one compression block: no compressed key, nothing to select; only the window branch is left
        k0 = max(0, t - window + 1)
        ss = torch.einsum("hd,shd->hs", qf * scale, k[k0:].float().repeat_interleave(G, 1))
        o_swa = torch.einsum("hs,shd->hd", torch.softmax(ss, -1), v[k0:].float().repeat_interleave(G, 1))
        gate = qf @ wg.float().t() + bg.float()
        o = o_swa * gate[:, 1:2]
        idx = torch.zeros(Hkv, 0, dtype=torch.long)
        return (o, idx, qf.new_zeros(Hkv, 0)) if return_scores else (o, idx)
    ckr, cvr = ck.repeat_interleave(G, 1), cv.repeat_interleave(G, 1)      # [Tc,Hq,D]
    raw = torch.einsum("hd,shd->hs", qf, ckr)
    vis = torch.arange(Tc) * stride + block <= t
    s = (raw * scale).masked_fill(~vis, float("-inf"))
    p = torch.nan_to_num(torch.softmax(s, -1), nan=0.0) if vis.any() else torch.zeros_like(s)
    o_cmp = torch.einsum("hs,shd->hd", p, cvr)
    psel = torch.softmax(raw, -1).reshape(Hkv, G, Tc).sum(1)
    pk, ps, pp = sel_block // stride + 1, sel_block // stride, block // stride - 2
    nb = pool_out_len(Tc, pk, ps, pp)
    sc = psel.new_zeros(Hkv, nb)
    for blk in range(nb):
        lo = blk * ps - pp
        hi = min(lo + pk, Tc + pp)
        sc[:, blk] = psel[:, max(lo, 0):min(hi, Tc)].sum(-1) / (hi - lo)
    idx = torch.argsort(-sc, dim=-1, stable=True)[:, :min(n_sel, nb)]      # [Hkv,n] (fewer when fewer blocks exist)
    o_slc = qf.new_zeros(Hq, D)
    for h in range(Hkv):
        pos = (idx[h].unsqueeze(1) * sel_block + torch.arange(sel_block)).reshape(-1)
        ok = pos <= t
        pos = pos[ok]
        if pos.numel():
            ss = torch.einsum("gd,nd->gn", qf[h * G:(h + 1) * G] * scale, k[pos, h].float())
            o_slc[h * G:(h + 1) * G] = torch.softmax(ss, -1) @ v[pos, h].float()
    k0 = max(0, t - window + 1)
    ss = torch.einsum("hd,shd->hs", qf * scale, k[k0:].float().repeat_interleave(G, 1))
    o_swa = torch.einsum("hs,shd->hd", torch.softmax(ss, -1), v[k0:].float().repeat_interleave(G, 1))
    gate = qf @ wg.float().t() + bg.float()
    o = o_slc * gate[:, 0:1] + o_swa * gate[:, 1:2] + o_cmp * gate[:, 2:3]
    if return_scores:
        return o, idx, sc
    return o, idx


# --------------------------------------------------------------------------
# helpers shared by the parity tests
# --------------------------------------------------------------------------


def index_sets_match(idx_test: torch.Tensor, scores: torch.Tensor, n: int, gap: float = 1e-3):
    """Compare selected block index sets against the oracle scores with the score-gap waiver:
    an index may differ from the oracle's top-n set only if its oracle score is within ``gap``
    of the oracle's n-th largest score.  idx_test [B,T,Hkv,n]; scores [B,Hkv,T,NB].
    Returns (number of rows with a non-waived mismatch, number of rows that differ at all)."""
    sc = scores.permute(0, 2, 1, 3)                                   # [B,T,Hkv,NB]
    nb = sc.shape[-1]
    ref_sorted, _ = torch.sort(sc, dim=-1, descending=True)
    nth = ref_sorted[..., n - 1:n]                                    # [B,T,Hkv,1]
    ref_idx = topn_blocks(scores, n)
    in_ref = torch.zeros_like(sc, dtype=torch.bool).scatter_(-1, ref_idx, True)
    in_tst = torch.zeros_like(sc, dtype=torch.bool).scatter_(-1, idx_test.long().clamp(0, nb - 1), True)
    dup_free = in_tst.sum(-1) == n
    diff = in_ref ^ in_tst
    waived = (sc - nth).abs() < gap
    hard = (diff & ~waived).any(-1) | ~dup_free
    return int(hard.sum()), int(diff.any(-1).sum())
