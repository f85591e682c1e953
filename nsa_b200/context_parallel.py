"""Context (sequence) parallelism for NSAAttention: every rank owns a slice of the query tokens of one long
sequence, K/V are all-gathered over NCCL, and each rank runs the NSA kernels for its queries only.

The reference has no distributed code; this follows the sharding of BASELINE config 4 (B=1, T=65536 split over
2/4/8 GPUs).  What moves over NVLink per layer:
  * one all-gather of the rank's K and V tokens (K and V travel as one tensor; Hkv is small: 134 MB in total at T=64K)
    and, in the backward, one reduce-scatter of dK/dV;
  * one all-gather of the compressed K/V (8.4 MB at T=64K): every rank compresses only its own 1/P of the compressed
    positions from the gathered K/V (their windows overlap neighbouring ranks' tokens, so the gather comes first), and
    in the backward the partial dCK/dCV of all ranks are reduce-scattered to the rank that owns the positions, which
    alone runs the compression backward for them.
Compression weight gradients and the gate's come out as per-rank partial sums and are all-reduced by the caller with
the other parameters (data-parallel style).

Causal work grows with the position, so contiguous slices would leave the last rank with most of the compressed
branch: with ``zigzag=True`` (default) the sequence is cut in 2P chunks and rank r owns chunks r and 2P-1-r.  A
chunk's kernels see only the keys up to the chunk's last token (nothing later can be attended), so the reverse index,
the kv-major backward grid and the dK/dV they write cover that prefix, not the whole sequence.
"""
import torch
import torch.distributed as dist

from .nsa import _NSACore


def chunk_layout(world, zigzag):
    """Chunk ids (in sequence order) held by each rank, in the order they are stored locally."""
    if not zigzag:
        return [[r] for r in range(world)]
    return [[r, 2 * world - 1 - r] for r in range(world)]


class _GatherTokens(torch.autograd.Function):
    """x_local [B,Tl,H,D] -> x_full [B,T,H,D] in sequence order.  Backward: the sum over ranks of the full-length
    gradient, restricted to the local tokens (reduce-scatter; all-reduce + slice on backends without it)."""

    @staticmethod
    def forward(ctx, x, group, zigzag):
        world = dist.get_world_size(group)
        B, Tl, H, D = x.shape
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        layout = chunk_layout(world, zigzag)
        per = len(layout[0])
        cl = Tl // per
        chunks = [None] * (world * per)
        for r in range(world):
            for i, cid in enumerate(layout[r]):
                chunks[cid] = parts[r][:, i * cl:(i + 1) * cl]
        ctx.meta = (group, zigzag, cl)
        return torch.cat(chunks, dim=1)

    @staticmethod
    def backward(ctx, g):
        group, zigzag, cl = ctx.meta
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        layout = chunk_layout(world, zigzag)
        g = g.contiguous()
        if dist.get_backend(group) == "nccl":
            # rank-major layout of the full gradient, then one reduce-scatter
            blocks = [torch.cat([g[:, cid * cl:(cid + 1) * cl] for cid in layout[r]], dim=1) for r in range(world)]
            out = torch.empty_like(blocks[rank])
            dist.reduce_scatter(out, [b.contiguous() for b in blocks], group=group)
            return out, None, None
        g = g.clone()          # the incoming gradient may be shared with other consumers: reduce a private copy
        dist.all_reduce(g, group=group)
        return torch.cat([g[:, cid * cl:(cid + 1) * cl] for cid in layout[rank]], dim=1), None, None


class _GatherRows(torch.autograd.Function):
    """x_local [B,n_r,H,D] (n_r may differ per rank: ``counts``) -> [B,sum n,H,D] in rank order.  Backward: reduce-scatter
    (every rank receives the summed gradient of the rows it contributed)."""

    @staticmethod
    def forward(ctx, x, counts, group):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        B, n, H, D = x.shape
        cap = max(counts)
        pad = x if n == cap else torch.cat([x, x.new_zeros(B, cap - n, H, D)], 1)
        parts = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(parts, pad.contiguous(), group=group)
        ctx.meta = (counts, group, cap)
        return torch.cat([parts[r][:, :counts[r]] for r in range(world)], 1)

    @staticmethod
    def backward(ctx, g):
        counts, group, cap = ctx.meta
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        B, _, H, D = g.shape
        blocks, pos = [], 0
        for r in range(world):
            blk = g[:, pos:pos + counts[r]]
            pos += counts[r]
            if counts[r] < cap:
                blk = torch.cat([blk, g.new_zeros(B, cap - counts[r], H, D)], 1)
            blocks.append(blk.contiguous())
        if dist.get_backend(group) == "nccl":
            out = torch.empty_like(blocks[rank])
            dist.reduce_scatter(out, blocks, group=group)
        else:
            full = torch.stack(blocks, 0)
            dist.all_reduce(full, group=group)
            out = full[rank]
        return out[:, :counts[rank]].contiguous(), None, None


def _compressed_ranges(Tc, world):
    """Compressed positions [lo, hi) owned by each rank (contiguous, as even as possible)."""
    per = (Tc + world - 1) // world
    return [(min(Tc, r * per), min(Tc, (r + 1) * per)) for r in range(world)]


def context_parallel_forward(module, q, k, v, group=None, zigzag=True, causal=True):
    """NSAAttention.forward for one context-sharded sequence batch.

    q [B,Tl,Hq,D], k, v [B,Tl,Hkv,D]: this rank's tokens (with ``zigzag`` the first half of the local tokens is chunk
    ``rank`` and the second half chunk ``2P-1-rank`` of the sequence cut in 2P chunks).  Returns o [B,Tl,Hq,D] for the
    same tokens.  Gradients: dq local; dk, dv summed over ranks and scattered back by the gather's backward; parameter
    gradients are per-rank partial sums (all-reduce them with the rest of the model's)."""
    from .compression_kv import compress_conv
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, Tl, Hq, D = q.shape
    Hkv = k.shape[2]
    layout = chunk_layout(world, zigzag)
    per = len(layout[0])
    if Tl % per:
        raise ValueError("local token count must be even for the zig-zag layout")
    cl = Tl // per
    T = Tl * world
    # K and V travel together: one all-gather forward, one reduce-scatter backward
    kv_full = _GatherTokens.apply(torch.cat([k, v], 2), group, zigzag)
    k_full, v_full = kv_full[:, :, :Hkv], kv_full[:, :, Hkv:]
    # compression sharded over the compressed positions: mine are [lo, hi), their windows cover tokens
    # [lo*stride, (hi-1)*stride + block)
    block, stride = module.compression_block, module.compression_stride
    Tc = (T - block) // stride + 1
    ranges = _compressed_ranges(Tc, world)
    lo, hi = ranges[rank]
    comp = module.compressor
    if hi > lo:
        t0, t1 = lo * stride, (hi - 1) * stride + block
        ks = k_full[:, t0:t1].reshape(B * (t1 - t0), Hkv, D)
        vs = v_full[:, t0:t1].reshape(B * (t1 - t0), Hkv, D)
        ck_part = compress_conv(ks, comp.compressor_k.weight, comp.compressor_k.bias, block, stride, B)
        cv_part = compress_conv(vs, comp.compressor_v.weight, comp.compressor_v.bias, block, stride, B)
        ckv_part = torch.cat([ck_part, cv_part], 2)
    else:
        ckv_part = k_full.new_zeros(B, 0, 2 * Hkv, D) + 0 * (comp.compressor_k.weight.sum() + comp.compressor_v.weight.sum())
    ckv = _GatherRows.apply(ckv_part, [h_ - l_ for l_, h_ in ranges], group)
    ck, cv = ckv[:, :, :Hkv].contiguous(), ckv[:, :, Hkv:].contiguous()
    scale = module.softmax_scale
    if scale is None or scale is True:
        scale = 1.0 if scale is True else D ** -0.5
    outs = []
    for i, cid in enumerate(layout[rank]):
        sl = slice(i * cl, (i + 1) * cl)
        q0 = cid * cl
        t_end = q0 + cl          # no key after the chunk's last token is ever attended
        cfg = (module.compression_stride, module.compression_block, bool(causal), float(scale), module.pool_kernel_size,
               module.pool_stride, module.pool_padding, module.selected_block_count, module.selection_block_size,
               module.sliding_window, q0)
        outs.append(_NSACore.apply(q[:, sl].contiguous(), k_full[:, :t_end].contiguous(), v_full[:, :t_end].contiguous(),
                                   ck, cv, module.gating.weight, module.gating.bias, cfg))
    return torch.cat(outs, dim=1)
