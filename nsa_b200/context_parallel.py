"""Context (sequence) parallelism for NSAAttention: every rank owns a slice of the query tokens of one long
sequence, K/V are all-gathered over NCCL, and each rank runs the NSA kernels for its queries only.

The reference has no distributed code; this follows the sharding of BASELINE config 4 (B=1, T=65536 split over
2/4/8 GPUs).  What moves over NVLink per layer: the all-gather of K and V (Hkv is small: 134 MB in total at
T=64K) and, in the backward, the reduce-scatter of dK/dV.  The compressed K/V are recomputed from the gathered
K/V on every rank (34 GFLOP, cheaper than another collective); their weight gradients come out as per-rank
partial sums, like the gate's, and are all-reduced by the caller with the other parameters (data-parallel style).

Causal work grows with the position, so contiguous slices would leave the last rank with most of the compressed
branch: with ``zigzag=True`` (default) the sequence is cut in 2P chunks and rank r owns chunks r and 2P-1-r.
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


def context_parallel_forward(module, q, k, v, group=None, zigzag=True, causal=True):
    """NSAAttention.forward for one context-sharded sequence batch.

    q [B,Tl,Hq,D], k, v [B,Tl,Hkv,D]: this rank's tokens (with ``zigzag`` the first half of the local tokens is chunk
    ``rank`` and the second half chunk ``2P-1-rank`` of the sequence cut in 2P chunks).  Returns o [B,Tl,Hq,D] for the
    same tokens.  Gradients: dq local; dk, dv summed over ranks and scattered back by the gather's backward; parameter
    gradients are per-rank partial sums (all-reduce them with the rest of the model's)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, Tl, Hq, D = q.shape
    Hkv = k.shape[2]
    layout = chunk_layout(world, zigzag)
    per = len(layout[0])
    if Tl % per:
        raise ValueError("local token count must be even for the zig-zag layout")
    cl = Tl // per
    T = Tl * world
    k_full = _GatherTokens.apply(k, group, zigzag)
    v_full = _GatherTokens.apply(v, group, zigzag)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=q.device)
    ck, cv, _ = module.compressor(k_full.reshape(B * T, Hkv, D), v_full.reshape(B * T, Hkv, D), cu, None)
    scale = module.softmax_scale
    if scale is None or scale is True:
        scale = 1.0 if scale is True else D ** -0.5
    outs = []
    for i, cid in enumerate(layout[rank]):
        sl = slice(i * cl, (i + 1) * cl)
        cfg = (module.compression_stride, module.compression_block, bool(causal), float(scale), module.pool_kernel_size,
               module.pool_stride, module.pool_padding, module.selected_block_count, module.selection_block_size,
               module.sliding_window, cid * cl)
        outs.append(_NSACore.apply(q[:, sl].contiguous(), k_full, v_full, ck, cv, module.gating.weight, module.gating.bias,
                                   cfg))
    return torch.cat(outs, dim=1)
