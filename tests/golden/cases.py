"""Seeded input generators shared by ``make_golden.py`` (which feeds them to the reference's own
functions) and by the oracle tests (which feed them to ``oracle/nsa_oracle.py``).

Inputs are regenerated from the seed rather than stored; each fixture carries a checksum of its
inputs so a drifting random stream is detected instead of silently comparing different data.
"""
import torch


def _r(x):
    """Round to bf16-representable values, so fp32 references and bf16 kernels see identical inputs."""
    return x.bfloat16().float()


def checksum(*tensors) -> float:
    acc = 0.0
    for t in tensors:
        tf = t.detach().double().reshape(-1)
        w = torch.arange(1, tf.numel() + 1, dtype=torch.float64) % 97 + 1
        acc += float((tf * w).sum())
    return acc


def cmp_case(name):
    """Compressed attention + selection.  Returns dict of tensors and hyper-parameters."""
    cfgs = {
        # name: seed, B, T, Hq, Hkv, D, block, stride, sel_block, n
        "cmp_l32": (101, 1, 192, 16, 1, 64, 32, 16, 64, 2),
        "cmp_l64": (102, 1, 192, 32, 2, 64, 64, 16, 64, 2),
    }
    seed, B, T, Hq, Hkv, D, block, stride, sel_block, n = cfgs[name]
    g = torch.Generator().manual_seed(seed)
    Tc = (T - block) // stride + 1
    q = _r(torch.randn(B, T, Hq, D, generator=g))
    ck = _r(torch.randn(B, Tc, Hkv, D, generator=g))
    cv = _r(torch.randn(B, Tc, Hkv, D, generator=g))
    do = _r(torch.randn(B, T, Hq, D, generator=g))
    return dict(q=q, ck=ck, cv=cv, do=do, block=block, stride=stride, Hkv=Hkv,
                pool_kernel=sel_block // stride + 1, pool_stride=sel_block // stride,
                pool_pad=block // stride - 2, n=n)


def sel_case(name):
    """Selected-block (+ sliding window) attention with block_counts and poisoned indices."""
    cfgs = {
        # name: seed, B, T, H, HQ, D, S, block_size, window
        "sel_only": (201, 2, 128, 1, 16, 64, 3, 32, 0),
        "sel_gqa2": (202, 2, 96, 2, 32, 64, 2, 16, 0),
        "swa_only": (203, 2, 128, 1, 16, 64, 2, 32, 48),
    }
    seed, B, T, H, HQ, D, S, bs, window = cfgs[name]
    g = torch.Generator().manual_seed(seed)
    q = _r(torch.randn(B, T, HQ, D, generator=g))
    k = _r(torch.randn(B, T, H, D, generator=g))
    v = _r(torch.randn(B, T, H, D, generator=g))
    g_slc = _r(torch.rand(B, T, HQ, generator=g))
    g_swa = _r(torch.rand(B, T, HQ, generator=g))
    do = _r(torch.randn(B, T, HQ, D, generator=g))
    idx = torch.full((B, T, H, S), T, dtype=torch.long)
    for b in range(B):
        for t in range(T):
            for h in range(H):
                perm = torch.randperm(max(1, t // bs + 1), generator=g)[:S]
                idx[b, t, h, :len(perm)] = perm
    idx = idx.sort(-1)[0]
    # a few rows whose every selected block lies in the future (empty selection)
    idx[0, 0, 0, :] = 3
    idx[1, 63, 0, :] = T // bs - 1
    counts = torch.randint(1, S + 1, (B, T, H), generator=g)
    if window > 0:
        g_slc = torch.zeros_like(g_slc)      # isolates the sliding-window term of naive_nsa
    return dict(q=q, k=k, v=v, g_slc=g_slc, g_swa=g_swa, do=do, idx=idx, counts=counts,
                block_size=bs, window=window)


def compress_case(name):
    cfgs = {
        # name: seed, B, T, H, D, block, stride
        "cmpr_l32": (301, 2, 112, 2, 64, 32, 16),
        "cmpr_l64": (302, 3, 160, 1, 64, 64, 16),
    }
    seed, B, T, H, D, block, stride = cfgs[name]
    g = torch.Generator().manual_seed(seed)
    x = _r(torch.randn(B * T, H, D, generator=g))
    w = _r(torch.randn(block * D, D, generator=g) * 0.05)
    conv_w = _r(torch.randn(D, D, block, generator=g) * 0.05)
    conv_b = _r(torch.randn(D, generator=g) * 0.05)
    cu = [T * i for i in range(B + 1)]
    return dict(x=x, w=w, conv_w=conv_w, conv_b=conv_b, cu=cu, B=B, T=T, block=block, stride=stride)


CMP_CASES = ["cmp_l32", "cmp_l64"]
SEL_CASES = ["sel_only", "sel_gqa2", "swa_only"]
COMPRESS_CASES = ["cmpr_l32", "cmpr_l64"]
