"""GPU parity tests: the CUDA kernels (reached through the C ABI via the nsa_b200 package) against the CPU
oracle and against the golden fixtures made from the reference's own functions.

Tolerance (outputs and gradients, bf16 kernels vs fp32 oracle on identical bf16-representable inputs):
2e-2 absolute / 1e-2 relative.  Selected block index sets must equal the oracle's except where the oracle
score is within 1e-3 of its n-th largest score.
"""
import os

import numpy as np
import pytest
import torch

import cases
from oracle import nsa_oracle as O
from parity_util import ATOL, RTOL, DEV, close as _close, dev as _dev, index_report

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _gold(name):
    d = np.load(os.path.join(GOLD, name + ".npz"))
    return {k: torch.from_numpy(np.asarray(d[k])) for k in d.files}


@pytest.fixture(scope="module")
def nsa():
    import nsa_b200
    yield nsa_b200
    nsa_b200._lib.device_status()


def _r(x):
    return x.bfloat16().float()


# ------------------------------------------------------------------------------------------------------
# golden fixtures (outputs of the reference's own functions)
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", cases.CMP_CASES)
def test_cmp_attention_golden(nsa, name):
    c, g = cases.cmp_case(name), _gold(name)
    q, ck, cv = (_dev(c[k]).requires_grad_(True) for k in ("q", "ck", "cv"))
    o, idx = nsa.triton_attention.flash_attn_func(q, ck, cv, c["stride"], c["block"], True, None, c["Hkv"],
                                                  c["pool_kernel"], c["pool_stride"], c["pool_pad"], c["n"])
    _close("o", o, g["o"])
    sc = O.pooled_scores(c["q"], c["ck"], c["Hkv"], c["pool_kernel"], c["pool_stride"], c["pool_pad"])
    hard, soft = O.index_sets_match(idx.cpu(), sc, c["n"], gap=1e-3)
    index_report("golden " + name, hard, soft, idx.numel() // idx.shape[-1])
    assert hard == 0, "%d rows select a block outside the 1e-3 waiver (%d rows differ at all)" % (hard, soft)
    o.backward(_dev(c["do"]))
    _close("dq", q.grad, g["dq"])
    _close("dck", ck.grad, g["dck"], scaled=True)
    _close("dcv", cv.grad, g["dcv"], scaled=True)
    nsa._lib.device_status()


@pytest.mark.parametrize("name", cases.SEL_CASES)
def test_selection_golden(nsa, name):
    c, g = cases.sel_case(name), _gold(name)
    q, k, v = (_dev(c[x]).requires_grad_(True) for x in ("q", "k", "v"))
    o = nsa.selection_attention(q, k, v, _dev(c["g_slc"]), _dev(c["g_swa"]), c["idx"].to(DEV), c["counts"].to(DEV),
                                c["block_size"], c["window"])
    _close("o", o, g["o"])
    if c["window"] > 0:
        o.backward(_dev(c["do"]))
        _close("dq", q.grad, g["dq"])
        _close("dk", k.grad, g["dk"], scaled=True)
        ok = ~torch.isnan(g["dv"])          # the reference's dv holds NaN at keys of its empty-selection rows
        _close("dv", torch.where(ok, v.grad.float().cpu(), torch.zeros(())), torch.nan_to_num(g["dv"], nan=0.0), scaled=True)
    nsa._lib.device_status()


@pytest.mark.parametrize("name", cases.COMPRESS_CASES)
def test_compression_golden(nsa, name):
    c, g = cases.compress_case(name), _gold(name)
    x = _dev(c["x"]).requires_grad_(True)
    w = _dev(c["w"]).requires_grad_(True)
    cu = torch.tensor(c["cu"], dtype=torch.int32, device=DEV)
    ck, cv, cu_out = nsa.compression_kv.compress_kv(x, x, w, w, cu, c["stride"], c["block"])
    _close("y", ck, g["y"])
    _close("y(v)", cv, g["y"])
    n = nsa.compression_kv.calc_compressed_len(c["T"], c["stride"], c["block"])
    assert cu_out.tolist() == [n * i for i in range(c["B"] + 1)]
    tgt = torch.sin(torch.arange(ck.numel(), dtype=torch.float32)).reshape(ck.shape)
    ck.backward(_dev(tgt))
    # the kernel sees the bf16-rounded upstream gradient; the golden used the fp32 one
    _close("dx", x.grad, g["dx"], scaled=True)
    _close("dw", w.grad, g["dw"], scaled=True)
    comp = nsa.compression_kv.KVCompressor(c["stride"], c["block"], x.shape[-1], DEV, torch.bfloat16)
    with torch.no_grad():
        comp.compressor_k.weight.copy_(c["conv_w"])
        comp.compressor_k.bias.copy_(c["conv_b"])
        comp.compressor_v.weight.copy_(c["conv_w"].flip(0))
        comp.compressor_v.bias.copy_(c["conv_b"].flip(0))
    yk, yv, _ = comp(_dev(c["x"]), _dev(c["x"] * 0.5), cu, None)
    _close("conv_k", yk, g["conv_k"])
    _close("conv_v", yv, g["conv_v"])
    nsa._lib.device_status()


# ------------------------------------------------------------------------------------------------------
# oracle comparisons at D = 128 / larger shapes, forward and backward
# ------------------------------------------------------------------------------------------------------
def _rand_indices(B, T, H, S, BS, gen, poison=True):
    idx = torch.full((B, T, H, S), -1, dtype=torch.long)
    for b in range(B):
        for t in range(T):
            for h in range(H):
                nblk = t // BS + 1
                perm = torch.randperm(nblk, generator=gen)[:S]
                idx[b, t, h, :len(perm)] = perm
    if poison:
        idx[0, 5, 0, :] = T // BS            # only future blocks: empty selection
        idx[-1, T - 1, -1, 0] = (T - 1) // BS  # make sure the local block is present somewhere
    return idx


@pytest.mark.parametrize("D,BS,S,Hq,Hkv,T,window", [(128, 64, 4, 32, 2, 384, 100), (64, 32, 5, 16, 1, 200, 0),
                                                    (128, 16, 3, 16, 1, 130, 33), (64, 64, 6, 32, 2, 300, 0),
                                                    (128, 64, 20, 16, 1, 450, 0), (64, 64, 36, 16, 1, 2400, 0),
                                                    (128, 64, 4, 32, 1, 300, 64)])   # last: 32 query heads per KV head
def test_selection_and_window_fwd_bwd(nsa, D, BS, S, Hq, Hkv, T, window):
    gen = torch.Generator().manual_seed(1234 + D + BS)
    B = 2 if T < 1000 else 1     # the 36-selection case (general kernel at 64-key blocks) is long: one sequence
    q = _r(torch.randn(B, T, Hq, D, generator=gen))
    k = _r(torch.randn(B, T, Hkv, D, generator=gen))
    v = _r(torch.randn(B, T, Hkv, D, generator=gen))
    do_slc = _r(torch.randn(B, T, Hq, D, generator=gen))
    do_swa = _r(torch.randn(B, T, Hq, D, generator=gen))
    idx = _rand_indices(B, T, Hkv, S, BS, gen)
    counts = torch.randint(1, S + 1, (B, T, Hkv), generator=gen)
    qd, kd, vd = (_dev(x).requires_grad_(True) for x in (q, k, v))
    o_slc, o_swa = nsa.selection_attn.ParallelNSAFunction.apply(qd, kd, vd, idx.to(DEV), counts.to(DEV), BS, window,
                                                                D ** -0.5, None)
    qo, ko, vo = (x.clone().requires_grad_(True) for x in (q, k, v))
    r_slc, r_lse = O.selected_attention(qo, ko, vo, idx, counts, BS)
    _close("o_slc", o_slc, r_slc)
    loss_k = (o_slc.float() * _dev(do_slc).float()).sum()
    loss_o = (r_slc * do_slc).sum()
    if window > 0:
        r_swa, _ = O.sliding_window_attention(qo, ko, vo, window)
        _close("o_swa", o_swa, r_swa)
        loss_k = loss_k + (o_swa.float() * _dev(do_swa).float()).sum()
        loss_o = loss_o + (r_swa * do_swa).sum()
    loss_k.backward()
    loss_o.backward()
    _close("dq", qd.grad, qo.grad)
    _close("dk", kd.grad, ko.grad, scaled=True)
    _close("dv", vd.grad, vo.grad, scaled=True)
    nsa._lib.device_status()


@pytest.mark.parametrize("case", [(128, 64, 4, 32, 2, 384, 100), (128, 64, 20, 16, 1, 450, 0)])
def test_selection_bwd_query_major_dq(nsa, case):
    """The same comparison with the small workspace: the selected branch's dQ then comes from the query-major kernel
    instead of the key-major kernel's per-visit partial tiles (the default, which the test above covers)."""
    old = nsa._lib.SEL_DQ_FROM_KV
    nsa._lib.SEL_DQ_FROM_KV = False
    try:
        test_selection_and_window_fwd_bwd(nsa, *case)
    finally:
        nsa._lib.SEL_DQ_FROM_KV = old


@pytest.mark.parametrize("case", [(128, 64, 4, 32, 2, 384, 100), (128, 64, 20, 16, 1, 450, 0), (128, 64, 4, 32, 1, 300, 64)])
def test_selection_fwd_query_major(nsa, case):
    """The same comparison with the selected branch's forward on the query-major kernel (no workspace) instead of the
    key-major tensor-core path (reverse index, per-visit partial tiles, slot-order merge), which is the default and which
    the test above covers.  The last case has two 16-head groups per KV head."""
    old = nsa._lib.SEL_FWD_KV
    nsa._lib.SEL_FWD_KV = False
    try:
        test_selection_and_window_fwd_bwd(nsa, *case)
    finally:
        nsa._lib.SEL_FWD_KV = old


def test_workspace_size_selects_the_selected_branch_kernels(nsa):
    """The C entry points pick the key-major tensor-core kernels only when the caller's workspace is large enough:
    a workspace that is too small must give exactly the query-major results (forward), and the two backward forms
    must agree (dK, dV bit-equal: the same kernel with and without the dQ partials; dQ within the bf16 rounding of
    the partial tiles)."""
    L, P, S = nsa._lib.lib(), nsa._lib.ptr, nsa._lib.stream
    B, T, Hq, Hkv, D, n, BS = 1, 640, 32, 2, 128, 6, 64
    gen = torch.Generator().manual_seed(77)
    q, do = (_dev(_r(torch.randn(B, T, Hq, D, generator=gen))) for _ in range(2))
    k, v = (_dev(_r(torch.randn(B, T, Hkv, D, generator=gen))) for _ in range(2))
    idx = _rand_indices(B, T, Hkv, n, BS, gen).to(torch.int32).to(DEV).contiguous()
    scale = D ** -0.5
    outs = []
    nws = L.nsa_sel_swa_fwd_workspace_bytes(B, T, T, Hq, Hkv, D, n, BS)
    for ws_bytes in (0, 4096, nws):
        o = torch.empty_like(q)
        lse = torch.empty(B, T, Hq, dtype=torch.float32, device=DEV)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=DEV)
        nsa._lib.check(L.nsa_sel_swa_fwd_ws(P(q), P(k), P(v), P(idx), 0, None, P(o), P(lse), None, None, None, None, None,
                                            None, None, P(ws) if ws_bytes else None, ws_bytes, B, T, Hq, Hkv, D, n, BS, 0,
                                            scale, T, 0, S()), "nsa_sel_swa_fwd_ws")
        outs.append((o, lse))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    _close("o key-major vs query-major", outs[2][0], outs[0][0].float().cpu())
    fin = torch.isfinite(outs[0][1])
    assert torch.equal(fin, torch.isfinite(outs[2][1]))
    assert (outs[2][1][fin] - outs[0][1][fin]).abs().max().item() < 5e-3
    o, lse = outs[0]
    delta = (o.float() * do.float()).sum(-1).contiguous()
    res = []
    for big in (False, True):
        nb = (L.nsa_sel_swa_bwd_workspace_bytes_dq(B, T, T, Hq, Hkv, D, n, BS) if big
              else L.nsa_sel_swa_bwd_workspace_bytes(B, T, Hkv, n, BS))
        ws = torch.empty(nb, dtype=torch.uint8, device=DEV)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        nsa._lib.check(L.nsa_sel_swa_bwd(P(q), P(k), P(v), P(idx), 0, None, P(do), P(lse), P(delta), None, None, None, None,
                                         None, P(dq), 0, P(dk), P(dv), P(ws), nb, B, T, Hq, Hkv, D, n, BS, 0, scale, S()),
                       "nsa_sel_swa_bwd")
        res.append((dq, dk, dv))
    assert torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][2], res[1][2])
    _close("dq key-major vs query-major", res[1][0], res[0][0].float().cpu())
    nsa._lib.device_status()


def test_selection_varlen_cu_seqlens(nsa):
    """parallel_nsa with cu_seqlens (packed sequences of different lengths, batch 1): block indices and masks are
    relative to each sequence, as in the reference's varlen indexing (nsa/selection_attn.py:419-425).  Forward and
    backward against the oracle evaluated sequence by sequence."""
    gen = torch.Generator().manual_seed(99)
    D, BS, S, Hq, Hkv, window = 128, 64, 4, 32, 2, 100
    lens = [130, 384, 77]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    q, k, v = (_r(torch.randn(1, T, h, D, generator=gen)) for h in (Hq, Hkv, Hkv))
    g_slc, g_swa = (_r(torch.rand(1, T, Hq, generator=gen)) for _ in range(2))
    do = _r(torch.randn(1, T, Hq, D, generator=gen))
    idx = torch.cat([_rand_indices(1, n, Hkv, S, BS, gen, poison=False) for n in lens], 1)
    qd, kd, vd = (_dev(x).requires_grad_(True) for x in (q, k, v))
    o = nsa.selection_attention(qd, kd, vd, _dev(g_slc), _dev(g_swa), idx.to(DEV), None, BS, window,
                                cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=DEV))
    o.backward(_dev(do))
    qo, ko, vo = (x.clone().requires_grad_(True) for x in (q, k, v))
    refs = []
    for a, b in zip(cu[:-1], cu[1:]):
        r = O.parallel_nsa(qo[:, a:b], ko[:, a:b], vo[:, a:b], g_slc[:, a:b], g_swa[:, a:b], idx[:, a:b], None, BS, window)
        (r * do[:, a:b]).sum().backward()
        refs.append(r.detach())
    _close("varlen o", o, torch.cat(refs, 1))
    _close("varlen dq", qd.grad, qo.grad)
    _close("varlen dk", kd.grad, ko.grad, scaled=True)
    _close("varlen dv", vd.grad, vo.grad, scaled=True)
    nsa._lib.device_status()


def test_module_takes_sequences_of_different_lengths(nsa):
    """NSAAttention.forward on packed sequences of unequal lengths equals the per-sequence calls (outputs and gradients)."""
    gen = torch.Generator().manual_seed(98)
    D, Hq, Hkv = 128, 16, 1
    lens = [320, 512]
    T = sum(lens)
    q, k, v = (_dev(_r(torch.randn(T, h, D, generator=gen))) for h in (Hq, Hkv, Hkv))
    do = _dev(_r(torch.randn(T, Hq, D, generator=gen)))
    mod = nsa.NSAAttention(D, True, selected_block_count=3, sliding_window=64, device=DEV, dtype=torch.bfloat16)
    cu = torch.tensor([0, lens[0], T], dtype=torch.int32, device=DEV)
    qa, ka, va = (x.clone().requires_grad_(True) for x in (q, k, v))
    out = mod(qa, ka, va, cu, max(lens))
    out.backward(do)
    wgrad = mod.gating.weight.grad.clone()
    mod.zero_grad()
    outs, grads = [], []
    for a, b in ((0, lens[0]), (lens[0], T)):
        qb, kb, vb = (x[a:b].clone().requires_grad_(True) for x in (q, k, v))
        ob = mod(qb, kb, vb, torch.tensor([0, b - a], dtype=torch.int32, device=DEV), b - a)
        ob.backward(do[a:b])
        outs.append(ob.detach())
        grads.append((qb.grad, kb.grad, vb.grad))
    assert torch.equal(out.detach(), torch.cat(outs, 0))
    for i, name in enumerate(("dq", "dk", "dv")):
        assert torch.equal((qa.grad, ka.grad, va.grad)[i], torch.cat([g[i] for g in grads], 0)), name
    _close("ragged d gating.weight", wgrad, mod.gating.weight.grad, atol=4e-2, scaled=True)
    nsa._lib.device_status()


@pytest.mark.parametrize("D,Hq,Hkv,T,block,stride,causal", [(128, 32, 2, 520, 32, 16, True), (64, 16, 1, 333, 64, 16, True),
                                                            (128, 32, 2, 520, 32, 16, False),
                                                            (64, 16, 1, 333, 64, 16, False)])
def test_cmp_attention_fwd_bwd(nsa, D, Hq, Hkv, T, block, stride, causal):
    gen = torch.Generator().manual_seed(77 + D)
    B, sel_block, n = 2, 64, 3
    Tc = (T - block) // stride + 1
    q = _r(torch.randn(B, T, Hq, D, generator=gen))
    ck = _r(torch.randn(B, Tc, Hkv, D, generator=gen) * 0.5)
    cv = _r(torch.randn(B, Tc, Hkv, D, generator=gen))
    do = _r(torch.randn(B, T, Hq, D, generator=gen))
    pk, ps, pp = sel_block // stride + 1, sel_block // stride, block // stride - 2
    qd, kd, vd = (_dev(x).requires_grad_(True) for x in (q, ck, cv))
    o, idx = nsa.triton_attention.flash_attn_func(qd, kd, vd, stride, block, causal, None, Hkv, pk, ps, pp, n)
    qo, ko, vo = (x.clone().requires_grad_(True) for x in (q, ck, cv))
    ro, _ = O.cmp_attention(qo, ko, vo, stride, block, causal)
    _close("o_cmp", o, ro)
    sc = O.pooled_scores(q, ck, Hkv, pk, ps, pp)
    hard, soft = O.index_sets_match(idx.cpu(), sc, n, gap=1e-3)
    index_report("cmp D=%d T=%d causal=%s" % (D, T, causal), hard, soft, idx.numel() // idx.shape[-1])
    assert hard == 0, "%d rows select a block outside the 1e-3 waiver (%d differ)" % (hard, soft)
    o.backward(_dev(do))
    (ro * do).sum().backward()
    _close("dq", qd.grad, qo.grad)
    _close("dck", kd.grad, ko.grad, scaled=True)
    _close("dcv", vd.grad, vo.grad, scaled=True)
    # the reference's repeated-head calling convention gives the same result
    o2, idx2 = nsa.triton_attention.flash_attn_func(_dev(q), _dev(ck).repeat_interleave(Hq // Hkv, 2),
                                                    _dev(cv).repeat_interleave(Hq // Hkv, 2), stride, block, causal, None,
                                                    Hkv, pk, ps, pp, n)
    assert torch.equal(o2, o) and torch.equal(idx2, idx)
    nsa._lib.device_status()


def test_causal_score_mode(nsa):
    """score_mode = causal: the selection scores are the compressed branch's own (scaled, masked) attention probabilities.
    Pooled scores and the selected sets against the oracle's causal restatement; no selected block starts after the
    query; the module's output with that selection against the oracle composition."""
    from nsa_b200 import _lib
    gen = torch.Generator().manual_seed(6)
    B, T, Hq, Hkv, D, block, stride, n = 1, 2080, 32, 2, 128, 32, 16, 4
    Tc = (T - block) // stride + 1
    q = _r(torch.randn(B, T, Hq, D, generator=gen))
    ck = _r(torch.randn(B, Tc, Hkv, D, generator=gen))
    cv = _r(torch.randn(B, Tc, Hkv, D, generator=gen))
    L, P, S = _lib.lib(), _lib.ptr, _lib.stream
    n_pool = L.nsa_pool_out_len(Tc, 5, 4, 0)
    qd, kd, vd = _dev(q), _dev(ck), _dev(cv)
    o = torch.empty_like(qd)
    lse = torch.empty(B, T, Hq, dtype=torch.float32, device=DEV)
    idx = torch.empty(B, T, Hkv, n, dtype=torch.int32, device=DEV)
    scores = torch.empty(B, Hkv, T, n_pool, dtype=torch.float32, device=DEV)
    _lib.check(L.nsa_cmp_attn_fwd_gated(P(qd), P(kd), P(vd), P(o), P(lse), P(idx), P(scores), None, None, None, None, None,
                                        B, T, Tc, Hq, Hkv, D, block, stride, 1, D ** -0.5, n, 5, 4, 0, 1, T, 0, S()),
               "nsa_cmp_attn_fwd_gated")
    ref = O.pooled_scores_causal(q, ck, Hkv, 5, 4, 0, stride, block)
    _close("causal pooled scores", scores, ref, atol=2e-3, rtol=1e-2)
    ro, _ = O.cmp_attention(q, ck, cv, stride, block, True)
    _close("o_cmp (causal score mode)", o, ro)
    # rows with fewer than n scored blocks pad with zero-score blocks (ties to the lower index); every block with a
    # positive score starts at or before the query
    hard, soft = O.index_sets_match(idx.cpu(), ref, n, gap=1e-3)
    index_report("causal score mode T=%d" % T, hard, soft, idx.numel() // n)
    assert hard == 0
    sel_score = torch.gather(ref.permute(0, 2, 1, 3), -1, idx.cpu().long().clamp_min(0))
    future = idx.cpu().long() * 64 > torch.arange(T).view(1, T, 1, 1)
    assert not (future & (sel_score > 1e-3)).any(), "a block in the query's future was selected with a real score"
    # the module with this mode: forward against the oracle composition on the kernel's own selection
    mod, q2, k2, v2, _ = _module_and_oracle(nsa, 1, 1024, 32, 2, 128, 4, 128, seed=77)
    mod.score_mode = "causal"
    cu = torch.tensor([0, 1024], dtype=torch.int32, device=DEV)
    q2d, k2d, v2d = (_dev(x.reshape(1024, -1, 128)) for x in (q2, k2, v2))
    with torch.no_grad():
        out = mod(q2d, k2d, v2d, cu, 1024)
        ckd, cvd, _ = mod.compressor(k2d, v2d, cu, None)
    sc2 = O.pooled_scores_causal(q2, ckd.float().cpu(), 2, 5, 4, 0, 16, 32)
    idx2 = O.topn_blocks(sc2, 4)
    wg, bg = mod.gating.weight.detach().float().cpu(), mod.gating.bias.detach().float().cpu()
    o_cmp, _ = O.cmp_attention(q2, ckd.float().cpu(), cvd.float().cpu(), 16, 32, True)
    o_slc, _ = O.selected_attention(q2, k2, v2, idx2, None, 64)
    o_swa, _ = O.sliding_window_attention(q2, k2, v2, 128)
    gate = _r(q2 @ wg.t() + bg)
    ref2 = o_slc * gate[..., 0:1] + o_swa * gate[..., 1:2] + o_cmp * gate[..., 2:3]
    # near-tie selections can differ from the oracle's top-n on a few rows: those rows are excluded, the rest must match
    err = (out.view(1, 1024, 32, 128).float().cpu() - ref2).abs().amax((-1, -2))
    assert float((err > 3e-2).float().mean()) < 0.02, "more than 2%% of the rows differ: %s" % err.topk(5).values
    nsa._lib.device_status()


def test_pooled_scores_dump_matches_oracle(nsa):
    """The fused score path (never written to HBM in production) can be dumped for inspection."""
    from nsa_b200 import _lib
    gen = torch.Generator().manual_seed(5)
    B, T, Hq, Hkv, D, block, stride = 1, 1024, 16, 1, 128, 32, 16
    Tc = (T - block) // stride + 1
    q = _r(torch.randn(B, T, Hq, D, generator=gen) * 0.3)
    ck = _r(torch.randn(B, Tc, Hkv, D, generator=gen) * 0.3)
    L = _lib.lib()
    n_pool = L.nsa_pool_out_len(Tc, 5, 4, 0)
    assert n_pool == T // 64
    qd, kd = _dev(q), _dev(ck)
    o = torch.empty_like(qd)
    lse = torch.empty(B, T, Hq, dtype=torch.float32, device=DEV)
    idx = torch.empty(B, T, Hkv, 16, dtype=torch.int32, device=DEV)
    scores = torch.empty(B, Hkv, T, n_pool, dtype=torch.float32, device=DEV)
    _lib.check(L.nsa_cmp_attn_fwd(_lib.ptr(qd), _lib.ptr(kd), _lib.ptr(kd), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(idx),
                                  _lib.ptr(scores), B, T, Tc, Hq, Hkv, D, block, stride, 1, D ** -0.5, 16, 5, 4, 0,
                                  _lib.stream()), "nsa_cmp_attn_fwd")
    ref = O.pooled_scores(q, ck, Hkv, 5, 4, 0)
    _close("pooled scores", scores, ref, atol=2e-3, rtol=1e-2)
    # T = 1024 has exactly 16 pooled blocks, so top-16 selects every block (BASELINE config 1's shape)
    assert (idx.sort(-1)[0].cpu() == torch.arange(16).view(1, 1, 1, 16)).all()
    _lib.device_status()


@pytest.mark.parametrize("D,H,block,stride,lens", [(128, 2, 32, 16, [256, 100, 48, 31]), (64, 3, 64, 16, [200, 64])])
def test_compression_varlen_fwd_bwd(nsa, D, H, block, stride, lens):
    gen = torch.Generator().manual_seed(9 + D)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    x = _r(torch.randn(cu[-1], H, D, generator=gen))
    w = _r(torch.randn(block * D, D, generator=gen) * 0.03)
    xd, wd = _dev(x).requires_grad_(True), _dev(w).requires_grad_(True)
    ck, cv, cu_out = nsa.compression_kv.compress_kv(xd, xd, wd, wd, torch.tensor(cu, dtype=torch.int32, device=DEV),
                                                    stride, block)
    xo, wo = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ry, rcu = O.compress_varlen(xo, wo, cu, block, stride)
    assert cu_out.tolist() == rcu
    _close("y", ck, ry)
    dy = _r(torch.randn(ry.shape, generator=gen))
    ck.backward(_dev(dy))
    (ry * dy).sum().backward()
    _close("dx", xd.grad, xo.grad)
    _close("dw", wd.grad, wo.grad, scaled=True)
    nsa._lib.device_status()


def _module_and_oracle(nsa, B, T, Hq, Hkv, D, n_sel, window, seed, causal=True):
    gen = torch.Generator().manual_seed(seed)
    q = _r(torch.randn(B, T, Hq, D, generator=gen))
    k = _r(torch.randn(B, T, Hkv, D, generator=gen))
    v = _r(torch.randn(B, T, Hkv, D, generator=gen))
    mod = nsa.NSAAttention(D, causal, None, 0.0, selected_block_count=n_sel, sliding_window=window, device=DEV,
                           dtype=torch.bfloat16)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(_r(torch.randn(p.shape, generator=gen) * 0.02))
        mod.gating.bias.copy_(_r(torch.tensor([0.5, 0.4, 0.6])))
    return mod, q, k, v, gen


@pytest.mark.parametrize("D,Hq,Hkv,T,n_sel,window,causal,fused", [(128, 32, 2, 1024, 4, 128, True, False),
                                                                  (64, 16, 1, 640, 3, 64, True, False),
                                                                  (128, 32, 2, 1024, 4, 128, False, False),
                                                                  (128, 32, 2, 1024, 4, 128, True, True),
                                                                  (64, 16, 1, 640, 3, 64, True, True)])
def test_module_forward_backward(nsa, D, Hq, Hkv, T, n_sel, window, causal, fused):
    """``causal`` is the module's constructor flag (default False in the reference, nsa/nsa.py:18): it only changes
    the mask of the compressed branch; selected and sliding-window attention are causal either way."""
    B = 2
    mod, q, k, v, gen = _module_and_oracle(nsa, B, T, Hq, Hkv, D, n_sel, window, seed=31 + D, causal=causal)
    mod.fuse_row_passes = fused      # the fused entry points (nsa_cmp_attn_fwd_gated, nsa_*_bwd_fused) or the streaming kernels
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=DEV)
    qd, kd, vd = (_dev(x.reshape(B * T, *x.shape[2:])).requires_grad_(True) for x in (q, k, v))
    out = mod(qd, kd, vd, cu, T)
    assert out.shape == (B * T, Hq, D)
    # stage 1: compression against the oracle
    ckd, cvd, _ = mod.compressor(kd.detach(), vd.detach(), cu, None)
    wk, bk = mod.compressor.compressor_k.weight.detach().float().cpu(), mod.compressor.compressor_k.bias.detach().float().cpu()
    wv, bv = mod.compressor.compressor_v.weight.detach().float().cpu(), mod.compressor.compressor_v.bias.detach().float().cpu()
    _close("ck", ckd, O.compress_conv(k, wk, bk, 32, 16))
    _close("cv", cvd, O.compress_conv(v, wv, bv, 32, 16))
    # stage 2: indices against the oracle scores on the kernel's compressed keys
    ck_b, cv_b = ckd.float().cpu(), cvd.float().cpu()
    _, idx = nsa.triton_attention.flash_attn_func(qd.detach().view(B, T, Hq, D), ckd, cvd, 16, 32, causal, None, Hkv, 5,
                                                  4, 0, n_sel)
    sc = O.pooled_scores(q, ck_b, Hkv, 5, 4, 0)
    hard, soft = O.index_sets_match(idx.cpu(), sc, n_sel, gap=1e-3)
    index_report("module D=%d T=%d causal=%s" % (D, T, causal), hard, soft, idx.numel() // idx.shape[-1])
    assert hard == 0, "%d rows outside the waiver (%d differ)" % (hard, soft)
    # stage 3: the whole forward and backward with indices fixed to the kernel's
    qo, ko, vo = (x.clone().requires_grad_(True) for x in (q, k, v))
    wk_o, bk_o, wv_o, bv_o = (t.clone().requires_grad_(True) for t in (wk, bk, wv, bv))
    ck_o = O.compress_conv(ko, wk_o, bk_o, 32, 16)
    cv_o = O.compress_conv(vo, wv_o, bv_o, 32, 16)
    ck_o.retain_grad()
    wg_o = mod.gating.weight.detach().float().cpu().requires_grad_(True)
    bg_o = mod.gating.bias.detach().float().cpu().requires_grad_(True)
    o_cmp, _ = O.cmp_attention(qo, ck_o, cv_o, 16, 32, causal)
    o_slc, _ = O.selected_attention(qo, ko, vo, idx.cpu(), None, 64)
    o_swa, _ = O.sliding_window_attention(qo, ko, vo, window)
    gate = qo @ wg_o.t() + bg_o
    ref = o_slc * gate[..., 0:1] + o_swa * gate[..., 1:2] + o_cmp * gate[..., 2:3]
    _close("module output", out.view(B, T, Hq, D), ref)
    do = _r(torch.randn(B, T, Hq, D, generator=gen))
    out.backward(_dev(do.reshape(B * T, Hq, D)))
    (ref * do).sum().backward()
    # dq is the bf16 sum of four bf16 branch gradients (selected, window, compressed, gate), as in the reference's
    # autograd graph: three extra roundings, so 3e-2 on the unit-RMS row
    _close("dq", qd.grad.view(B, T, Hq, D), qo.grad, atol=3e-2, scaled=True)
    _close("dk", kd.grad.view(B, T, Hkv, D), ko.grad, atol=3e-2, scaled=True)
    _close("dv", vd.grad.view(B, T, Hkv, D), vo.grad, scaled=True)
    # parameter gradients sit behind two bf16-rounded gradient stages (branch gradient, then the compression or
    # gate backward summed over every token): 4e-2 on the unit-RMS row
    for name, got, ref_g in (("gating.weight", mod.gating.weight.grad, wg_o.grad),
                             ("gating.bias", mod.gating.bias.grad, bg_o.grad),
                             ("compressor_k.weight", mod.compressor.compressor_k.weight.grad, wk_o.grad),
                             ("compressor_v.weight", mod.compressor.compressor_v.weight.grad, wv_o.grad),
                             ("compressor_v.bias", mod.compressor.compressor_v.bias.grad, bv_o.grad)):
        _close("d " + name, got, ref_g, atol=4e-2, scaled=True)
    # The key-side bias gradient is exactly zero in exact arithmetic (a constant added to every compressed key shifts
    # each score row by a constant); the kernel's value is the sum over B*Tc*Hkv rows of bf16-rounded dCK entries, so it
    # is bounded by that rounding noise: 2^-8 * sqrt(rows) * RMS(dCK).
    assert bk_o.grad.abs().max() < 1e-3
    rows = ck_o.grad.numel() // D
    noise = 2.0 ** -8 * rows ** 0.5 * float(ck_o.grad.square().mean().sqrt())
    got = mod.compressor.compressor_k.bias.grad.float().cpu()
    assert got.abs().max() < 4 * noise, "d compressor_k.bias %.3g exceeds the rounding bound %.3g" % (
        float(got.abs().max()), 4 * noise)
    nsa._lib.device_status()


@pytest.mark.parametrize("D,rows", [(128, 4999), (64, 130)])
def test_gate_projection_and_row_prepass(nsa, D, rows):
    """nsa_gate_fwd / nsa_rowdot3 / nsa_gate_bwd against fp32 torch on the same bf16 inputs (nn.Linear(head_dim, 3) of
    nsa/nsa.py:59,117 and its autograd)."""
    L, P, S = nsa._lib.lib(), nsa._lib.ptr, nsa._lib.stream
    gen = torch.Generator().manual_seed(5 + D)
    q, do, o0, o1, o2, dq0 = (_r(torch.randn(rows, D, generator=gen)) for _ in range(6))
    w = _r(torch.randn(3, D, generator=gen) * 0.1)
    b = _r(torch.randn(3, generator=gen))
    qd, dod, o0d, o1d, o2d, wd, bd = (_dev(x) for x in (q, do, o0, o1, o2, w, b))
    g = [torch.empty(rows, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    nsa._lib.check(L.nsa_gate_fwd(P(qd), P(wd), P(bd), P(g[0]), P(g[1]), P(g[2]), rows, D, S()), "gate_fwd")
    ref_g = q @ w.t() + b
    for x in range(3):
        _close("gate %d" % x, g[x], ref_g[:, x], atol=1e-2)
    delta = [torch.empty(rows, dtype=torch.float32, device=DEV) for _ in range(3)]
    dg = [torch.empty(rows, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    nsa._lib.check(L.nsa_rowdot3(P(o0d), P(o1d), P(o2d), P(dod), P(g[0]), P(g[1]), P(g[2]), P(delta[0]), P(delta[1]),
                                 P(delta[2]), P(dg[0]), P(dg[1]), P(dg[2]), rows, D, S()), "rowdot3")
    for x, o in enumerate((o0, o1, o2)):
        rs = (o * do).sum(-1)
        _close("dgate %d" % x, dg[x], rs, atol=6e-2, rtol=1e-2)
        _close("delta %d" % x, delta[x], rs * g[x].float().cpu(), atol=1e-3, rtol=1e-3)
    dqd = _dev(dq0).clone()
    dw, db = torch.empty(3, D, dtype=torch.bfloat16, device=DEV), torch.empty(3, dtype=torch.bfloat16, device=DEV)
    nb = L.nsa_gate_bwd_workspace_bytes(rows, D)
    ws = torch.empty(nb, dtype=torch.uint8, device=DEV)
    nsa._lib.check(L.nsa_gate_bwd(P(qd), P(dg[0]), P(dg[1]), P(dg[2]), P(wd), P(dqd), P(dw), P(db), P(ws), nb, rows, D,
                                  S()), "gate_bwd")
    dgf = torch.stack([x.float().cpu() for x in dg], -1)        # [rows, 3], the bf16 values the kernel read
    _close("dq", dqd, dq0 + dgf @ w, atol=3e-2)
    _close("dw", dw, dgf.t() @ q, atol=4e-2, scaled=True)
    _close("db", db.view(1, 3), dgf.sum(0).view(1, 3), atol=4e-2, scaled=True)
    nsa._lib.device_status()


# ------------------------------------------------------------------------------------------------------
# full-size properties (BASELINE.json config 2: B=4, T=8192, Hq=64, Hkv=4, D=128, top-16 of 64-key blocks)
# ------------------------------------------------------------------------------------------------------
def _config2_indices(B, T, H, S, BS, gen, device):
    """min(S, t//BS+1) distinct causally valid blocks, always with block 0 and the local block; rest = -1."""
    t = torch.arange(T, device=device)
    nblk = (t // BS + 1).view(1, T, 1, 1)
    NB = T // BS
    r = torch.rand(B, T, H, NB, generator=gen, device=device)
    blk = torch.arange(NB, device=device).view(1, 1, 1, NB)
    r = torch.where(blk < nblk, r, torch.full_like(r, -1.0))
    r = torch.where((blk == 0) | (blk == nblk - 1), torch.full_like(r, 2.0), r)
    top = torch.topk(r, S, dim=-1)
    return torch.where(top.values >= 0, top.indices, torch.full_like(top.indices, -1)).to(torch.int32)


def test_selection_full_size_properties(nsa):
    B, T, Hq, Hkv, D, S, BS = 4, 8192, 64, 4, 128, 16, 64
    gen = torch.Generator(device=DEV).manual_seed(1)
    q = torch.randn(B, T, Hq, D, generator=gen, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, generator=gen, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, T, Hkv, D, generator=gen, device=DEV, dtype=torch.bfloat16)
    idx = _config2_indices(B, T, Hkv, S, BS, gen, DEV)
    ones = torch.ones(B, T, Hq, device=DEV, dtype=torch.bfloat16)
    o = nsa.selection_attention(q, k, v, ones, ones, idx, None, BS, 0)
    o2 = nsa.selection_attention(q, k, v, ones, ones, idx, None, BS, 0)
    assert torch.equal(o, o2), "two runs differ: the kernel is not deterministic"
    # soft-max weights sum to one: with V = 1 every row (all have a valid key here) is exactly 1
    o1 = nsa.selection_attention(q, k, torch.ones_like(v), ones, ones, idx, None, BS, 0)
    assert (o1.float() - 1).abs().max() < 1e-2
    # linearity in V
    v2 = torch.randn_like(v)
    oa = nsa.selection_attention(q, k, (v + v2), ones, ones, idx, None, BS, 0).float()
    ob = nsa.selection_attention(q, k, v2, ones, ones, idx, None, BS, 0).float()
    assert (oa - (o.float() + ob)).abs().max() < 6e-2
    # sampled rows against the oracle
    rows = [(0, 0), (0, 63), (1, 64), (2, 4097), (3, 8191), (1, 1000)]
    kc, vc = k.cpu().float(), v.cpu().float()
    for b, t in rows:
        ref, _ = O.selected_attention(q[b:b + 1, t:t + 1].cpu().float(), kc[b:b + 1], vc[b:b + 1],
                                      idx[b:b + 1, t:t + 1].cpu().long(), None, BS, q_pos=torch.tensor([t]))
        _close("row (%d,%d)" % (b, t), o[b, t], ref[0, 0])
    nsa._lib.device_status()


# ------------------------------------------------------------------------------------------------------
# query shards (context parallelism): the kernels run on a slice of the queries against the whole K/V
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("prefix", [False, True])
def test_query_shards_match_unsharded_run(nsa, prefix):
    """Emulates 2 ranks with the zig-zag layout on one GPU: four query chunks run one after the other through the
    sharded entry points; outputs, selected indices and dQ must equal the unsharded run, dK/dV/dCK/dCV must sum to it.
    With ``prefix`` a chunk is given only the keys up to its own last token (what the context-parallel wrapper
    passes): nothing later can be attended, so the results are the same."""
    from nsa_b200.nsa import _NSACore
    gen = torch.Generator().manual_seed(77)
    B, T, Hq, Hkv, D, n_sel, window = 1, 1024, 32, 2, 128, 4, 128
    Tc = (T - 32) // 16 + 1
    q, k, v = (_dev(_r(torch.randn(B, T, h, D, generator=gen))) for h in (Hq, Hkv, Hkv))
    ck, cv = (_dev(_r(torch.randn(B, Tc, Hkv, D, generator=gen) * 0.5)) for _ in range(2))
    wg = _dev(_r(torch.randn(3, D, generator=gen) * 0.05))
    bg = _dev(_r(torch.tensor([0.5, 0.4, 0.6])))
    do = _dev(_r(torch.randn(B, T, Hq, D, generator=gen)))

    def run(q0, Tq):
        sl = slice(q0, q0 + Tq)
        end = q0 + Tq if prefix else T
        leaves = [t.clone().requires_grad_(True) for t in (q[:, sl].contiguous(), k[:, :end].contiguous(),
                                                           v[:, :end].contiguous(), ck, cv, wg, bg)]
        cfg = (16, 32, True, D ** -0.5, 5, 4, 0, n_sel, 64, window, q0)
        o = _NSACore.apply(*leaves, cfg)
        o.backward(do[:, sl].contiguous())
        grads = [t.grad for t in leaves]
        for i in (1, 2):     # dk, dv of a key prefix: zero beyond it
            grads[i] = torch.cat([grads[i], grads[i].new_zeros(B, T - end, Hkv, D)], 1)
        return o.detach(), grads

    o_full, g_full = run(0, T)
    chunk = T // 4
    o_parts, dq_parts = {}, {}
    sums = [torch.zeros_like(t, dtype=torch.float32) for t in g_full[1:]]
    for cid in (0, 3, 1, 2):                      # rank 0 owns chunks 0 and 3, rank 1 owns 1 and 2
        o, grads = run(cid * chunk, chunk)
        o_parts[cid], dq_parts[cid] = o, grads[0]
        for s_, g_ in zip(sums, grads[1:]):
            s_ += g_.float()
    assert torch.equal(torch.cat([o_parts[c] for c in range(4)], 1), o_full)
    assert torch.equal(torch.cat([dq_parts[c] for c in range(4)], 1), g_full[0])
    for name, s_, ref in zip(("dk", "dv", "dck", "dcv", "d gating.weight", "d gating.bias"), sums, g_full[1:]):
        _close(name + " summed over shards", s_.reshape(-1, s_.shape[-1]), ref.reshape(-1, ref.shape[-1]), atol=4e-2,
               scaled=True)
    nsa._lib.device_status()


def test_module_step_is_bit_reproducible(nsa):
    """Twelve forward + backward passes of the module on the same inputs must agree bit for bit (no atomics, no
    scheduling-dependent result).  The module's own selection leaves many queries with zero to two visible blocks,
    which is the case that exposed a stale-tile race in the selected-attention producer/consumer hand-over."""
    torch.manual_seed(0)
    B, T, Hq, Hkv, D, S, W = 2, 1024, 32, 2, 128, 4, 128
    q = torch.randn(B * T, Hq, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B * T, Hkv, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B * T, Hkv, D, device=DEV, dtype=torch.bfloat16)
    do = torch.randn(B * T, Hq, D, device=DEV, dtype=torch.bfloat16)
    mod = nsa.NSAAttention(D, True, None, 0.0, selected_block_count=S, sliding_window=W, device=DEV, dtype=torch.bfloat16)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=DEV)
    ref = None
    for it in range(12):
        qd, kd, vd = (x.clone().requires_grad_(True) for x in (q, k, v))
        for p in mod.parameters():
            p.grad = None
        out = mod(qd, kd, vd, cu, T)
        out.backward(do)
        torch.randn(1 << (10 + it), device=DEV).sum()           # unrelated work of varying length between passes
        cur = {"out": out.detach(), "dq": qd.grad, "dk": kd.grad, "dv": vd.grad}
        cur.update({"d " + n: p.grad.clone() for n, p in mod.named_parameters()})
        if ref is None:
            ref = {n: t.clone() for n, t in cur.items()}
        else:
            for n in cur:
                assert torch.equal(cur[n], ref[n]), "%s differs between pass 0 and pass %d" % (n, it)
    nsa._lib.device_status()


def test_decode_rows_match_oracle(nsa):
    """One new token per sequence against a packed K/V cache of ragged lengths (BASELINE config 5's shape in small)."""
    from nsa_b200.decode import compress_cache, nsa_decode
    gen = torch.Generator().manual_seed(404)
    Hq, Hkv, D, n_sel, window = 32, 2, 128, 3, 64
    lens = [300, 1061, 2048, 517, 20, 40, 95]      # incl. shorter than one compression block and not multiples of 64
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    q = _r(torch.randn(len(lens), Hq, D, generator=gen))
    k = _r(torch.randn(cu[-1], Hkv, D, generator=gen))
    v = _r(torch.randn(cu[-1], Hkv, D, generator=gen))
    mod = nsa.NSAAttention(D, True, selected_block_count=n_sel, sliding_window=window, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(_r(torch.randn(p.shape, generator=gen) * 0.02))
        mod.gating.bias.copy_(_r(torch.tensor([0.5, 0.4, 0.6])))
    kd, vd = _dev(k), _dev(v)
    cache = compress_cache(mod, kd, vd, cu)
    o = nsa_decode(mod, _dev(q), kd, vd, cu, cache=cache)
    o2 = nsa_decode(mod, _dev(q), kd, vd, torch.tensor(cu, dtype=torch.int32, device=DEV))   # re-compressing path
    assert torch.equal(o, o2)
    ck, cv, _, cu_c = cache
    wk, bk = (t.detach().float().cpu() for t in (mod.compressor.compressor_k.weight, mod.compressor.compressor_k.bias))
    wv, bv = (t.detach().float().cpu() for t in (mod.compressor.compressor_v.weight, mod.compressor.compressor_v.bias))
    wg, bg = mod.gating.weight.detach().float().cpu(), mod.gating.bias.detach().float().cpu()
    for i, L in enumerate(lens):
        ks, vs = k[cu[i]:cu[i + 1]], v[cu[i]:cu[i + 1]]
        if L >= 32:
            _close("ck of sequence %d" % i, ck[cu_c[i]:cu_c[i + 1]], O.compress_conv(ks.unsqueeze(0), wk, bk, 32, 16)[0])
        # the row itself, evaluated by the oracle on the kernel's compressed cache (bf16) so that near-tie selections
        # do not confound the comparison; gates as the bf16 tensors the module produces
        ref, ref_idx, sc = O.nsa_decode_row(q[i], ks, vs, wk, bk, wv, bv, wg, bg, n_sel=n_sel, window=window,
                                            ck=ck[cu_c[i]:cu_c[i + 1]].cpu(), cv=cv[cu_c[i]:cu_c[i + 1]].cpu(),
                                            return_scores=True)
        _close("decode row %d (L=%d)" % (i, L), o[i], ref, atol=3e-2)
    nsa._lib.device_status()


def test_decode_cache_extension(nsa):
    """Appending tokens: the extended cache equals a cache compressed from scratch, and a decode step on it equals the
    stateless step (only the compressed positions completed by the new tokens are computed)."""
    from nsa_b200.decode import compress_cache, extend_compress_cache, nsa_decode
    gen = torch.Generator().manual_seed(405)
    Hq, Hkv, D = 32, 2, 128
    old, grow = [300, 47, 31, 1024], [1, 17, 40, 0]
    new = [a + b for a, b in zip(old, grow)]
    cu_old, cu_new = [0], [0]
    for a, b in zip(old, new):
        cu_old.append(cu_old[-1] + a)
        cu_new.append(cu_new[-1] + b)
    k_new = _dev(_r(torch.randn(cu_new[-1], Hkv, D, generator=gen)))
    v_new = _dev(_r(torch.randn(cu_new[-1], Hkv, D, generator=gen)))
    take = torch.cat([torch.arange(cu_new[i], cu_new[i] + old[i]) for i in range(len(old))]).to(DEV)
    k_old, v_old = k_new[take].contiguous(), v_new[take].contiguous()
    mod = nsa.NSAAttention(D, True, selected_block_count=3, sliding_window=64, device=DEV, dtype=torch.bfloat16)
    cache = compress_cache(mod, k_old, v_old, cu_old)
    ext = extend_compress_cache(mod, cache, k_new, v_new, cu_new)
    full = compress_cache(mod, k_new, v_new, cu_new)
    assert ext.cu_c == full.cu_c
    # (the appended positions come from the equal-length tcgen05 kernel, the from-scratch cache from the ragged one: the
    # same contraction summed in a different order, so entries may differ by one bf16 rounding step)
    _close("extended ck", ext.ck, full.ck, atol=1.6e-2, rtol=0)
    _close("extended cv", ext.cv, full.cv, atol=1.6e-2, rtol=0)
    q = _dev(_r(torch.randn(len(old), Hq, D, generator=gen)))
    _close("decode on the extended cache", nsa_decode(mod, q, k_new, v_new, cu_new, cache=ext),
           nsa_decode(mod, q, k_new, v_new, cu_new))
    nsa._lib.device_status()
