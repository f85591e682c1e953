"""Pins the CPU oracle (oracle/nsa_oracle.py) to outputs of the reference's own functions
stored under tests/golden/ (see tests/golden/make_golden.py for how they were made)."""
import os

import numpy as np
import pytest
import torch

import cases
from oracle import nsa_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    d = np.load(os.path.join(GOLD, name + ".npz"))
    return {k: torch.from_numpy(np.asarray(d[k])) for k in d.files}


def _close(a, b, tol=2e-5):
    torch.testing.assert_close(a.float(), b.float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("name", cases.CMP_CASES)
def test_cmp_attention_matches_reference(name):
    c, g = cases.cmp_case(name), _load(name)
    assert abs(cases.checksum(c["q"], c["ck"], c["cv"], c["do"]) - float(g["chk"])) < 1e-6
    q = c["q"].clone().requires_grad_(True)
    ck = c["ck"].clone().requires_grad_(True)
    cv = c["cv"].clone().requires_grad_(True)
    o, lse = O.cmp_attention(q, ck, cv, c["stride"], c["block"], causal=True)
    _close(o, g["o"])
    (o * c["do"]).sum().backward()
    _close(q.grad, g["dq"], 1e-4)
    _close(ck.grad, g["dck"], 1e-4)
    _close(cv.grad, g["dcv"], 1e-4)
    # rows before the first visible compressed position are zero with lse = -inf
    assert torch.isinf(lse[:, :c["block"]]).all() and (o[:, :c["block"]] == 0).all()
    sc = O.pooled_scores(c["q"], c["ck"], c["Hkv"], c["pool_kernel"], c["pool_stride"], c["pool_pad"])
    hard, soft = O.index_sets_match(g["idx"].long(), sc, c["n"], gap=1e-6)
    assert hard == 0
    # and the oracle's own top-n agrees with itself under the lower-index tie rule
    idx = O.topn_blocks(sc, c["n"])
    assert O.index_sets_match(idx, sc, c["n"], gap=0.0) == (0, 0)


@pytest.mark.parametrize("name", cases.SEL_CASES)
def test_selected_and_window_match_reference(name):
    c, g = cases.sel_case(name), _load(name)
    assert abs(cases.checksum(c["q"], c["k"], c["v"], c["do"]) - float(g["chk"])) < 1e-6
    q = c["q"].clone().requires_grad_(True)
    k = c["k"].clone().requires_grad_(True)
    v = c["v"].clone().requires_grad_(True)
    o = O.parallel_nsa(q, k, v, c["g_slc"], c["g_swa"], c["idx"], c["counts"], c["block_size"],
                       c["window"])
    _close(o, g["o"])
    if c["window"] > 0:
        (o * c["do"]).sum().backward()
        _close(q.grad, g["dq"], 1e-4)
        _close(k.grad, g["dk"], 1e-4)
        # the reference's dv carries NaN at the keys gathered by its two empty-selection rows
        # (its own test overwrites such entries, tests/test_parallel_nsa.py:216-221); compare
        # everywhere else
        ok = ~torch.isnan(g["dv"])
        assert ok.float().mean() > 0.7
        _close(torch.where(ok, v.grad, torch.zeros_like(v.grad)), torch.nan_to_num(g["dv"], nan=0.0), 1e-4)


@pytest.mark.parametrize("name", cases.COMPRESS_CASES)
def test_compression_matches_reference(name):
    c, g = cases.compress_case(name), _load(name)
    assert abs(cases.checksum(c["x"], c["w"], c["conv_w"], c["conv_b"]) - float(g["chk"])) < 1e-6
    x = c["x"].clone().requires_grad_(True)
    w = c["w"].clone().requires_grad_(True)
    y, cu_out = O.compress_varlen(x, w, c["cu"], c["block"], c["stride"])
    _close(y, g["y"], 1e-4)
    n = O.compressed_len_varlen(c["T"], c["block"], c["stride"])
    assert cu_out == [n * i for i in range(c["B"] + 1)]
    tgt = torch.sin(torch.arange(y.numel(), dtype=torch.float32)).reshape(y.shape)
    (y * tgt).sum().backward()
    _close(x.grad, g["dx"], 1e-4)
    _close(w.grad, g["dw"], 1e-4)
    H, D = c["x"].shape[1:]
    xb = c["x"].reshape(c["B"], c["T"], H, D)
    _close(O.compress_conv(xb, c["conv_w"], c["conv_b"], c["block"], c["stride"]), g["conv_k"], 1e-4)
    _close(O.compress_conv(xb * 0.5, c["conv_w"].flip(0), c["conv_b"].flip(0), c["block"],
                           c["stride"]), g["conv_v"], 1e-4)
    assert g["conv_k"].shape[1] == O.compressed_len_conv(c["T"], c["block"], c["stride"])


def test_pool_matches_torch_avg_pool():
    """The restated pooling equals torch's avg_pool1d(ceil_mode=True) for both paddings."""
    g = torch.Generator().manual_seed(7)
    for Tc, k, s, p in [(63, 5, 4, 0), (511, 5, 4, 0), (61, 5, 4, 2), (9, 5, 4, 2), (15, 5, 4, 0)]:
        x = torch.rand(3, Tc, generator=g)
        ref = torch.nn.functional.avg_pool1d(x.unsqueeze(0), k, s, p, True)[0]
        nb = O.pool_out_len(Tc, k, s, p)
        assert ref.shape[-1] == nb
        mine = torch.stack([x[:, max(b * s - p, 0):min(min(b * s - p + k, Tc + p), Tc)].sum(-1)
                            / (min(b * s - p + k, Tc + p) - (b * s - p)) for b in range(nb)], -1)
        _close(mine, ref, 1e-6)


def test_decode_row_equals_last_row_of_full_forward():
    g = torch.Generator().manual_seed(11)
    T, Hq, Hkv, D = 320, 16, 1, 16
    q = torch.randn(1, T, Hq, D, generator=g)
    k = torch.randn(1, T, Hkv, D, generator=g)
    v = torch.randn(1, T, Hkv, D, generator=g)
    wk, wv = (torch.randn(D, D, 32, generator=g) * 0.05 for _ in range(2))
    bk, bv = (torch.randn(D, generator=g) * 0.05 for _ in range(2))
    wg, bg = torch.randn(3, D, generator=g) * 0.1, torch.randn(3, generator=g) * 0.1
    full = O.nsa_forward(q, k, v, wk, bk, wv, bv, wg, bg, n_sel=3, window=64)
    row, _ = O.nsa_decode_row(q[0, -1], k[0], v[0], wk, bk, wv, bv, wg, bg, n_sel=3, window=64)
    _close(row, full[0, -1], 1e-4)


def test_causal_scores_restatement_properties():
    """pooled_scores_causal (no counterpart in the reference): only visible compressed positions carry weight, every
    row's probabilities sum to the number of heads in the group, and the pooling is the same as pooled_scores'."""
    import torch
    from oracle import nsa_oracle as O
    gen = torch.Generator().manual_seed(3)
    B, T, Hq, Hkv, D, block, stride = 1, 320, 4, 2, 16, 32, 16
    Tc = (T - block) // stride + 1
    q, ck = torch.randn(B, T, Hq, D, generator=gen), torch.randn(B, Tc, Hkv, D, generator=gen)
    sc = O.pooled_scores_causal(q, ck, Hkv, 5, 4, 0, stride, block)
    nb = sc.shape[-1]
    for t in (0, 31, 32, 100, 319):
        nvis = 0 if t < block else min(Tc, (t - block) // stride + 1)
        first_dead = (nvis + 3) // 4          # pooled block b covers positions 4b .. 4b+4
        assert float(sc[0, :, t, first_dead:].abs().max()) == 0.0 if first_dead < nb else True
    # un-pool: with kernel 5 / stride 4 position 4b is shared by blocks b-1 and b; check against a direct evaluation
    s = torch.einsum("bthd,bshd->bhts", q, ck.repeat_interleave(Hq // Hkv, 2)) * D ** -0.5
    masked = torch.arange(Tc).unsqueeze(0) * stride + block > torch.arange(T).unsqueeze(1)
    p = torch.softmax(s.masked_fill(masked, float("-inf")), -1).nan_to_num(0.0)
    p = p.reshape(B, Hkv, Hq // Hkv, T, Tc).sum(2)
    direct = torch.stack([p[..., 4 * b:min(4 * b + 5, Tc)].sum(-1) / (min(4 * b + 5, Tc) - 4 * b) for b in range(nb)], -1)
    assert torch.allclose(sc, direct, atol=1e-6)
