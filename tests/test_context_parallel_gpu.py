"""Context-parallel NSA on two GPUs against the single-GPU module: outputs, input gradients and (all-reduced)
parameter gradients; rank 0 also checks the single-GPU run it compares with against the CPU oracle (output, dq, dk,
dv at T=4096: two key tiles of compressed keys), so the sharded run is tied to the oracle and not only to the same
kernels.  Skipped when fewer than two GPUs are visible.  Every rank appends its verdict to the file named by
NSA_CP_TEST_LOG, if set."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import nsa_b200
    from nsa_b200.context_parallel import chunk_layout, context_parallel_forward
    B, T, Hq, Hkv, D = 1, 4096, 32, 2, 128
    gen = torch.Generator().manual_seed(5)
    q, k, v, do = (torch.randn(B, T, h, D, generator=gen).to(dev, torch.bfloat16) for h in (Hq, Hkv, Hkv, Hq))
    mod = nsa_b200.NSAAttention(D, True, selected_block_count=8, sliding_window=256, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(torch.randn(p.shape, generator=gen) * 0.02)
    layout = chunk_layout(world, True)[rank]
    cl = T // (2 * world)
    take = lambda x: torch.cat([x[:, c * cl:(c + 1) * cl] for c in layout], 1).contiguous()
    ql, kl, vl = (take(x).requires_grad_(True) for x in (q, k, v))
    o = context_parallel_forward(mod, ql, kl, vl, None, zigzag=True)
    o.backward(take(do))
    pg = [p.grad.clone() for p in mod.parameters()]
    for g in pg:
        dist.all_reduce(g)
    # single-GPU reference on this rank's device
    for p in mod.parameters():
        p.grad = None
    qf, kf, vf = (x.reshape(B * T, -1, D).clone().requires_grad_(True) for x in (q, k, v))
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    of = mod(qf, kf, vf, cu, T)
    of.backward(do.reshape(B * T, Hq, D))

    def close(a, b, atol, scaled=True):
        a, b = a.float(), b.float()
        s = b.square().mean(-1, keepdim=True).sqrt().clamp_min(1.0) if scaled else 1.0
        return bool((((a - b) / s).abs() <= atol + 1e-2 * (b / s).abs()).all())

    # (the gate GEMM runs on differently shaped inputs in the two runs, so outputs agree to rounding, not bitwise)
    checks = {
        "o": close(o, take(of.view(B, T, Hq, D)), 2e-2, scaled=False),
        "dq": close(ql.grad, take(qf.grad.view(B, T, Hq, D)), 3e-2),
        "dk": close(kl.grad, take(kf.grad.view(B, T, Hkv, D)), 3e-2),
        "dv": close(vl.grad, take(vf.grad.view(B, T, Hkv, D)), 3e-2),
    }
    for (name, _), g, p in zip(mod.named_parameters(), pg, mod.parameters()):
        if name == "compressor.compressor_k.bias":
            continue   # exactly zero in exact arithmetic; both runs hold only bf16 rounding noise of dCK
        checks["d " + name] = close(g, p.grad, 4e-2)
    if rank == 0:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from oracle import nsa_oracle as O
        qc, kc, vc, dc = (x.float().cpu() for x in (q, k, v, do))
        ckd, cvd, _ = mod.compressor(kf.detach(), vf.detach(), cu, None)
        _, idx = nsa_b200.triton_attention.flash_attn_func(qf.detach().view(B, T, Hq, D), ckd, cvd, 16, 32, True, None, Hkv,
                                                           5, 4, 0, 8)
        wk, bk, wv, bv, wg, bg = (t.detach().float().cpu() for t in (
            mod.compressor.compressor_k.weight, mod.compressor.compressor_k.bias, mod.compressor.compressor_v.weight,
            mod.compressor.compressor_v.bias, mod.gating.weight, mod.gating.bias))
        qo, ko, vo = (x.clone().requires_grad_(True) for x in (qc, kc, vc))
        ck_o, cv_o = O.compress_conv(ko, wk, bk, 32, 16), O.compress_conv(vo, wv, bv, 32, 16)
        refs = []
        for a_ in range(0, T, 512):
            b_ = a_ + 512
            pos = torch.arange(a_, b_)
            o_cmp, _ = O.cmp_attention(qo[:, a_:b_], ck_o, cv_o, 16, 32, True, q_pos=pos)
            o_slc, _ = O.selected_attention(qo[:, a_:b_], ko, vo, idx.cpu()[:, a_:b_], None, 64, q_pos=pos)
            o_swa, _ = O.sliding_window_attention(qo[:, a_:b_], ko, vo, 256, q0=a_)
            gate = qo[:, a_:b_] @ wg.t() + bg
            ref = o_slc * gate[..., 0:1] + o_swa * gate[..., 1:2] + o_cmp * gate[..., 2:3]
            (ref * dc[:, a_:b_]).sum().backward(retain_graph=True)
            refs.append(ref.detach())
        checks["single-GPU o vs oracle"] = close(of.view(B, T, Hq, D).cpu(), torch.cat(refs, 1), 2e-2, scaled=False)
        checks["single-GPU dq vs oracle"] = close(qf.grad.view(B, T, Hq, D).cpu(), qo.grad, 3e-2)
        checks["single-GPU dk vs oracle"] = close(kf.grad.view(B, T, Hkv, D).cpu(), ko.grad, 3e-2)
        checks["single-GPU dv vs oracle"] = close(vf.grad.view(B, T, Hkv, D).cpu(), vo.grad, 3e-2)
    ok = all(checks.values())
    if not ok:
        print("rank", rank, "failed:", [n for n, c in checks.items() if not c], flush=True)
    log = os.environ.get("NSA_CP_TEST_LOG")
    if log:
        with open(log, "a") as f:
            f.write("rank %d of %d: %s  %s\n" % (rank, world, "PASS" if ok else "FAIL", sorted(checks.items())))
    nsa_b200._lib.device_status()
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_rank_context_parallel_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, 29641, ret), nprocs=2, join=True)
    assert all(ret[r] for r in range(2)), dict(ret)
