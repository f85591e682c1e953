"""Generate the golden fixtures of this directory by running the REFERENCE's own functions.

Usage (only where the reference checkout is available):

    python tests/golden/make_golden.py /path/to/reference

The reference is loaded by file path: ``nsa/torch_attention.py`` (``attention_ref``),
``tests/test_parallel_nsa.py`` (``naive_nsa``), ``tests/test_compression_kv_bwd.py``
(``compute_reference_kv``) and ``nsa/compression_kv.py`` (``KVCompressor``).  Nothing of the
reference is copied here; only its outputs on the seeded inputs of ``cases.py`` are stored.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root):
    torch.manual_seed(0)
    # a stub ``nsa`` package so the reference test file imports without its Triton kernels
    stub = types.ModuleType("nsa")
    stub.selection_attention = None
    sys.modules["nsa"] = stub
    ta = _load(os.path.join(ref_root, "nsa", "torch_attention.py"), "ref_torch_attention")
    pn = _load(os.path.join(ref_root, "tests", "test_parallel_nsa.py"), "ref_parallel_nsa")
    ck_mod = _load(os.path.join(ref_root, "nsa", "compression_kv.py"), "ref_compression_kv")
    stub_ck = types.ModuleType("nsa.compression_kv")
    stub_ck.compress_kv = None
    stub_ck.calc_compressed_len = ck_mod.calc_compressed_len
    sys.modules["nsa.compression_kv"] = stub_ck
    src = open(os.path.join(ref_root, "tests", "test_compression_kv_bwd.py")).read()
    # the reference file ends by calling main() on CUDA; load only its function definitions
    ns = {}
    exec(compile(src.split("def main()")[0].replace('DEVICE = "cuda"', 'DEVICE = "cpu"'),
                 "ref_test_compression_kv_bwd", "exec"), ns)
    compute_reference_kv = ns["compute_reference_kv"]

    out = {}
    # ---- compressed attention + indices: attention_ref -----------------------------------
    for name in cases.CMP_CASES:
        c = cases.cmp_case(name)
        q = c["q"].clone().requires_grad_(True)
        ck = c["ck"].clone().requires_grad_(True)
        cv = c["cv"].clone().requires_grad_(True)
        G = q.shape[2] // ck.shape[2]
        ckr = ck.repeat_interleave(G, dim=2)
        cvr = cv.repeat_interleave(G, dim=2)
        o, idx = ta.attention_ref(q, ckr, cvr, c["stride"], c["block"], causal=True, upcast=True,
                                  pool_num_kv_head=c["Hkv"], pool_kernel_size=c["pool_kernel"],
                                  pool_stride=c["pool_stride"], pool_padding=c["pool_pad"],
                                  select_block_count=c["n"])
        (o * c["do"]).sum().backward()
        out[name] = dict(o=o, idx=idx, dq=q.grad, dck=ck.grad, dcv=cv.grad,
                         chk=cases.checksum(c["q"], c["ck"], c["cv"], c["do"]))
    # ---- selected / sliding window: naive_nsa ----------------------------------------------
    for name in cases.SEL_CASES:
        c = cases.sel_case(name)
        q = c["q"].clone().requires_grad_(True)
        k = c["k"].clone().requires_grad_(True)
        v = c["v"].clone().requires_grad_(True)
        ref = pn.naive_nsa(q=q, k=k, v=v, g_slc=c["g_slc"], g_swa=c["g_swa"], block_indices=c["idx"],
                           block_counts=c["counts"], block_size=c["block_size"],
                           window_size=c["window"])
        if c["window"] == 0:
            # the reference test's own convention for rows with an empty selection
            ref = torch.nan_to_num(ref, nan=0.0)
            out[name] = dict(o=ref, chk=cases.checksum(c["q"], c["k"], c["v"], c["do"]))
        else:
            (ref * c["do"]).sum().backward()
            out[name] = dict(o=ref, dq=q.grad, dk=k.grad, dv=v.grad,
                             chk=cases.checksum(c["q"], c["k"], c["v"], c["do"]))
    # ---- compression -------------------------------------------------------------------------
    for name in cases.COMPRESS_CASES:
        c = cases.compress_case(name)
        x = c["x"].clone().requires_grad_(True)
        w = c["w"].clone().requires_grad_(True)
        y = compute_reference_kv(x, w, torch.tensor(c["cu"]), c["block"], c["stride"])
        tgt = torch.sin(torch.arange(y.numel(), dtype=torch.float32)).reshape(y.shape)
        (y * tgt).sum().backward()
        comp = ck_mod.KVCompressor(c["stride"], c["block"], x.shape[-1], "cpu", torch.float32)
        with torch.no_grad():
            comp.compressor_k.weight.copy_(c["conv_w"])
            comp.compressor_k.bias.copy_(c["conv_b"])
            comp.compressor_v.weight.copy_(c["conv_w"].flip(0))
            comp.compressor_v.bias.copy_(c["conv_b"].flip(0))
        yk, yv, _ = comp(c["x"], c["x"] * 0.5, torch.tensor(c["cu"]), None)
        out[name] = dict(y=y, dx=x.grad, dw=w.grad, conv_k=yk, conv_v=yv,
                         chk=cases.checksum(c["x"], c["w"], c["conv_w"], c["conv_b"]))
    for name, d in out.items():
        arrs = {}
        for key, val in d.items():
            if torch.is_tensor(val):
                val = val.detach()
                arrs[key] = val.numpy().astype(np.int32 if val.dtype == torch.long else np.float32)
            else:
                arrs[key] = np.float64(val)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrs)
        print(name, {k: getattr(a, "shape", ()) for k, a in arrs.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference>")
    main(sys.argv[1])
