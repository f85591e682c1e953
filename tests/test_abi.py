"""CPU-side checks of the C ABI: the shared library builds for sm_100a, loads, exports every symbol that
include/nsa_b200.h declares, and rejects bad arguments without touching a GPU."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "nsa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nsa_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_loads_and_exports_header_symbols():
    import __graft_entry__ as g
    g.build()
    from nsa_b200 import _lib
    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert len(names) >= 14
    for n in names:
        assert hasattr(handle, n), "libnsa_b200.so does not export %s" % n
    assert sorted(_lib.SIGNATURES) == names, "python binding and header disagree"
    assert _lib.lib().nsa_abi_version() == 1


def test_argument_checks_need_no_gpu():
    from nsa_b200 import _lib
    L = _lib.lib()
    assert L.nsa_pool_out_len(511, 5, 4, 0) == 128 and L.nsa_pool_out_len(4095, 5, 4, 0) == 1024
    assert L.nsa_pool_out_len(63, 5, 4, 0) == 16 and L.nsa_pool_out_len(61, 5, 4, 2) == 16
    rc = L.nsa_sel_swa_fwd(None, None, None, None, 0, None, None, None, None, None, None, None, None, None, None,
                           1, 64, 16, 1, 128, 4, 64, 0, 1.0, None)
    assert rc < 0 and b"null" in L.nsa_last_error()
    one = ctypes.c_void_p(16)
    rc = L.nsa_cmp_attn_fwd(one, one, one, one, one, None, None, 1, 64, 3, 24, 2, 128, 32, 16, 1, 1.0, 0, 0, 0, 0, None)
    assert rc == -3 and b"multiple of 16" in L.nsa_last_error()
    rc = L.nsa_cmp_attn_fwd(one, one, one, one, one, None, None, 1, 64, 3, 16, 1, 96, 32, 16, 1, 1.0, 0, 0, 0, 0, None)
    assert rc == -2 and b"head_dim" in L.nsa_last_error()
    base = L.nsa_sel_swa_bwd_workspace_bytes(8, 8192, 4, 16, 64)
    assert base > 8 * 4 * 8192 * 16 * 4
    # the larger workspaces add one [16 heads x D] bf16 tile per (token, kv head, slot): B*T*Hq*S*D*2 bytes, plus the
    # inverse index (and, for the forward, 16 (max, sum) pairs per tile)
    tiles = 8 * 8192 * 64 * 16 * 128 * 2
    dq = L.nsa_sel_swa_bwd_workspace_bytes_dq(8, 8192, 8192, 64, 4, 128, 16, 64)
    fw = L.nsa_sel_swa_fwd_workspace_bytes(8, 8192, 8192, 64, 4, 128, 16, 64)
    assert base + tiles < dq < base + tiles + (1 << 28) and dq < fw < dq + (1 << 30)
    # a query shard needs tiles for its own rows only
    assert L.nsa_sel_swa_fwd_workspace_bytes(1, 65536, 8192, 64, 4, 128, 16, 64) < fw
    from nsa_b200 import _lib as lib_mod
    assert lib_mod.sel_swa_fwd_workspace_bytes(1, 512, 512, 16, 1, 64, 4, 64) == 0      # head_dim 64: query-major kernel
    assert lib_mod.sel_swa_fwd_workspace_bytes(1, 512, 512, 16, 1, 128, 4, 32) == 0     # 32-key blocks: query-major kernel
    assert L.nsa_kernel_launch_count() == 0


def test_package_surface_matches_the_reference():
    import inspect
    import nsa_b200 as nsa
    assert nsa.selection_attention is nsa.selection_attn.parallel_nsa
    sig = inspect.signature(nsa.selection_attention)
    assert list(sig.parameters) == ["q", "k", "v", "g_slc", "g_swa", "block_indices", "block_counts", "block_size",
                                    "window_size", "scale", "cu_seqlens", "head_first"]
    sig = inspect.signature(nsa.NSAAttention.__init__)
    assert list(sig.parameters)[1:] == ["head_dim", "causal", "softmax_scale", "attention_dropout", "deterministic",
                                        "compression_stride", "compression_block", "selection_block",
                                        "selected_block_count", "sliding_window", "device", "dtype"]
    m = nsa.NSAAttention(64, True)
    assert set(m.state_dict()) == {"compressor.compressor_k.weight", "compressor.compressor_k.bias",
                                   "compressor.compressor_v.weight", "compressor.compressor_v.bias", "gating.weight",
                                   "gating.bias"}
    assert tuple(m.compressor.compressor_k.weight.shape) == (64, 64, 32)
    assert (m.pool_kernel_size, m.pool_stride, m.pool_padding) == (5, 4, 0)
    assert nsa.compression_kv.calc_compressed_len(1024, 16, 32) == 62
    v = nsa.compression_kv.KVCompressorVarlen(16, 32, 64, None, None)
    assert tuple(v.k_weight.shape) == (32 * 64, 64)


def test_no_cpu_fallback():
    import pytest
    import torch
    import nsa_b200 as nsa
    q = torch.zeros(1, 64, 16, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        nsa.selection_attention(q, q[:, :, :1], q[:, :, :1], q[..., 0], q[..., 0],
                                torch.zeros(1, 64, 1, 2, dtype=torch.long))
