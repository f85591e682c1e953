"""ctypes binding of libnsa_b200.so (the C ABI of include/nsa_b200.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libnsa_b200.so")

_c_void_p, _c_int, _c_float, _c_size_t, _c_ll = (ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t,
                                                  ctypes.c_longlong)
P, I, F, Z, L = _c_void_p, _c_int, _c_float, _c_size_t, _c_ll

# name -> (restype, argtypes); mirrors include/nsa_b200.h declaration by declaration
SIGNATURES = {
    "nsa_abi_version": (I, []),
    "nsa_last_error": (ctypes.c_char_p, []),
    "nsa_device_status": (I, []),
    "nsa_kernel_launch_count": (L, []),
    "nsa_compress_fwd": (I, [P, P, P, P, P, P, I, I, I, I, I, I, P]),
    "nsa_compress_fwd_uniform": (I, [P, P, P, P, I, I, I, I, I, I, P]),
    "nsa_compress_bwd": (I, [P, P, P, P, P, P, P, Z, P, P, I, I, I, I, I, I, I, P]),
    "nsa_compress_bwd_workspace_bytes": (Z, [I, I, I, I]),
    "nsa_compress_bwd_noalloc": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P]),
    "nsa_cmp_attn_fwd": (I, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, I, I, P]),
    "nsa_pool_out_len": (I, [I, I, I, I]),
    "nsa_cmp_attn_fwd_gated": (I, [P] * 12 + [I, I, I, I, I, I, I, I, I, F, I, I, I, I, I, I, I, P]),
    "nsa_cmp_attn_bwd": (I, [P, P, P, P, P, P, P, P, I, P, P, P, Z, I, I, I, I, I, I, I, I, I, F, P]),
    "nsa_cmp_attn_bwd_workspace_bytes": (Z, [I, I, I, I, I]),
    "nsa_sel_swa_fwd": (I, [P, P, P, P, I, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P]),
    "nsa_sel_swa_bwd": (I, [P, P, P, P, I, P, P, P, P, P, P, P, P, P, P, I, P, P, P, Z, I, I, I, I, I, I, I, I, F, P]),
    "nsa_sel_swa_bwd_workspace_bytes": (Z, [I, I, I, I, I]),
    "nsa_sel_swa_bwd_workspace_bytes_dq": (Z, [I, I, I, I, I, I, I, I]),
    "nsa_cmp_attn_fwd_sharded": (I, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, I, I, I, I, P]),
    "nsa_cmp_attn_bwd_sharded": (I, [P, P, P, P, P, P, P, P, I, P, P, P, Z, I, I, I, I, I, I, I, I, I, F, I, I, P]),
    "nsa_sel_swa_fwd_sharded": (I, [P, P, P, P, I, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P]),
    "nsa_sel_swa_fwd_ws": (I, [P, P, P, P, I, P, P, P, P, P, P, P, P, P, P, P, Z, I, I, I, I, I, I, I, I, F, I, I, P]),
    "nsa_sel_swa_fwd_workspace_bytes": (Z, [I, I, I, I, I, I, I, I]),
    "nsa_sel_swa_bwd_sharded": (I, [P, P, P, P, I, P, P, P, P, P, P, P, P, P, P, I, P, P, P, Z, I, I, I, I, I, I, I, I,
                                    F, I, I, P]),
    "nsa_sel_swa_bwd_fused": (I, [P, P, P, P, I, P] + [P] * 11 + [P, I, P, P, P, Z, I, I, I, I, I, I, I, I, F, I, I, P]),
    "nsa_cmp_attn_bwd_fused": (I, [P] * 10 + [I, P, P, P, Z, I, I, I, I, I, I, I, I, I, F, I, I, P]),
    "nsa_gather_probe": (I, [P, P, P, I, I, I, I, I, I, I, I, P]),
    "nsa_decode_fwd": (I, [P] * 20 + [Z, I, L, L, I, I, I, I, I, I, I, I, I, F, P]),
    "nsa_decode_workspace_bytes": (Z, [I, I]),
    "nsa_rowdot": (I, [P, P, P, P, P, L, I, P]),
    "nsa_combine": (I, [P, P, P, P, P, P, P, L, I, P]),
    "nsa_gate_fwd": (I, [P, P, P, P, P, P, L, I, P]),
    "nsa_rowdot3": (I, [P] * 13 + [L, I, P]),
    "nsa_gate_bwd_workspace_bytes": (L, [L, I]),
    "nsa_gate_bwd": (I, [P] * 9 + [L, L, I, P]),
}

_lib = None


def lib():
    """The loaded library.  Raises if it has not been built (python -m nsa_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libnsa_b200.so is missing at %s: build it with `python -m nsa_b200.build`. "
                "There is no CPU or PyTorch fallback for these operators." % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc, what):
    if rc != 0:
        msg = lib().nsa_last_error().decode() if rc < 0 else "CUDA error %d at launch" % rc
        raise RuntimeError("%s failed (%d): %s" % (what, rc, msg))


def device_status():
    """Synchronise and raise if a kernel reported that it gave up waiting (never expected)."""
    rc = lib().nsa_device_status()
    if rc != 0:
        raise RuntimeError("nsa_b200 device status %d: %s" % (rc, lib().nsa_last_error().decode()))


# Selected-branch dQ from the key-major backward kernel (needs B*Tq*Hq*S*D*2 more bytes of workspace) or from the
# query-major dQ kernel.  The library picks the path from the workspace size it is handed.
SEL_DQ_FROM_KV = True


def sel_swa_bwd_workspace_bytes(B, T, Tq, Hq, Hkv, D, S, BS):
    if SEL_DQ_FROM_KV and D == 128 and BS == 64:
        return lib().nsa_sel_swa_bwd_workspace_bytes_dq(B, T, Tq, Hq, Hkv, D, S, BS)
    return lib().nsa_sel_swa_bwd_workspace_bytes(B, T, Hkv, S, BS)


# Selected-branch forward key-major on the tensor cores (needs a workspace of about B*Tq*Hq*S*D*2 bytes) or query-major.
SEL_FWD_KV = True


def sel_swa_fwd_workspace_bytes(B, T, Tq, Hq, Hkv, D, S, BS):
    if SEL_FWD_KV and D == 128 and BS == 64 and S <= 32 and Hq % (16 * Hkv) == 0:
        return lib().nsa_sel_swa_fwd_workspace_bytes(B, T, Tq, Hq, Hkv, D, S, BS)
    return 0


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def require(t, name, dtype=torch.bfloat16):
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor: nsa_b200 has no CPU path" % name)
    if dtype is not None and t.dtype != dtype:
        raise TypeError("%s must be %s (got %s)" % (name, dtype, t.dtype))
    return t.contiguous()
