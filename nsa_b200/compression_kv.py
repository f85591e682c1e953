"""K/V block compression with the reference's API (nsa/compression_kv.py).

``compress_kv``, ``calc_compressed_len``, ``KVCompressorVarlen`` and ``KVCompressor`` keep the reference's
names, arguments, parameter names/shapes and return values; the work is done by ``nsa_compress_fwd`` /
``nsa_compress_bwd`` of libnsa_b200.so.
"""
import math

import torch
import torch.nn as nn
from torch.nn import init

from . import _lib


def calc_compressed_len(x, stride, size):
    """nsa/compression_kv.py:9-10 (the functional path's length rule, one less than Conv1d's)."""
    return (x - size) // stride


_cu_cache = {}


def _cu_tensor(values, device):
    key = (tuple(values), str(device))
    t = _cu_cache.get(key)
    if t is None:
        if len(_cu_cache) > 64:
            _cu_cache.clear()
        t = torch.tensor(list(values), dtype=torch.int32, device=device)
        _cu_cache[key] = t
    return t


class _CompressOne(torch.autograd.Function):
    """y = compress(x; w, bias) for one tensor.  x [tok,H,D]; w [l*D, D]; bias [D] or None."""

    @staticmethod
    def forward(ctx, x, w, bias, cu_in, cu_out, block, stride):
        x = _lib.require(x, "x")
        w = _lib.require(w, "w")
        bias = _lib.require(bias, "bias")
        tok, H, D = x.shape
        if w.shape != (block * D, D):
            raise ValueError("weight must have shape [block*D, D] = %s, got %s" % ((block * D, D), tuple(w.shape)))
        nseq = len(cu_in) - 1
        total_out = cu_out[-1]
        max_out = max([cu_out[i + 1] - cu_out[i] for i in range(nseq)] + [0])
        max_in = max([cu_in[i + 1] - cu_in[i] for i in range(nseq)] + [0])
        y = torch.empty(total_out, H, D, dtype=torch.bfloat16, device=x.device)
        cin, cout = _cu_tensor(cu_in, x.device), _cu_tensor(cu_out, x.device)
        lens = [cu_in[i + 1] - cu_in[i] for i in range(nseq)]
        uniform = (nseq > 0 and len(set(lens)) == 1 and lens[0] >= block and lens[0] % stride == 0
                   and cu_out[1] - cu_out[0] == (lens[0] - block) // stride + 1)
        if total_out > 0 and uniform:
            _lib.check(_lib.lib().nsa_compress_fwd_uniform(_lib.ptr(x), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(y), nseq,
                                                           lens[0], H, D, block, stride, _lib.stream()),
                       "nsa_compress_fwd_uniform")
        elif total_out > 0:
            _lib.check(_lib.lib().nsa_compress_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(y), _lib.ptr(cin),
                                                   _lib.ptr(cout), nseq, H, D, block, stride, max_out, _lib.stream()),
                       "nsa_compress_fwd")
        ctx.save_for_backward(x, w, cin, cout)
        ctx.meta = (nseq, H, D, block, stride, max_in, total_out, bias is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, cin, cout = ctx.saved_tensors
        nseq, H, D, block, stride, max_in, total_out, has_bias = ctx.meta
        dy = _lib.require(dy, "dy")
        need_x, need_w, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1], has_bias and ctx.needs_input_grad[2]
        dx = torch.empty_like(x) if need_x else None
        dw = torch.empty(block * D, D, dtype=torch.float32, device=x.device) if need_w else None
        db = torch.empty(D, dtype=torch.float32, device=x.device) if need_b else None
        L = _lib.lib()
        ws_bytes = L.nsa_compress_bwd_workspace_bytes(nseq, H, D, block) if need_w else 0
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
        if total_out > 0:
            _lib.check(L.nsa_compress_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(dx), _lib.ptr(dw), _lib.ptr(db),
                                          _lib.ptr(ws), ws_bytes, _lib.ptr(cin), _lib.ptr(cout), nseq, H, D, block, stride,
                                          max_in, total_out, _lib.stream()), "nsa_compress_bwd")
        else:
            for t in (dx, dw, db):
                if t is not None:
                    t.zero_()
        return dx, dw, db, None, None, None, None


def _host_cu(cu_seq_len):
    if torch.is_tensor(cu_seq_len):
        return [int(c) for c in cu_seq_len.tolist()]   # one host sync, as nsa/compression_kv.py:184
    return [int(c) for c in cu_seq_len]


def compress_kv(k, v, w_k, w_v, cu_seq_len, block_stride, block_size):
    """Drop-in for ``compress_kv`` (nsa/compression_kv.py:269): returns (ck, cv, cu_out_len int32)."""
    cu_in = _host_cu(cu_seq_len)
    cu_out = [0]
    for i in range(len(cu_in) - 1):
        cu_out.append(cu_out[-1] + max(calc_compressed_len(cu_in[i + 1] - cu_in[i], block_stride, block_size), 0))
    ck = _CompressOne.apply(k, w_k, None, cu_in, cu_out, block_size, block_stride)
    cv = _CompressOne.apply(v, w_v, None, cu_in, cu_out, block_size, block_stride)
    return ck, cv, _cu_tensor(cu_out, k.device)


def compress_conv(x, weight, bias, block, stride, B):
    """Module-path compression of x [B*T,H,D] with an nn.Conv1d weight [D,D,block] and bias [D]:
    the contraction of nsa/compression_kv.py:301-307, output [B,Tc,H,D] with Tc = (T-block)//stride + 1."""
    tok, H, D = x.shape
    T = tok // B
    Tc = (T - block) // stride + 1 if T >= block else 0
    cu_in = [T * i for i in range(B + 1)]
    cu_out = [Tc * i for i in range(B + 1)]
    wm = weight.permute(2, 1, 0).reshape(block * D, D)   # rows j*D+c, columns o (autograd permutes back)
    y = _CompressOne.apply(x, wm, bias, cu_in, cu_out, block, stride)
    return y.view(B, Tc, H, D)


class KVCompressorVarlen(nn.Module):
    """nsa/compression_kv.py:272-289: parameters k_weight, v_weight [block*D, D], kaiming-uniform."""

    def __init__(self, block_stride, block_size, head_dim, device, dtype):
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.block_stride = block_stride
        self.block_size = block_size
        self.k_weight = nn.Parameter(torch.empty(block_size * head_dim, head_dim, **factory_kwargs))
        self.v_weight = nn.Parameter(torch.empty(block_size * head_dim, head_dim, **factory_kwargs))
        self.reset_parameters()

    def forward(self, k, v, cu_seq_len, group=None):
        return compress_kv(k, v, self.k_weight, self.v_weight, cu_seq_len, self.block_stride, self.block_size)

    def reset_parameters(self) -> None:
        init.kaiming_uniform_(self.k_weight, a=math.sqrt(5))
        init.kaiming_uniform_(self.v_weight, a=math.sqrt(5))


class KVCompressor(nn.Module):
    """nsa/compression_kv.py:292-312: two nn.Conv1d(D, D, block, stride) parameter sets (state_dict
    keys compressor_k.weight/bias, compressor_v.weight/bias), applied by the CUDA compression kernel."""

    def __init__(self, block_stride, block_size, head_dim, device, dtype):
        super().__init__()
        factory_kwargs = {"device": device, "dtype": dtype}
        self.block_stride = block_stride
        self.block_size = block_size
        self.compressor_k = nn.Conv1d(head_dim, head_dim, block_size, block_stride, **factory_kwargs)
        self.compressor_v = nn.Conv1d(head_dim, head_dim, block_size, block_stride, **factory_kwargs)

    def forward(self, k, v, cu_seq_len, group=None):
        """k,v [B*T,H,D] (equal-length sequences) -> ck,cv [B,Tc,H*group,D], and cu_seq_len unchanged.
        ``group`` repeats every KV head ``group`` times as the reference does; pass None to keep the
        compact [B,Tc,H,D] form, which the compressed-attention kernel reads directly."""
        B = cu_seq_len.shape[0] - 1
        ck = compress_conv(k, self.compressor_k.weight, self.compressor_k.bias, self.block_size, self.block_stride, B)
        cv = compress_conv(v, self.compressor_v.weight, self.compressor_v.bias, self.block_size, self.block_stride, B)
        if group is not None:
            ck = ck.repeat_interleave(group, dim=2)
            cv = cv.repeat_interleave(group, dim=2)
        return ck, cv, cu_seq_len
