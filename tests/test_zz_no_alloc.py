"""The allocation-free compression backward (nsa_compress_bwd_noalloc) against the regular entry point.

Some users of libnsa_b200.so cannot call cudaMalloc at the moment they need the backward pass -- a serving or
training runtime that partitions all device memory up front, or a host application that owns the allocator and
gives plugins none.  For them the library carries its own fixed scratch array.  This test calls that entry point
through the C ABI twice in a row (the array keeps the previous call's partials, so the second call proves nothing
stale leaks into the result) and compares dx, dW and dbias with nsa_compress_bwd, whose workspace the caller
allocates.  It lives in a file that pytest collects last and needs nothing from the other tests.
"""
import pytest
import torch

ATOL, RTOL = 2e-2, 1e-2


def _close(name, got, ref):
    err = (got.float() - ref.float()).abs()
    bad = err > ATOL + RTOL * ref.float().abs()
    assert not bad.any(), "%s: %d/%d outside tolerance, max abs err %.4g" % (name, int(bad.sum()), bad.numel(),
                                                                              float(err.max()))


@pytest.mark.gpu
@pytest.mark.parametrize("D,H,block,stride,lens", [(128, 4, 32, 16, [512, 200, 96]), (64, 2, 64, 16, [300, 64])])
def test_noalloc_matches_workspace_entry_point(D, H, block, stride, lens):
    from nsa_b200 import _lib
    L = _lib.lib()
    dev = "cuda"
    gen = torch.Generator().manual_seed(123 + D)
    cu_in = [0]
    cu_out = [0]
    for n in lens:
        cu_in.append(cu_in[-1] + n)
        cu_out.append(cu_out[-1] + (n - block) // stride + 1)
    nseq, tok, out_tok = len(lens), cu_in[-1], cu_out[-1]
    cin = torch.tensor(cu_in, dtype=torch.int32, device=dev)
    cout = torch.tensor(cu_out, dtype=torch.int32, device=dev)
    w = (torch.randn(block * D, D, generator=gen) * 0.03).to(dev, torch.bfloat16)
    P, S = _lib.ptr, _lib.stream

    def run(entry, x, dy):
        dx = torch.empty_like(x)
        dw = torch.empty(block * D, D, dtype=torch.float32, device=dev)
        db = torch.empty(D, dtype=torch.float32, device=dev)
        if entry == "workspace":
            nbytes = L.nsa_compress_bwd_workspace_bytes(nseq, H, D, block)
            ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            rc = L.nsa_compress_bwd(P(x), P(w), P(dy), P(dx), P(dw), P(db), P(ws), nbytes, P(cin), P(cout), nseq, H, D,
                                    block, stride, max(lens), out_tok, S())
        else:
            rc = L.nsa_compress_bwd_noalloc(P(x), P(w), P(dy), P(dx), P(dw), P(db), P(cin), P(cout), nseq, H, D, block,
                                            stride, max(lens), out_tok, S())
        _lib.check(rc, entry)
        torch.cuda.synchronize()
        return dx, dw, db

    for call in range(2):                      # two calls in a row, different data each time
        x = torch.randn(tok, H, D, generator=gen).to(dev, torch.bfloat16)
        dy = torch.randn(out_tok, H, D, generator=gen).to(dev, torch.bfloat16)
        ref = run("workspace", x, dy)
        got = run("noalloc", x, dy)
        for name, g, r in zip(("dx", "dw", "dbias"), got, ref):
            _close("call %d %s" % (call, name), g, r)
        assert ref[1].abs().max() > 0.1       # the comparison is not vacuous
    _lib.device_status()


@pytest.mark.gpu
def test_noalloc_rejects_shapes_beyond_its_scratch():
    from nsa_b200 import _lib
    L = _lib.lib()
    one = torch.zeros(16, dtype=torch.float32, device="cuda")
    p = _lib.ptr(one)
    # block*D*D = 512*128*128 floats = 32 MiB > the 16 MiB built-in array
    rc = L.nsa_compress_bwd_noalloc(p, p, p, p, p, p, p, p, 1, 1, 128, 512, 16, 1024, 33, _lib.stream())
    assert rc < 0 and b"exceeds the built-in scratch" in L.nsa_last_error()
