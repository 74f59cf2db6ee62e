"""Helpers of the GPU parity tests: tolerances and oracle comparison."""

import os
import sys

import numpy as np
import torch

import oracle

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402,F401

# Parity bounds of the benchmark specification, against the fp32 oracle:
# 16-bit outputs max-abs 2e-2, fp32 outputs 1e-4, LSE 1e-3.
OUT_TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}
LSE_TOL = 1e-3


def dev():
    return torch.device("cuda", 0)


def randn(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


def assert_close(out, lse, want, want_lse, dtype, what=""):
    out = out.detach().float().cpu()
    want = want.detach().float().cpu()
    assert out.shape == want.shape, (what, out.shape, want.shape)
    assert torch.isfinite(out).all(), f"{what}: non-finite output"
    err = float((out - want).abs().max())
    assert err <= OUT_TOL[dtype], f"{what}: max-abs error {err:.3e} > {OUT_TOL[dtype]:.0e}"
    if lse is not None:
        lse = lse.detach().float().cpu()
        want_lse = want_lse.detach().float().cpu()
        inf_a, inf_b = torch.isinf(lse) & (lse > 0), torch.isinf(want_lse) & (want_lse > 0)
        assert torch.equal(inf_a, inf_b), f"{what}: +inf LSE rows differ"
        fin = ~inf_b
        if fin.any():
            e2 = float((lse[fin] - want_lse[fin]).abs().max())
            assert e2 <= LSE_TOL, f"{what}: LSE error {e2:.3e} > {LSE_TOL:.0e}"
    return err


def oracle_fwd(q, k, v, **kw):
    return oracle.xla_attention(q.cpu(), k.cpu(), v.cpu(), return_lse=True, **kw)


def load_golden(name):
    fx = np.load(os.path.join(os.path.dirname(__file__), "golden", f"{name}.npz"))
    return torch.from_numpy(fx["out"].astype(np.float32)), torch.from_numpy(fx["lse"])
