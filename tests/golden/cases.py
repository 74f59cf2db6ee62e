"""Golden cases: how each fixture's inputs are drawn and which call it checks.

Shared by ``make_golden.py`` (which writes the ``.npz`` files with the oracle's
outputs) and by the tests (which regenerate the same inputs from the seeds and
compare).  Inputs are not stored: ``numpy.random.Generator(PCG64)`` is
reproducible across machines, and every fixture carries checksums of its inputs so
a drift in the generator is detected.
"""

import math

import numpy as np
import torch

_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}

# name -> dict(kind, dims..., dtype, flags)
CASES = {
    # fp32 causal MHA (configuration 1 in miniature and at full size)
    "c1_small": dict(kind="fwd", B=1, Lq=40, Lkv=40, Hq=2, Hkv=2, D=16, Dv=16, dtype="f32", causal=True),
    "c1_full": dict(kind="fwd", B=2, Lq=256, Lkv=256, Hq=4, Hkv=4, D=64, Dv=64, dtype="f32", causal=True),
    # GQA prefill bf16 (configuration 2 scaled down), causal and not
    "c2_small": dict(kind="fwd", B=1, Lq=384, Lkv=384, Hq=4, Hkv=2, D=128, Dv=128, dtype="bf16", causal=False),
    "c2_small_causal": dict(kind="fwd", B=1, Lq=384, Lkv=384, Hq=4, Hkv=2, D=128, Dv=128, dtype="bf16", causal=True),
    # key-length mask + dense bias (configuration 3 scaled down)
    "c3_small": dict(kind="fwd", B=2, Lq=256, Lkv=256, Hq=2, Hkv=2, D=64, Dv=64, dtype="bf16", causal=False,
                     kv_lengths=True, bias=True),
    # ragged, unaligned: lengths 50 x 77, D = 24, causal + bias (tests/test_attention_xla.py:424-431 shape family)
    "ragged_bias": dict(kind="fwd", B=2, Lq=50, Lkv=77, Hq=4, Hkv=2, D=24, Dv=24, dtype="f32", causal=True, bias=True),
    # decode (configuration 4 scaled down)
    "c4_small": dict(kind="decode", B=3, Lq=1, Lkv=1500, Hq=8, Hkv=2, D=128, Dv=128, dtype="bf16", kv_lengths=True),
    # latent attention (configuration 5 scaled down): rank 64 + rotary 64, nope 128
    "c5_small": dict(kind="mla", B=1, Lq=256, S=256, H=2, Dqk=192, Dv=128, R=128, dtype="bf16", causal=True),
}


def _normal(rng, shape, dtype, std=1.0):
    return torch.from_numpy(rng.standard_normal(size=shape, dtype=np.float32) * np.float32(std)).to(dtype)


def make_inputs(name):
    c = CASES[name]
    seed = int.from_bytes(name.encode(), "little") % (2**31)
    r = [np.random.Generator(np.random.PCG64(s)) for s in np.random.SeedSequence(seed).spawn(6)]
    dt = _DT[c["dtype"]]
    if c["kind"] in ("fwd", "decode"):
        q = _normal(r[0], (c["B"], c["Lq"], c["Hq"], c["D"]), dt)
        k = _normal(r[1], (c["B"], c["Lkv"], c["Hkv"], c["D"]), dt)
        v = _normal(r[2], (c["B"], c["Lkv"], c["Hkv"], c["Dv"]), dt)
        out = dict(q=q, k=k, v=v, sm_scale=1.0 / math.sqrt(c["D"]), causal=bool(c.get("causal", False)))
        if c.get("kv_lengths"):
            lo = max(1, c["Lkv"] // 4)
            out["kv_lengths"] = torch.from_numpy(r[3].integers(lo, c["Lkv"] + 1, size=c["B"]).astype(np.int32))
        if c.get("bias"):
            out["bias"] = _normal(r[4], (1, c["Hq"], c["Lq"], c["Lkv"]), torch.float32)
        return out
    if c["kind"] == "mla":
        q = _normal(r[0], (c["B"], c["Lq"], c["H"], c["Dqk"]), dt)
        cache = _normal(r[1], (c["B"], c["S"], c["R"]), dt)
        wk = _normal(r[2], (c["H"], c["Dqk"], c["R"]), dt, 0.1)
        wv = _normal(r[3], (c["H"], c["Dv"], c["R"]), dt, 0.1)
        return dict(q=q, cache=cache, wk=wk, wv=wv, sm_scale=1.0 / math.sqrt(c["Dqk"]), causal=bool(c.get("causal")))
    raise ValueError(name)


def input_checksums(inp):
    return {k: float(v.double().sum()) for k, v in inp.items() if isinstance(v, torch.Tensor)}


def oracle_outputs(name, inp):
    """(out fp32, lse fp32) from the CPU oracle for case ``name``."""
    import oracle

    c = CASES[name]
    if c["kind"] in ("fwd", "decode"):
        out, lse = oracle.xla_attention(
            inp["q"], inp["k"], inp["v"], causal=inp["causal"], kv_lengths=inp.get("kv_lengths"),
            bias=inp.get("bias"), sm_scale=inp["sm_scale"], return_lse=True)
    else:
        out, lse = oracle.mla_reference(
            inp["q"], inp["cache"], inp["wk"], inp["wv"], sm_scale=inp["sm_scale"], causal=inp["causal"],
            factorisation="materialized", return_lse=True)
    return out.float(), lse.float()
