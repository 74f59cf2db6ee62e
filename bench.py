#!/usr/bin/env python
"""Benchmark of the attention forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (``value``): GQA prefill forward, bf16, B=4 Hq=32 Hkv=8 S=4096 D=128,
non-causal, in TFLOP/s with the inputs resident in HBM.  One step is one forward
over the whole batch.  With N > 1 (launched by torchrun, one rank per GPU) every
rank runs the same per-GPU batch (weak scaling, no collective on the data path)
and ``value`` is the aggregate over all ranks divided by the slowest rank's time.

The same JSON line also carries the end-to-end number through the public API with
pinned host buffers (``e2e``), the roofline of the dominant kernel, the CPU
baseline (the oracle port on the host cores, bounded sample) and, as additional
objects, the other configurations: causal prefill, masked + biased attention,
latent attention, split-KV decode (HBM GB/s) and -- with N > 1 -- the decode with
the KV sequence sharded over the ranks plus its all-gather and combine.

``--impl reference`` times the reference's CPU attention path (the oracle port:
the reference itself needs jax, which is not installable offline) on the host
cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

C2 = dict(B=4, Hq=32, Hkv=8, S=4096, D=128)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


PREFILL_PROFILE = "profiles/attn_fwd_sm100_prefill_b2_s4096.md"


def profiled_prefill_traffic(batch):
    """DRAM read + write bytes per launch of the headline kernel, from the tracked ncu summary
    of the B=2 case (last capture column), scaled with the batch; None if the file is absent."""
    import re

    try:
        text = open(os.path.join(ROOT, PREFILL_PROFILE)).read()
        tot = 0.0
        for name in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
            row = re.search(r"\| `" + re.escape(name) + r"` \|(.*)\|", text).group(1)
            tot += float(re.findall(r"([0-9.]+) MB", row)[-1]) * 1e6
        return tot * batch / 2.0
    except Exception:
        return None


def rounded(obj, digits=4):
    """Floats to `digits` significant digits (keeps the JSON line short)."""
    if isinstance(obj, float):
        return float(f"{obj:.{digits}g}") if obj == obj and abs(obj) != float("inf") else obj
    if isinstance(obj, dict):
        return {k: rounded(v, digits) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [rounded(v, digits) for v in obj]
    return obj


def prefill_flops(B, Hq, Lq, Lkv, D, Dv, causal):
    if causal:  # sum over rows of (i + 1) keys, rows beyond Lkv see Lkv keys
        pairs = sum(min(i + 1, Lkv) for i in range(Lq))
    else:
        pairs = Lq * Lkv
    return 2.0 * B * Hq * pairs * (D + Dv)


class ClockSampler:
    """Samples SM clocks and clock-event reasons through NVML (read-only) every
    couple of milliseconds while a region runs; falls back to nvidia-smi."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index=0):
        self.index, self.sm, self.bits, self.max_mhz = index, [], 0, None
        self.stop, self.th, self.proc = threading.Event(), None, None

    def _nvml_loop(self, nv, handle):
        getr = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                self.bits |= int(getr(handle))
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                handle = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.th = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.th.start()
        except Exception:
            self.th = None
            try:
                q = "clocks.sm,clocks.max.sm,clocks_event_reasons.active"
                self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                              "--format=csv,noheader,nounits", "-lms", "50"],
                                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            except Exception:
                self.proc = None
        return self

    def __exit__(self, *a):
        self.stop.set()
        if self.th:
            self.th.join(timeout=1)
        if self.proc:
            time.sleep(0.1)
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=2)
                for line in out.splitlines():
                    f = [x.strip() for x in line.split(",")]
                    self.sm.append(float(f[0]))
                    self.max_mhz = float(f[1])
                    self.bits |= int(f[2], 16)
            except Exception:
                pass

    def summary(self):
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.sm), "sm_min_mhz": min(self.sm), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for b, n in self.REASONS.items() if self.bits & b), "samples": len(self.sm)}


def time_steps(fn, steps, warmup, dist_on=False):
    """W untimed steps, then exactly K steps between CUDA events on the launching
    stream, bracketed by barrier + synchronize. Returns total milliseconds."""
    import torch.distributed as dist

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def max_over_ranks(ms, dist_on):
    if not dist_on:
        return ms
    import torch.distributed as dist

    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def cpu_baseline(budget_s=12.0, threads=None):
    """The oracle port on the host cores: configuration 2 (non-causal) one batch
    row at a time until about `budget_s` seconds are spent (at least one row)."""
    import oracle

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    c = oracle.make_config(2, B=1)
    oracle.xla_attention(c["q"][:, :512], c["k"][:, :512], c["v"][:, :512], sm_scale=c["sm_scale"])  # warm the pool
    done, t0 = 0, time.perf_counter()
    while done < C2["B"] and (done == 0 or time.perf_counter() - t0 < budget_s):
        oracle.xla_attention(c["q"], c["k"], c["v"], sm_scale=c["sm_scale"])
        done += 1
    dt = time.perf_counter() - t0
    fl = prefill_flops(done, C2["Hq"], C2["S"], C2["S"], C2["D"], C2["D"], False)
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{done} of {C2['B']} batch rows of the workload, {dt:.1f} s, torch fp32 port of the XLA path"}


WORKLOAD = "GQA prefill fwd bf16 B{b} Hq32 Hkv8 S4096 D128 non-causal (per GPU)"


def run_reference(args, rank):
    """--impl reference: the reference's CPU attention path on the host cores, on the
    same workload as the GPU arm: one step = the whole batch, same warm-up count."""
    if rank != 0:
        return
    import oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    c = oracle.make_config(2, B=args.batch)

    def step():
        for b in range(args.batch):  # one batch row at a time bounds the fp32 score memory
            oracle.xla_attention(c["q"][b:b + 1], c["k"][b:b + 1], c["v"][b:b + 1], sm_scale=c["sm_scale"])

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    fl = prefill_flops(args.batch, C2["Hq"], C2["S"], C2["S"], C2["D"], C2["D"], False) * args.steps
    val = fl / dt / 1e12
    sample = f"each step = the whole workload (B={args.batch}), {threads} threads"
    _emit({
        "impl": "reference", "metric": "attn_fwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD.format(b=args.batch)},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "oracle port of probjax's XLA CPU path (the reference needs jax, not installable offline)",
    })


def bench_extra(name, fn, steps, warmup, work, unit, peak, bound, pk_note, profile=None):
    """Time one secondary configuration (the faster of two timed batches); returns a small dict (never
    raises).  `profile` names the tracked ncu summary of the kernel behind the number."""
    try:
        # Two timed batches of `steps` steps each, the faster one reported: one batch in some tens of runs
        # came out far slower than every other run of the same build.  A slower batch that differs by more
        # than a quarter stays visible as "ms_other".
        a = time_steps(fn, steps, warmup) / steps
        b = time_steps(fn, steps, 1) / steps
        ms = min(a, b)
        ach = work / (ms * 1e-3)
        out = {"ms": ms, "value": ach, "unit": unit, "bound": bound, "frac": ach / peak}
        if max(a, b) > 1.25 * ms:
            out["ms_other"] = max(a, b)
        if profile:  # file under profiles/ (without the .md) that holds the ncu summary of this kernel
            out["profile"] = os.path.splitext(os.path.basename(profile))[0]
        return out
    except Exception as e:  # keep the headline line alive
        return {"error": f"{type(e).__name__}: {e}"[:200]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-extras", action="store_true", help="headline only (used for profiling captures)")
    ap.add_argument("--skip-cpu", action="store_true", help="do not time the CPU baseline")
    ap.add_argument("--batch", type=int, default=C2["B"], help="batch rows of the headline workload (profiling captures use a smaller one)")
    ap.add_argument("--skip-e2e", action="store_true", help="do not time the host-buffer path")
    ap.add_argument("--only-decode", action="store_true", help="time only the decode configuration (profiling captures)")
    ap.add_argument("--only-backward", action="store_true",
                    help="time only the backward of the headline shape on --batch rows (profiling captures)")
    ap.add_argument("--only-linear", action="store_true",
                    help="time only the fused QKV projection of the headline shape (profiling captures)")
    ap.add_argument("--only-masked-bias", action="store_true",
                    help="time only the masked + biased configuration on --batch batch rows (profiling captures)")
    ap.add_argument("--only-latent-decode", action="store_true",
                    help="time only the absorbed latent decode on --batch sequences (profiling captures)")
    ap.add_argument("--only-waves", action="store_true",
                    help="time the unmasked forward on 8 .. 512 equal work items (256 query rows x 4096 keys each): "
                         "the staircase of waves and what cutting the last wave into KV halves buys "
                         "(PJX_FWD_SPLIT_TAIL=0 switches the halves off)")
    ap.add_argument("--only-prefill", action="store_true",
                    help="time only the headline forward, non-causal and causal, without checking the result "
                         "(what-if builds of the forward kernel, whose outputs are wrong on purpose)")
    ap.add_argument("--only-latent", action="store_true",
                    help="time only the latent-attention configuration on --batch batch rows (profiling captures)")
    ap.add_argument("--only-modifier", default=None,
                    choices=["band", "row_limits", "one_segment", "packed_8x512", "head_scale", "causal_alibi", "soft_cap"],
                    help="time only the headline shape on --batch rows under one structured mask or score term "
                         "(profiling captures of the forward kernel's band / modifier variants)")
    ap.add_argument("--kernel", default=None, choices=[None, "b200:generic", "b200:tcgen05"],
                    help="force one forward kernel for the headline (default: the library's own choice)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import oracle
    import probjax_b200 as pj
    from probjax_b200 import _lib

    _lib.lib()  # raises if the CUDA library is not built: there is no other path
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist_on = world > 1
    if dist_on:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    pk = peaks()

    if args.only_decode:
        only_decode(args, dev, pk)
        return
    if args.only_backward:
        only_backward(args, dev, pk)
        return
    if args.only_linear:
        only_linear(args, dev, pk)
        return
    if args.only_masked_bias:
        only_masked_bias(args, dev, pk)
        return
    if args.only_waves:
        only_waves(args, dev, pk)
        return
    if args.only_prefill:
        only_prefill(args, dev, pk)
        return
    if args.only_modifier:
        only_modifier(args, dev, pk)
        return
    if args.only_latent_decode:
        only_latent_decode(args, dev, pk)
        return
    if args.only_latent:
        only_latent(args, dev, pk)
        return

    # ---------------------------------------------------------------- headline
    c = oracle.make_config(2, B=args.batch)
    q, k, v = c["q"].to(dev), c["k"].to(dev), c["v"].to(dev)
    sc = c["sm_scale"]
    flops = prefill_flops(args.batch, C2["Hq"], C2["S"], C2["S"], C2["D"], C2["D"], False)

    def step():
        return pj.attention_forward(q, k, v, sm_scale=sc, impl=args.kernel)

    n0 = _lib.launch_count()
    step()
    launches_per_step = _lib.launch_count() - n0  # kernels of this library per step
    with ClockSampler(local_rank) as cs:
        ms_total = time_steps(step, args.steps, args.warmup, dist_on)
    pj.check_status(dev)
    ms_total = max_over_ranks(ms_total, dist_on)
    ms = ms_total / args.steps
    value = flops * world / (ms * 1e-3) / 1e12
    per_gpu = flops / (ms * 1e-3) / 1e12
    clocks = cs.summary()

    # ------------------------------------------------------------- end to end
    qh, kh, vh = c["q"].pin_memory(), c["k"].pin_memory(), c["v"].pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    oh = torch.empty(tuple(q.shape), dtype=q.dtype, pin_memory=True)

    def step_host():  # H2D q,k,v + kernel + D2H o; returns after the result is in host memory
        return pj.attention_forward(qh, kh, vh, sm_scale=sc, out=oh)

    ms_e2e = max_over_ranks(time_steps(step_host, e2e_steps, 3, dist_on), dist_on) / e2e_steps
    h2d = sum(t.numel() * t.element_size() for t in (qh, kh, vh))
    d2h = q.numel() * q.element_size()
    e2e = {"value": flops * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "call": "attention_forward on pinned host tensors (pjx_attn_fwd_host)"}

    # one-shot parity of the headline result: batch row 0 against the oracle (outside every timed region)
    try:
        got0 = step()[0:1].float().cpu()
        want0 = oracle.xla_attention(c["q"][0:1], c["k"][0:1], c["v"][0:1], sm_scale=sc).float()
        parity = float((got0 - want0).abs().max())
        del got0, want0
    except Exception as e:
        parity = f"{type(e).__name__}: {e}"[:120]
    alg_bytes = sum(t.numel() * t.element_size() for t in (q, k, v)) + q.numel() * q.element_size()
    out = {
        "metric": "attn_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD.format(b=args.batch),
                   "l2": "335 MB of inputs+outputs per step exceed the 126 MB L2: no flush",
                   "parallelism": f"batch-sharded x{world}, no collective" if world > 1 else "single GPU"},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": per_gpu / pk["bf16_tflops"],
                     # measured DRAM bytes per launch of this kernel: the ncu capture of the B=2 case, scaled
                     # with the batch (traffic grows in proportion); the algorithmic bytes beside it
                     "traffic": profiled_prefill_traffic(args.batch), "traffic_source": PREFILL_PROFILE,
                     "algorithmic_bytes": alg_bytes,
                     "of": f"{pk['source']} burst peak", "kernel": "attn_fwd_sm100_kernel<128,128,128,2,2,bf16>",
                     "frac_of_sustained": per_gpu / pk["bf16_tflops_sustained"]},
        "e2e": e2e, "gpu_launches": int(launches_per_step * args.steps), "clocks": clocks,
        "parity_max_abs_err": parity,
    }
    if isinstance(parity, float) and not parity <= 2e-2:
        raise SystemExit(f"headline result differs from the oracle: max-abs error {parity}")

    # ------------------------------------------------- other configurations
    if not args.skip_extras:
        xs, xw = max(5, min(args.steps, 20)), 3
        extras = {}
        fl_c = prefill_flops(C2["B"], C2["Hq"], C2["S"], C2["S"], C2["D"], C2["D"], True)
        extras["prefill_causal"] = bench_extra(
            "causal", lambda: pj.attention_forward(q, k, v, causal=True, sm_scale=sc), xs, xw, fl_c / 1e12,
            "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"], PREFILL_PROFILE)
        try:  # sliding window of 1024 keys (the band form of the mask): keys j with i-1023 <= j <= i
            win = 1024
            rows = torch.arange(C2["S"], dtype=torch.float64)
            fl_w = 4.0 * C2["B"] * C2["Hq"] * C2["D"] * float(torch.clamp(rows + 1, max=win).sum())
            extras["prefill_window_1024"] = bench_extra(
                "window", lambda: pj.attention_forward(q, k, v, band=(-(win - 1), 0), sm_scale=sc), xs, xw, fl_w / 1e12,
                "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
        except Exception as e:
            extras["prefill_window_1024"] = {"error": str(e)[:300]}
        try:  # structured masks and score terms evaluated inside the kernel, through the mask / bias objects:
            # packed sequences (8 segments of 512 tokens, causal inside each) and causal attention with ALiBi
            seg = (torch.arange(C2["S"], device=dev) // 512).to(torch.int32)[None]
            m_seg = pj.BlockDiagonalCausalMask(seg)
            extras["prefill_packed_8x512_causal"] = bench_extra(
                "packed", lambda: pj.mha(q, k, v, mask=m_seg, sm_scale=sc), xs, xw,
                8 * prefill_flops(C2["B"], C2["Hq"], 512, 512, C2["D"], C2["D"], True) / 1e12,
                "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
            m_c, b_al = pj.CausalMask(), pj.CausalAlibiBias()
            extras["prefill_causal_alibi"] = bench_extra(
                "alibi", lambda: pj.mha(q, k, v, mask=m_c, bias=b_al, sm_scale=sc), xs, xw, fl_c / 1e12,
                "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
        except Exception as e:
            extras["prefill_packed_8x512_causal"] = {"error": str(e)[:300]}
        try:  # backward of the headline shape (tcgen05 dQ and dK/dV kernels + the delta kernel);
            # FLOPs counted as 2.5 x the forward (five products), although the split design computes seven
            o_b, lse_b = pj.attention_forward(q, k, v, sm_scale=sc, return_lse=True)
            g_b = torch.randn_like(o_b)
            extras["backward"] = bench_extra(
                "bwd", lambda: pj.attention_backward(q, k, v, o_b, lse_b, g_b, sm_scale=sc), xs, xw,
                2.5 * flops / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"], "profiles/bwd_sm100_b2_s4096.md")
            o_c, lse_c = pj.attention_forward(q, k, v, causal=True, sm_scale=sc, return_lse=True)
            extras["backward_causal"] = bench_extra(
                "bwd_causal", lambda: pj.attention_backward(q, k, v, o_c, lse_c, g_b, causal=True, sm_scale=sc), xs, xw,
                2.5 * fl_c / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
            del o_b, lse_b, g_b, o_c, lse_c
        except Exception as e:
            extras["backward"] = {"error": str(e)[:300]}
        try:  # fused QKV projection of the headline shape: [B*S, d_model] x [(Hq + 2 Hkv) * D, d_model]^T
            d_model = 4096
            m_rows, n_out = args.batch * C2["S"], (C2["Hq"] + 2 * C2["Hkv"]) * C2["D"]
            xg = torch.randn((m_rows, d_model), device=dev).bfloat16()
            wg = (torch.randn((n_out, d_model), device=dev) / 64).bfloat16()
            extras["qkv_projection"] = bench_extra(
                "linear", lambda: pj.linear(xg, wg), xs, xw, 2.0 * m_rows * n_out * d_model / 1e12, "TFLOP/s",
                pk["bf16_tflops"], "tensor", pk["source"], "profiles/gemm_tn_sm100_qkv_projection.md")
            del xg, wg
        except Exception as e:
            extras["qkv_projection"] = {"error": str(e)[:300]}
        try:  # configuration 1: exact fp32 causal MHA, latency-bound (time and parity only)
            c1 = oracle.make_config(1)
            q1, k1, v1 = c1["q"].to(dev), c1["k"].to(dev), c1["v"].to(dev)
            fl1 = prefill_flops(2, 4, 256, 256, 64, 64, True)
            extras["fp32_causal_small"] = bench_extra(
                "c1", lambda: pj.attention_forward(q1, k1, v1, causal=True, sm_scale=c1["sm_scale"]), xs * 5, xw,
                fl1 / 1e12, "TFLOP/s", 72.0, "fp32 FMA nominal", "nominal")
            got = pj.attention_forward(q1, k1, v1, causal=True, sm_scale=c1["sm_scale"]).cpu()
            want = oracle.xla_attention(c1["q"], c1["k"], c1["v"], causal=True, sm_scale=c1["sm_scale"])
            extras["fp32_causal_small"]["max_abs_error_vs_oracle"] = float((got - want).abs().max())
        except Exception as e:
            extras["fp32_causal_small"] = {"error": str(e)[:300]}
        try:
            c3 = oracle.make_config(3)
            q3, k3, v3 = c3["q"].to(dev), c3["k"].to(dev), c3["v"].to(dev)
            l3, b3 = c3["kv_lengths"].to(dev), c3["bias"].to(dev)
            fl3 = 4.0 * 16 * 1024 * 64 * float(c3["kv_lengths"].sum())
            extras["masked_bias"] = bench_extra(
                "c3", lambda: pj.attention_forward(q3, k3, v3, kv_lengths=l3, bias=b3, sm_scale=c3["sm_scale"]), xs, xw,
                fl3 / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"],
                "profiles/attn_fwd_sm100_masked_bias_b8_s1024.md")
            by3 = 2 * q3.numel() * 2 + 2 * 16 * 64 * 2 * float(c3["kv_lengths"].sum()) + 4.0 * 16 * 1024 * float(c3["kv_lengths"].max())
            if "ms" in extras["masked_bias"]:
                extras["masked_bias"]["hbm_gbs"] = by3 / (extras["masked_bias"]["ms"] * 1e-3) / 1e9
            del q3, k3, v3, b3
        except Exception as e:
            extras["masked_bias"] = {"error": str(e)[:300]}
        try:
            c5 = oracle.make_config(5)
            q5, ch5, wk5, wv5 = c5["q"].to(dev), c5["cache"].to(dev), c5["wk"].to(dev), c5["wv"].to(dev)
            fl5 = 2.0 * 8 * 2048 * 512 * 16 * 256 + prefill_flops(8, 16, 2048, 2048, 192, 128, True)
            extras["latent"] = bench_extra(
                "c5", lambda: pj.mla(q5, ch5, wk5, wv5, mask=pj.CausalMask(), sm_scale=c5["sm_scale"]), xs, xw,
                fl5 / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"],
                "profiles/attn_fwd_sm100_latent_b4_s2048.md")
            del q5, ch5
        except Exception as e:
            extras["latent"] = {"error": str(e)[:300]}
        try:
            for tag, full in (("decode_32k", True), ("decode_ragged", False)):
                c4 = oracle.make_config(4, full=full)
                q4, k4, v4, l4 = c4["q"].to(dev), c4["k"].to(dev), c4["v"].to(dev), c4["kv_lengths"].to(dev)
                by4 = 4096.0 * float(c4["kv_lengths"].sum()) + 2 * q4.numel() * 2 + 16 * 32 * 4
                # the all-32768 cache is full: no per-sequence lengths are passed for it
                extras[tag] = bench_extra(
                    tag, lambda: pj.decode_forward(q4, k4, v4, kv_lengths=None if full else l4, sm_scale=c4["sm_scale"],
                                                   return_lse=True),
                    xs, xw, by4 / 1e9, "GB/s", pk["hbm_gbs"], "hbm", pk["source"], "profiles/decode_splitkv_b4_32k.md")
                if "value" in extras[tag]:
                    extras[tag]["frac_of_nominal_8TBs"] = extras[tag]["value"] / 8000.0
                if full and "value" in extras[tag]:
                    # the decode half of the metric, repeated where the driver keeps it
                    out["roofline"]["decode_32k_gbs"] = extras[tag]["value"]
                    out["roofline"]["decode_32k_frac"] = extras[tag]["frac"]
                if dist_on and full:
                    ref4 = pj.decode_forward(q4, k4, v4, kv_lengths=l4, sm_scale=c4["sm_scale"], return_lse=True)
                    sh = sharded_decode_bench(c4, ref4, dev, rank, world, xs, xw, pk)
                    extras["decode_32k_seq_sharded"] = sh
                    if "value" in sh.get("fused", {}) and "value" in extras[tag]:
                        out["roofline"]["decode_sharded_gbs"] = sh["fused"]["value"]
                        out["roofline"]["decode_sharded_eff"] = sh["fused"]["value"] / (world * extras[tag]["value"])
                        out["roofline"]["decode_sharded_max_abs_err"] = sh["fused"]["max_abs_err"]
                    del ref4
                del q4, k4, v4
        except SystemExit:
            raise
        except Exception as e:
            extras["decode"] = {"error": str(e)[:300]}
        try:  # the all-32768 decode over a paged cache (pages of 256 keys, shuffled in the pool)
            c4 = oracle.make_config(4, full=True)
            q4, l4 = c4["q"].to(dev), c4["kv_lengths"].to(dev)
            page, Bc, cap = 256, c4["k"].shape[0], c4["k"].shape[1]
            mp = cap // page
            perm = torch.randperm(Bc * mp, generator=torch.Generator().manual_seed(1)).view(Bc, mp).to(torch.int32)
            kp = torch.empty((Bc * mp, page) + tuple(c4["k"].shape[2:]), dtype=c4["k"].dtype, device=dev)
            vp = torch.empty_like(kp)
            kp[perm.view(-1).long().to(dev)] = c4["k"].to(dev).view(Bc * mp, page, *c4["k"].shape[2:])
            vp[perm.view(-1).long().to(dev)] = c4["v"].to(dev).view(Bc * mp, page, *c4["v"].shape[2:])
            permd = perm.to(dev)
            by4p = 4096.0 * float(c4["kv_lengths"].sum()) + 2 * q4.numel() * 2 + 16 * 32 * 4
            extras["decode_32k_paged"] = bench_extra(
                "decode_paged", lambda: pj.decode_paged(q4, kp, vp, permd, l4, sm_scale=c4["sm_scale"]), xs, xw,
                by4p / 1e9, "GB/s", pk["hbm_gbs"], "hbm", pk["source"], "profiles/decode_splitkv_b4_32k.md")
            del kp, vp
        except Exception as e:
            extras["decode_32k_paged"] = {"error": str(e)[:300]}
        try:  # decode step of absorbed latent attention: 16 heads over a 576-wide latent cache of 32768 keys
            Bl, Hl, Rl, Sl = 16, 16, 576, 32768
            gl = torch.Generator(device=dev).manual_seed(5)
            ql = torch.randn((Bl, 1, Hl, Rl), generator=gl, device=dev).bfloat16()
            cl = (torch.randn((Bl, Sl, Rl), generator=gl, device=dev) * 0.5).bfloat16()
            extras["latent_decode_32k"] = bench_extra(
                "latent_decode", lambda: pj.mla_decode(ql, cl, sm_scale=Rl ** -0.5), xs, xw,
                (cl.numel() * 2 + 2 * ql.numel() * 2) / 1e9, "GB/s", pk["hbm_gbs"], "hbm", pk["source"],
                "profiles/decode_latent_b4_32k.md")
            del ql, cl
        except Exception as e:
            extras["latent_decode_32k"] = {"error": str(e)[:200]}
        extras["decode_128k"] = long_context_decode_bench(dev, rank, world, xs, xw, pk, dist_on)
        if dist_on and "value" in extras["decode_128k"]:
            out["roofline"]["decode_128k_sharded_gbs"] = extras["decode_128k"]["value"]
            out["roofline"]["decode_128k_sharded_max_abs_err"] = extras["decode_128k"].get("max_abs_err")
        out["extras"] = compact_extras(extras, world)

    if rank == 0 and not args.skip_cpu and world == 1:
        try:
            out["cpu_baseline"] = cpu_baseline()
        except Exception as e:
            out["cpu_baseline"] = {"error": str(e)[:300]}
    failed = [f"{k}: {v['parity_failure']}" for k, v in _walk(out.get("extras", {})) if "parity_failure" in v]
    if rank == 0:
        _emit(out)
    if dist_on:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("parity failure: " + "; ".join(failed))


def compact_extras(extras, world):
    """Keeps the one JSON line short enough to survive a truncated capture of stdout: the bound of an entry
    follows from its unit and is dropped, and so is the unit where it is the line's own (TFLOP/s); the slower variants of the sharded decode keep their time, rate
    and error only; a multi-GPU line keeps the entries that depend on the number of GPUs (the others are in
    the one-GPU line of the same build)."""
    keep_multi = ("prefill_causal", "decode_32k", "decode_ragged", "decode_32k_seq_sharded", "decode_128k")
    out = {}
    for name, entry in extras.items():
        if world > 1 and name not in keep_multi:
            continue
        if isinstance(entry, dict):
            entry = {k: v for k, v in entry.items()
                     if k not in ("bound", "frac_of_nominal_8TBs") and not (k == "unit" and v == "TFLOP/s")}
            if name == "decode_32k_seq_sharded":
                for mode, res in list(entry.items()):
                    if isinstance(res, dict):
                        keys = ("ms", "value", "frac", "max_abs_err", "lse_err", "oracle_max_abs_err", "oracle_lse_err",
                                "parity_failure", "error") if mode == "fused" else ("ms", "value", "max_abs_err",
                                                                                    "parity_failure", "error")
                        entry[mode] = {k: res[k] for k in keys if k in res}
                entry["unit"] = "GB/s aggregate"
        out[name] = entry
    return out


def _walk(d, prefix=""):
    """(path, dict) for every dict nested in d."""
    for k, v in d.items():
        if isinstance(v, dict):
            yield prefix + k, v
            yield from _walk(v, prefix + k + ".")


def only_decode(args, dev, pk):
    """Decode at full context on `--batch` sequences, nothing else: the command
    profiling captures of the split-KV kernel run."""
    import oracle
    import probjax_b200 as pj

    c4 = oracle.make_config(4, B=args.batch, full=True)
    q4, k4, v4, l4 = c4["q"].to(dev), c4["k"].to(dev), c4["v"].to(dev), c4["kv_lengths"].to(dev)
    by4 = 4096.0 * float(c4["kv_lengths"].sum()) + 2 * q4.numel() * 2 + args.batch * 32 * 4
    res = bench_extra("decode", lambda: pj.decode_forward(q4, k4, v4, sm_scale=c4["sm_scale"], return_lse=True),
                      args.steps, args.warmup, by4 / 1e9, "GB/s", pk["hbm_gbs"], "hbm", pk["source"])
    res["config"] = {"workload": f"GQA split-KV decode bf16 B{args.batch} Hq32 Hkv8 D128, 32768 keys each"}
    _emit(res)


def only_backward(args, dev, pk):
    """Backward of the headline shape on `--batch` batch rows, nothing else: the command
    profiling captures of the dQ and dK/dV kernels run."""
    import oracle
    import probjax_b200 as pj

    c = oracle.make_config(2, B=args.batch)
    q, k, v = c["q"].to(dev), c["k"].to(dev), c["v"].to(dev)
    o, lse = pj.attention_forward(q, k, v, sm_scale=c["sm_scale"], return_lse=True)
    g = torch.randn_like(o)
    fl = 2.5 * prefill_flops(args.batch, C2["Hq"], C2["S"], C2["S"], C2["D"], C2["D"], False)
    res = bench_extra("backward", lambda: pj.attention_backward(q, k, v, o, lse, g, sm_scale=c["sm_scale"]), args.steps,
                      args.warmup, fl / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
    res["config"] = {"workload": f"GQA attention backward bf16 B{args.batch} Hq32 Hkv8 S4096 D128 non-causal "
                                 "(FLOPs counted as 2.5 x forward)"}
    _emit(res)


def only_linear(args, dev, pk):
    """The fused QKV projection of the headline shape, [batch * 4096, 4096] x [6144, 4096]^T, nothing
    else: the command profiling captures of the projection GEMM run."""
    import probjax_b200 as pj

    d_model = 4096
    m_rows, n_out = args.batch * C2["S"], (C2["Hq"] + 2 * C2["Hkv"]) * C2["D"]
    xg = torch.randn((m_rows, d_model), device=dev).bfloat16()
    wg = (torch.randn((n_out, d_model), device=dev) / 64).bfloat16()
    res = bench_extra("linear", lambda: pj.linear(xg, wg), args.steps, args.warmup, 2.0 * m_rows * n_out * d_model / 1e12,
                      "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
    res["config"] = {"workload": f"QKV projection bf16 [{m_rows}, {d_model}] x [{n_out}, {d_model}]^T"}
    _emit(res)


def only_masked_bias(args, dev, pk):
    """The masked + biased configuration (bf16 B8 H16 S1024 D64, per-batch key lengths, fp32 bias
    [1,16,1024,1024]) on `--batch` batch rows, nothing else: the command profiling captures of the
    staged-bias instantiation of the forward kernel run."""
    import oracle
    import probjax_b200 as pj

    c3 = oracle.make_config(3, B=args.batch)
    q3, k3, v3 = c3["q"].to(dev), c3["k"].to(dev), c3["v"].to(dev)
    l3, b3 = c3["kv_lengths"].to(dev), c3["bias"].to(dev)
    fl3 = 4.0 * 16 * 1024 * 64 * float(c3["kv_lengths"].sum())
    res = bench_extra("c3", lambda: pj.attention_forward(q3, k3, v3, kv_lengths=l3, bias=b3, sm_scale=c3["sm_scale"]),
                      args.steps, args.warmup, fl3 / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
    res["config"] = {"workload": f"masked + biased attention bf16 B{args.batch} H16 S1024 D64, fp32 bias [1,16,1024,1024]",
                     "kv_lengths": c3["kv_lengths"].tolist()}
    _emit(res)


def only_latent_decode(args, dev, pk):
    """The decode step of absorbed latent attention (16 heads over a 576-wide latent cache of 32768 keys)
    on `--batch` sequences, nothing else: the command profiling captures of `decode_latent_kernel` run."""
    import probjax_b200 as pj

    Bl, Hl, Rl, Sl = args.batch, 16, 576, 32768
    gl = torch.Generator(device=dev).manual_seed(5)
    ql = torch.randn((Bl, 1, Hl, Rl), generator=gl, device=dev).bfloat16()
    cl = (torch.randn((Bl, Sl, Rl), generator=gl, device=dev) * 0.5).bfloat16()
    res = bench_extra("latent_decode", lambda: pj.mla_decode(ql, cl, sm_scale=Rl ** -0.5, impl=args.kernel), args.steps,
                      args.warmup, (cl.numel() * 2 + 2 * ql.numel() * 2) / 1e9, "GB/s", pk["hbm_gbs"], "hbm", pk["source"])
    pj.check_status(dev)
    res["config"] = {"workload": f"absorbed latent decode bf16 B{Bl} H16 R576, 32768 keys each",
                     "kernel": args.kernel or "library's choice"}
    _emit(res)


def only_waves(args, dev, pk):
    """Unmasked bf16 forward, one work item (256 query rows x 4096 keys, D = 128) per query head, for head counts
    around the multiples of the SM count: time per call and launches per call."""
    import probjax_b200 as pj
    from probjax_b200 import _lib

    g = torch.Generator(device=dev).manual_seed(0)
    k = torch.randn((1, 4096, 8, 128), device=dev, generator=g).bfloat16()
    v = torch.randn((1, 4096, 8, 128), device=dev, generator=g).bfloat16()
    out = {"config": {"workload": "GQA forward bf16, Lq 256 per head, Lkv 4096, Hkv 8, D 128, unmasked",
                      "kv_halves": os.environ.get("PJX_FWD_SPLIT_TAIL", "1") != "0"}, "items_us_launches": []}
    for items in (8, 72, 144, 152, 216, 296, 304, 368, 440, 512):
        q = torch.randn((1, 256, items, 128), device=dev, generator=g).bfloat16()
        n0 = _lib.launch_count()
        pj.attention_forward(q, k, v, sm_scale=0.088)
        launches = _lib.launch_count() - n0
        ms = time_steps(lambda: pj.attention_forward(q, k, v, sm_scale=0.088), args.steps, args.warmup) / args.steps
        out["items_us_launches"].append([items, ms * 1e3, launches])
    pj.check_status(dev)
    _emit(out)


def only_prefill(args, dev, pk):
    """The headline forward on `--batch` batch rows, non-causal and causal, timing only: the command the
    what-if builds of the forward kernel (`python -m probjax_b200.build --what-if N`, loaded through
    PJX_ATTENTION_LIB) are timed with."""
    import oracle
    import probjax_b200 as pj

    c = oracle.make_config(2, B=args.batch)
    q, k, v = c["q"].to(dev), c["k"].to(dev), c["v"].to(dev)
    out = {"config": {"workload": f"GQA prefill bf16 B{args.batch} Hq32 Hkv8 S4096 D128", "library": os.environ.get("PJX_ATTENTION_LIB", "in-tree")}}
    for name, causal in (("noncausal", False), ("causal", True)):
        fl = prefill_flops(args.batch, C2["Hq"], C2["S"], C2["S"], C2["D"], C2["D"], causal)
        res = bench_extra(name, lambda: pj.attention_forward(q, k, v, causal=causal, sm_scale=c["sm_scale"], impl=args.kernel),
                          args.steps, args.warmup, fl / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
        out[name] = {"ms": res["ms"], "tflops": res["value"]}
    _emit(out)


def only_modifier(args, dev, pk):
    """The headline shape on `--batch` batch rows under one structured mask or score term, with the mask data
    on the device: `band` is a band that never cuts (the band variant of the kernel with nothing to mask),
    `row_limits` per-row key limits that never cut and `one_segment` a single segment (the mask-only
    modifier level), `head_scale` a positive per-head scale (the full level with no work per element)."""
    import oracle
    import probjax_b200 as pj

    c = oracle.make_config(2, B=args.batch)
    q, k, v = c["q"].to(dev), c["k"].to(dev), c["v"].to(dev)
    S, H, sc = C2["S"], C2["Hq"], c["sm_scale"]
    causal = False
    kw = {}
    if args.only_modifier == "band":
        def fn():
            return pj.attention_forward(q, k, v, band=(-(1 << 20), 1 << 20), sm_scale=sc)
    else:
        if args.only_modifier == "row_limits":
            kw = dict(mask=pj.KeyPaddingMask(torch.full((S,), S, dtype=torch.int32, device=dev)))
        elif args.only_modifier == "one_segment":
            kw = dict(mask=pj.SameSegmentMask(torch.zeros((1, S), dtype=torch.int32, device=dev)))
        elif args.only_modifier == "packed_8x512":
            kw = dict(mask=pj.BlockDiagonalCausalMask((torch.arange(S, device=dev) // 512).to(torch.int32)[None]))
        elif args.only_modifier == "head_scale":
            kw = dict(bias=pj.PerHeadScaleBias(torch.linspace(0.5, 1.5, H, device=dev)))
        elif args.only_modifier == "causal_alibi":
            kw, causal = dict(mask=pj.CausalMask(), bias=pj.CausalAlibiBias()), True
        elif args.only_modifier == "soft_cap":
            kw = dict(bias=pj.SoftCappingBias(30.0))

        def fn():
            return pj.mha(q, k, v, sm_scale=sc, **kw)

    if args.only_modifier == "packed_8x512":
        fl = 8 * prefill_flops(args.batch, H, 512, 512, C2["D"], C2["D"], True)
    else:
        fl = prefill_flops(args.batch, H, S, S, C2["D"], C2["D"], causal)
    res = bench_extra(args.only_modifier, fn, args.steps, args.warmup, fl / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
    _emit({"config": {"workload": f"GQA prefill bf16 B{args.batch} Hq32 Hkv8 S4096 D128, {args.only_modifier}"},
           "ms": res.get("ms"), "tflops": res.get("value"), "error": res.get("error")})


def only_latent(args, dev, pk):
    """The latent-attention configuration (bf16 H16 S2048 causal, rank 512 + 64 rotary) on `--batch`
    batch rows, nothing else: the command profiling captures of the (192,128) instantiation of the
    forward kernel and of the up-projection GEMM at K = 576 run."""
    import oracle
    import probjax_b200 as pj

    c5 = oracle.make_config(5, B=args.batch)
    q5, ch5, wk5, wv5 = c5["q"].to(dev), c5["cache"].to(dev), c5["wk"].to(dev), c5["wv"].to(dev)
    fl5 = 2.0 * args.batch * 2048 * 512 * 16 * 256 + prefill_flops(args.batch, 16, 2048, 2048, 192, 128, True)
    res = bench_extra("c5", lambda: pj.mla(q5, ch5, wk5, wv5, mask=pj.CausalMask(), sm_scale=c5["sm_scale"]), args.steps,
                      args.warmup, fl5 / 1e12, "TFLOP/s", pk["bf16_tflops"], "tensor", pk["source"])
    res["config"] = {"workload": f"latent attention bf16 B{args.batch} H16 S2048 causal, rank 512 + 64 rotary"}
    _emit(res)


def _parity(o, lse, ref_o, ref_lse, tol_o=2e-2, tol_lse=1e-3):
    """max-abs errors of (o, lse) against a reference pair, and whether they pass the bounds."""
    eo = float((o.float() - ref_o.float()).abs().max())
    el = float((lse.float() - ref_lse.float()).abs().max())
    res = {"max_abs_err": eo, "lse_err": el}
    if not (eo <= tol_o and el <= tol_lse):
        res["parity_failure"] = f"o {eo:.3e} lse {el:.3e}"
    return res


def long_context_decode_bench(dev, rank, world, steps, warmup, pk, dist_on, context=131072):
    """The decode geometry of configuration 4 at a 128k context (device-generated
    N(0,1) cache, all keys valid): on one GPU the whole cache, on N GPUs the KV
    sequence sharded with the fused exchange.  At 8 GPUs each rank still streams 16k
    keys per sequence, so the fixed cost of the exchange is amortised.  With N > 1 the
    sharded result is compared (outside the timed region) with the one-GPU decode over
    the concatenation of all ranks' shards, which every rank regenerates from the seeds."""
    import probjax_b200 as pj
    from probjax_b200 import dist as pjd

    try:
        B, Hq, Hkv, D, page = 16, 32, 8, 128, 256
        local = context // world
        q = torch.randn((B, 1, Hq, D), generator=torch.Generator(device=dev).manual_seed(99), device=dev).bfloat16()
        # every rank holds the whole cache (8.6 GB) for the check; its own shard is a slice of it
        k_all = torch.empty((B, context, Hkv, D), device=dev, dtype=torch.bfloat16)
        v_all = torch.empty_like(k_all)
        for r in range(world):
            g = torch.Generator(device=dev).manual_seed(1234 + r)
            k_all[:, r * local:(r + 1) * local] = torch.randn((B, local, Hkv, D), generator=g, device=dev, dtype=torch.float16)
            v_all[:, r * local:(r + 1) * local] = torch.randn((B, local, Hkv, D), generator=g, device=dev, dtype=torch.float16)
        k = k_all[:, rank * local:(rank + 1) * local].contiguous() if dist_on else k_all
        v = v_all[:, rank * local:(rank + 1) * local].contiguous() if dist_on else v_all
        lens = torch.full((B,), context, dtype=torch.int32)
        sc = 1.0 / (D ** 0.5)
        ll = lens.to(dev)
        check = {}
        if dist_on:
            fn = pjd.FusedShardedDecoder(q, k, v, lens, page=page, sm_scale=sc, overlap_steps=True)
            ref = pj.decode_forward(q, k_all, v_all, kv_lengths=ll, sm_scale=sc, return_lse=True)
            o, lse = fn(return_lse=True)
            fn.check_status()
            check = _parity(o, lse, ref[0], ref[1])
            del ref
        else:

            def fn():  # every sequence is full: no lengths
                return pj.decode_forward(q, k, v, sm_scale=sc, return_lse=True)

        if dist_on:
            del k_all, v_all
        ms = max_over_ranks(time_steps(fn, steps, warmup, dist_on), dist_on) / steps
        if dist_on:
            fn.check_status()
        by = 4096.0 * B * context
        ach = by / (ms * 1e-3) / 1e9
        return dict({"ms": ms, "value": ach, "unit": "GB/s aggregate", "context": context, "n_gpus": world,
                     "bound": "hbm", "frac": ach / world / pk["hbm_gbs"]}, **check)
    except Exception as e:
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def sharded_decode_bench(c4, ref, dev, rank, world, steps, warmup, pk):
    """Decode at 32k context with the KV sequence block-cyclically sharded over
    the ranks.  Timed three ways: the fused exchange (peer stores and flags inside
    the kernels), NCCL all-gathers between the kernels, and the latter as one CUDA
    graph per step.  Outside the timed region every rank compares each variant's
    (o, lse) with `ref`, the one-GPU decode over the unsharded cache, and a few
    sequences of the fused result with the oracle."""
    import oracle
    from probjax_b200 import dist as pjd

    out = {}
    try:
        page = 256
        kl = pjd.shard_cache(c4["k"], rank, world, page).to(dev)
        vl = pjd.shard_cache(c4["v"], rank, world, page).to(dev)
        q4 = c4["q"].to(dev)
        lens = c4["kv_lengths"]
        by = 4096.0 * float(lens.sum())
        for mode in ("fused", "fused_serial", "nccl", "nccl_graph"):
            try:
                if mode.startswith("fused"):  # peer stores inside the kernel, no library collective; "fused" lets
                    # a step stream its cache while the previous step's exchange drains, "fused_serial" does not
                    dec = pjd.FusedShardedDecoder(q4, kl, vl, lens, page=page, sm_scale=c4["sm_scale"],
                                                  overlap_steps=(mode == "fused"))
                else:
                    dec = pjd.ShardedDecoder(q4, kl, vl, lens, page=page, sm_scale=c4["sm_scale"],
                                             use_graph=(mode == "nccl_graph"))
                ms = max_over_ranks(time_steps(dec, steps * 5, warmup, True), True) / (steps * 5)
                o, lse = dec(return_lse=True)
                torch.cuda.synchronize(dev)
                if mode.startswith("fused"):
                    dec.check_status()
                ach = by / (ms * 1e-3) / 1e9
                out[mode] = dict({"ms": ms, "value": ach, "unit": "GB/s aggregate", "bound": "hbm",
                                  "frac": ach / world / pk["hbm_gbs"]}, **_parity(o, lse, ref[0], ref[1]))
                if mode == "fused":  # two sequences against the CPU oracle as well
                    want, want_lse = oracle.xla_attention(c4["q"][:2], c4["k"][:2], c4["v"][:2], kv_lengths=lens[:2],
                                                          sm_scale=c4["sm_scale"], return_lse=True)
                    vs_oracle = _parity(o[:2].cpu(), lse[:2].cpu(), want, want_lse)
                    out[mode]["oracle_max_abs_err"] = vs_oracle["max_abs_err"]
                    out[mode]["oracle_lse_err"] = vs_oracle["lse_err"]
                    if "parity_failure" in vs_oracle:
                        out[mode]["parity_failure"] = "vs oracle " + vs_oracle["parity_failure"]
            except Exception as e:
                out[mode] = {"error": f"{type(e).__name__}: {e}"[:300]}
        out["page"] = page
        return out
    except Exception as e:
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def _emit(obj):
    """The one JSON line of the run, on the process's original stdout."""
    os.write(_REAL_STDOUT, (json.dumps(rounded(obj), separators=(",", ":")) + "\n").encode())


# Libraries (NCCL's version banner, for one) write to file descriptor 1; the contract is one JSON
# line on stdout, so everything else is sent to stderr and the line goes out through a saved copy.
_REAL_STDOUT = 1

if __name__ == "__main__":
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = sys.stderr
    main()
