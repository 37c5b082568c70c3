#!/usr/bin/env python
"""Throughput of the routed-expert MoE block: tokens/s of one block call over synthetic input.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl ours|reference]
                    [--workloads all|none|c0,c1_t8,...]

N = 1 runs the whole block on one B200; N > 1 (launched by torch.distributed.run, one rank per
GPU) shards the experts across ranks and the tokens with them (expert parallelism: one library
call per rank, token rows exchanged with NCCL send/recv), so the total work is fixed as N grows
("strong" scaling).  Rank 0 prints ONE JSON line: the headline fields describe `--workload`
(default c3, the shape the metric is quoted on); `workloads` holds the other named shapes, each
with its own step time, roofline fraction, parity against the CPU oracle and clock record.

`--impl reference` times the CPU restatement of the reference's own MoE block (oracle/, the Rust
original cannot be built here) on the host cores, on a bounded token sample of the same workload.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_block_tokens_per_s"
UNIT = "tokens/s"
CSRC = os.path.join(ROOT, "speedycolibri_b200", "csrc")


def measured_peaks():
    """HBM GB/s and bf16 TFLOP/s measured on this pool (driver-written file), else the fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# DRAM bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum) of the expert kernels,
# keyed by (workload, tokens, kernel).  Every entry names the kernel source it was captured from
# and the first 12 hex digits of that file's sha256 at capture time: when the file has changed
# since, the figure is stale and the bench prints null instead.  The c3 figures are the c3s capture
# (same matrices, 1/8 of the experts and tokens, so 1/8 of every stream) times 8: a full c3 launch
# holds too much on the device for a multi-pass capture.  c4 has no figure: its skewed routing leaves
# a different share of the experts active than the small case c4s, so the streams do not scale by a
# constant.  The captures are summarised under profiles/.
NCU_TRAFFIC = {
    ("c3s", 512, "gate_up"): (634600000, "profiles/k_ffn_tct_c3s_full.md", "expert_tc_tmem.cu", "2356b26d8fea"),
    ("c3s", 512, "down"): (338200000, "profiles/k_ffn_tct_c3s_full.md", "expert_tc_tmem.cu", "2356b26d8fea"),
    ("c3", 4096, "gate_up"): (5076800000, "profiles/k_ffn_tct_c3s_full.md (c3s capture x 8)", "expert_tc_tmem.cu", "2356b26d8fea"),
    ("c3", 4096, "down"): (2705600000, "profiles/k_ffn_tct_c3s_full.md (c3s capture x 8)", "expert_tc_tmem.cu", "2356b26d8fea"),
    ("c2", 512, "gate_up"): (442300000, "profiles/k_ffn_tct_c2_full.md", "expert_tc_tmem.cu", "2356b26d8fea"),
    ("c2", 512, "down"): (224100000, "profiles/k_ffn_tct_c2_full.md", "expert_tc_tmem.cu", "2356b26d8fea"),
    ("c1", 8, "gate_up"): (94800128, "profiles/k_ffn_mm_c1_full.md", "expert_small.cu", "e50bd732c27b"),
    ("c1", 8, "down"): (46207488, "profiles/k_ffn_mm_c1_full.md", "expert_small.cu", "e50bd732c27b"),
    ("c4s", 2048, "gate_up"): (1264600000, "profiles/k_ffn_tc_c4s_full.md", "expert_tc.cu", "454ac79fc581"),
    ("c4s", 2048, "down"): (715900000, "profiles/k_ffn_tc_c4s_full.md", "expert_tc.cu", "454ac79fc581"),
}


def file_stamp(name: str) -> str:
    try:
        return hashlib.sha256(open(os.path.join(CSRC, name), "rb").read()).hexdigest()[:12]
    except OSError:
        return "missing"


def ncu_traffic(workload: str, tokens: int, kernel: str):
    ent = NCU_TRAFFIC.get((workload, tokens, kernel))
    if ent is None:
        return None, None
    nbytes, source, src_file, stamp = ent
    if file_stamp(src_file) != stamp:
        return None, f"{source}: stale ({src_file} changed since the capture)"
    return nbytes, source


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()  # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.th.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def shape_named(name: str, tokens: int = 0):
    """'c3', 'c1_t4' (c1 with 4 tokens) ... -> MoeShape."""
    from speedycolibri_b200.configs import CONFIGS

    base, _, t = name.partition("_t")
    shape = CONFIGS[base]
    if t:
        shape = shape.with_tokens(int(t))
    if tokens:
        shape = shape.with_tokens(tokens)
    return shape


def config_dict(shape, world, extra=None):
    from speedycolibri_b200.configs import FMT_NVFP4

    d = {"workload": shape.name, "hidden": shape.H, "experts": shape.E, "shared_expert": shape.shared, "top_k": shape.k,
         "intermediate": shape.I, "tokens": shape.T, "weights": "nvfp4" if shape.fmt == FMT_NVFP4 else "fp8_e4m3_b128",
         "router": ("softmax" if shape.score == 0 else "sigmoid") + (f"+group{shape.n_group}/{shape.topk_group}" if shape.n_group > 1 else ""),
         "parallelism": f"ep{world}" if world > 1 else "single", "note": shape.note}
    d.update(extra or {})
    return d


# ---------------------------------------------------------------------------------------------------
# CPU side: the oracle as the timed baseline and as the parity checker
# ---------------------------------------------------------------------------------------------------
def time_oracle(L, x_bits, threads: int):
    from oracle import oracle

    oracle.set_threads(threads)
    t0 = time.perf_counter()
    res = L.moe_block(x_bits)
    return time.perf_counter() - t0, res


def cpu_baseline_figures(shape, make_layer_for, x_bits_all, budget_s: float = 25.0):
    """The CPU restatement timed on a bounded token sample, all host threads and one thread.
    make_layer_for(x_bits) -> oracle layer holding the experts those tokens route to.  The sample
    is 256 tokens (fewer only when the shape has fewer, or when a 16-token probe says 256 would
    exceed the budget: then 64); the single-thread figure uses a 16-token sample (or fewer)."""
    from oracle import oracle

    cores = oracle.hardware_threads()
    T = x_bits_all.shape[0]
    probe_n = min(T, 16)
    xp = x_bits_all[:probe_n]
    Lp = make_layer_for(xp)
    dt_probe, _ = time_oracle(Lp, xp, cores)
    n = min(T, 256)
    if n > probe_n and dt_probe / probe_n * n > budget_s:
        n = min(T, 64)
    if n > probe_n:
        xs = x_bits_all[:n]
        Ls = make_layer_for(xs)
        dt, _ = time_oracle(Ls, xs, cores)
    else:
        n, dt = probe_n, dt_probe
    dt1, _ = time_oracle(Lp, xp, 1)
    oracle.set_threads(cores)
    return {"value": n / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"first {n} of {shape.T} tokens, one pass, {cores} threads ({dt:.1f} s); tokens/s scales linearly in tokens (rows are independent)",
            "single_thread": {"value": probe_n / dt1, "unit": UNIT, "cores": 1,
                              "sample": f"first {probe_n} of {shape.T} tokens, one pass, 1 thread ({dt1:.1f} s): what the reference's matmul does (linear.rs:153-155)"}}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle
    from oracle.layers import host_sample_layer
    from speedycolibri_b200 import synth

    shape = shape_named(args.workload, args.tokens)
    cores = oracle.hardware_threads()
    oracle.set_threads(cores)
    # bounded sample, host-generated weights for the experts it touches.  The sample follows the rule
    # of the GPU arm's cpu_baseline: 256 tokens, or 64 / 16 when a 16-token probe says the whole
    # --steps/--warmup run would not end within a few minutes
    t0 = time.perf_counter()
    cache = {}
    n_tok = int(args.ref_tokens) if args.ref_tokens else min(shape.T, 16)
    x = synth.host_tokens(shape, max(n_tok, min(shape.T, 256)))
    L, n_active = host_sample_layer(shape, x[:n_tok], cache)
    if not args.ref_tokens and shape.T > n_tok:
        dt_probe, _ = time_oracle(L, x[:n_tok], cores)
        setup_per_expert = (time.perf_counter() - t0 - dt_probe) / max(1, len(cache))
        per_step_budget = 150.0 / max(1, args.steps + args.warmup)
        for want in (min(shape.T, 256), min(shape.T, 64)):
            est_step = dt_probe / n_tok * want
            est_setup = setup_per_expert * min(shape.E, want * shape.k)
            if want > n_tok and est_step <= per_step_budget and est_setup <= 90.0:
                n_tok = want
                L, n_active = host_sample_layer(shape, x[:n_tok], cache)
                break
    xs = x[:n_tok]
    setup_s = time.perf_counter() - t0
    for _ in range(args.warmup):
        L.moe_block(xs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        L.moe_block(xs)
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    value = n_tok / dt
    sample = f"{n_tok} of {shape.T} tokens per step ({n_active} routed experts + shared touched), {cores} threads; setup {setup_s:.0f}s untimed"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config_dict(shape, 1),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------
class Ctx:
    """Process-wide state of one bench run (one rank)."""

    def __init__(self, args):
        import torch

        from speedycolibri_b200 import _lib, backend

        self.args = args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            # the exchange stores into peer memory with plain stores and uses NCCL only for one-word and handle
            # all-gathers at set-up: in-switch reduction buys nothing here, and a rank that dies while its
            # memory is bound to a multicast object takes its peers with it
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
                os.environ.pop("NCCL_DEBUG")  # its banner goes to stdout, which carries the one JSON line
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        backend.init([self.local])
        self.lib = _lib.load()
        self.peaks = measured_peaks()
        self.flush_buf = None

    def barrier(self):
        import torch

        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def flush(self):
        """Evict L2: 256 MB written, then read back so that the lines a step evicts are clean
        (evicting dirty lines would charge the step for the flush's own write-back)."""
        import torch

        if self.flush_buf is None:
            self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
        self.flush_buf.fill_(1)
        self.flush_buf.view(torch.int64).sum()

    def timed(self, fn, steps, warmup, flushed=False):
        """ms per step (max over ranks, CUDA events on the current stream) and kernels launched."""
        import torch

        for _ in range(warmup):
            fn()
        self.barrier()
        n0 = self.lib.coli_b200_launch_count()
        if flushed:
            pairs = []
            for _ in range(steps):
                self.flush()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                pairs.append((a, b))
            self.barrier()
            ms = sum(a.elapsed_time(b) for a, b in pairs)
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            self.barrier()
            ms = e0.elapsed_time(e1)
        launches = self.lib.coli_b200_launch_count() - n0
        if self.dist is not None:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, launches // max(1, steps)

    def timed_with_clocks(self, fn, steps, warmup, flushed):
        import torch

        with ClockSampler(self.local) as clk:
            ms_step, launches = self.timed(fn, steps, max(3, warmup), flushed=flushed)
            # nvidia-smi needs a few hundred ms to deliver its first sample: when the timed region is
            # shorter than that, the same step keeps running (untimed, same count on every rank) so
            # that the clock record still describes the GPU under this load
            spent_ms = ms_step * steps
            if self.args.profile_run:
                spent_ms = 1e9  # under a profiler: no extra steps
            if spent_ms < 800.0:
                extra = int(min(20000, max(1, (800.0 - spent_ms) / max(ms_step, 1e-3))))
                for _ in range(extra):
                    fn()
                torch.cuda.synchronize()
        clocks = clk.summary()
        if spent_ms < 800.0 and not self.args.profile_run:
            clocks["note"] = "timed region shorter than the sampler's start-up; samples include the same step repeated after it"
        return ms_step, launches, clocks


def sample_tokens(T: int, n: int):
    return np.unique(np.linspace(0, T - 1, min(n, T)).astype(int))


def compare_with_oracle(L, x_bits, got_bits, got_idx, got_w):
    from oracle import oracle
    from speedycolibri_b200 import synth

    oracle.set_threads(oracle.hardware_threads())
    res = L.moe_block(x_bits)
    a = synth.bf16_bits_to_f32(got_bits).astype(np.float64)
    b = synth.bf16_bits_to_f32(res["out"]).astype(np.float64)
    return {"routing_exact": bool(np.array_equal(got_idx, res["idx"]) and np.array_equal(got_w.view(np.uint32), res["w"].view(np.uint32))),
            "rel_l2": float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)), "tokens_checked": int(x_bits.shape[0]),
            "tolerance": 1e-2}


def bits(t):
    import torch

    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def roofline_of(ctx, shape, phases, ms_step, active, clocks):
    """Roofline of the dominant expert kernel from the live per-phase CUDA-event times."""
    peaks = ctx.peaks
    rows = shape.T * shape.k + (shape.T if shape.shared else 0)
    n_mats = active + (1 if shape.shared else 0)
    kern = {"gate_up": dict(bytes=n_mats * 2 * shape.matrix_bytes(shape.I, shape.H) + 2 * shape.T * shape.H,
                            flops=4 * shape.H * shape.I * rows),
            "down": dict(bytes=n_mats * shape.matrix_bytes(shape.H, shape.I) + 2 * shape.T * shape.H,
                         flops=2 * shape.H * shape.I * rows)}
    dom = max(kern, key=lambda k: phases[k])
    t_s = phases[dom] * 1e-3
    # the tensor denominator follows the clock the GPU actually ran at: the burst figure while the
    # sampled SM clock stayed near its maximum, the sustained one when the power cap pulled it down
    near_max = bool(clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and clocks["sm_mhz"] >= 0.85 * clocks["sm_max_mhz"])
    tc_peak = peaks["bf16_tflops"] if near_max else peaks["bf16_tflops_sustained"]
    hbm_t = kern[dom]["bytes"] / (peaks["hbm_gbs"] * 1e9)
    tc_t = kern[dom]["flops"] / (tc_peak * 1e12)
    tf = kern[dom]["flops"] / t_s / 1e12
    gbs = kern[dom]["bytes"] / t_s / 1e9
    if tc_t > hbm_t:
        r = {"bound": "tensor", "achieved": tf, "peak": tc_peak, "unit": "TFLOP/s", "frac": tf / tc_peak,
             "peak_kind": "burst" if near_max else "sustained"}
    else:
        r = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"]}
    traffic, src = ncu_traffic(shape.name, shape.T, dom)
    r.update({"traffic": traffic, "traffic_source": src, "kernel": dom, "kernel_ms": phases[dom], "peak_source": f"of {peaks['source']}",
              "algorithmic_bytes": kern[dom]["bytes"], "algorithmic_flops": kern[dom]["flops"],
              "hbm_frac": gbs / peaks["hbm_gbs"], "tensor_frac_burst": tf / peaks["bf16_tflops"],
              "tensor_frac_sustained": tf / peaks["bf16_tflops_sustained"], "active_experts": active,
              "block_hbm_frac": shape.bytes_moved(active) / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
              "block_tensor_frac_burst": shape.flops() / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"]})
    return r


def bench_single(ctx, shape, layer, steps, warmup, headline):
    """One workload on one GPU.  `layer`: resident synthetic weights of the shape's architecture."""
    import torch

    from oracle.layers import oracle_layer_from_device
    from speedycolibri_b200 import synth
    from speedycolibri_b200.moe import Config, MoeBlock

    blk = MoeBlock(Config.from_shape(shape), layer, shape.T, device=ctx.local)
    x = synth.device_tokens(shape, device=ctx.local)
    out = torch.empty_like(x)
    # workloads whose weights could stay in the 126 MB L2 between steps get it flushed before every timed step
    flush_l2 = shape.bytes_moved(shape.E) <= 4 * 126e6
    ms_step, launches, clocks = ctx.timed_with_clocks(lambda: blk.forward(x, out), steps, warmup, flush_l2)
    res = {"ms_per_step": ms_step, "value": shape.T / (ms_step * 1e-3), "tokens": shape.T, "gpu_launches": int(launches), "clocks": clocks,
           "l2": "L2 flushed before every timed step (256 MB written, then read)" if flush_l2
           else "weights streamed per step exceed the 126 MB L2"}
    # per-phase times (measurement mode of the library: events between phases)
    blk.profile(True)
    for _ in range(steps):
        if flush_l2:
            ctx.flush()
        blk.forward(x, out)
    ms, calls = blk.phase_ms()
    blk.profile(False)
    phases = {k: v / calls for k, v in ms.items()}
    idx, w = blk.last_routing(shape.T)
    active = len(set(idx.reshape(-1).tolist()))
    res["phase_ms"] = phases
    res["roofline"] = roofline_of(ctx, shape, phases, ms_step, active, clocks)
    # parity: sampled tokens against the CPU oracle, with the experts exported from the GPU
    if not ctx.args.no_parity and not ctx.args.profile_run:
        blk.forward(x, out)
        torch.cuda.synchronize()
        toks = sample_tokens(shape.T, ctx.args.parity_tokens)
        L = oracle_layer_from_device(shape, layer, set(idx[toks].reshape(-1).tolist()))
        tt = torch.from_numpy(toks).to(ctx.dev)
        res["parity"] = compare_with_oracle(L, bits(x[tt]), bits(out[tt]), idx[toks], w[toks])
        del L
    if ctx.args.profile_run:  # a run made to be profiled: the timed and the per-phase steps only
        blk.close()
        res["e2e"] = None
        return res
    # end to end: pinned host buffers, host-pointer call (H2D + block + D2H inside the timed region)
    xh = torch.empty((shape.T, shape.H), dtype=torch.bfloat16).pin_memory()
    oh = torch.empty((shape.T, shape.H), dtype=torch.bfloat16).pin_memory()
    xh.copy_(x.cpu())
    lib_stream = torch.cuda.ExternalStream(blk.stream(), device=ctx.dev)

    def e2e_run(n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(lib_stream)
        for _ in range(n):
            blk.moe_ptr(xh.data_ptr(), oh.data_ptr(), shape.T)  # synchronous
        e1.record(lib_stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    e2e_run(2)
    e2e_ms = e2e_run(steps)
    io_bytes = shape.T * shape.H * 2
    res["e2e"] = {"value": shape.T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
                  "ms_per_step": e2e_ms}
    if headline and not ctx.args.no_cpu_baseline:
        x_bits = bits(x[:min(shape.T, 256)])
        res["cpu_baseline"] = cpu_baseline_figures(
            shape, lambda xb: oracle_layer_from_device(shape, layer, set(idx[:xb.shape[0]].reshape(-1).tolist())), x_bits)
    blk.close()
    return res


def realised_expert_load(ctx, shape, x_all):
    """Rows per expert of this batch (the realised routing histogram), computed on every rank with a
    routing-only handle: the weights an LPT placement is built from (sharding.rs:87-109)."""
    import torch

    from speedycolibri_b200 import synth
    from speedycolibri_b200.moe import Config, Layer, MoeBlock

    lay = Layer(router=synth.device_router_bits(shape, ctx.local), experts=[None] * shape.E, router_bias=synth.select_bias(shape),
                logit_bias=synth.zipf_logit_bias(shape), shared=None)
    other = (ctx.rank + 1) % ctx.world  # a handle that owns no expert needs no weights
    blk = MoeBlock(Config.from_shape(shape), lay, shape.T, device=ctx.local, ep_rank=ctx.rank, ep_world=ctx.world,
                   expert_owner=[other] * shape.E)
    idx = torch.empty((shape.T, shape.k), dtype=torch.int32, device=ctx.dev)
    w = torch.empty((shape.T, shape.k), dtype=torch.float32, device=ctx.dev)
    blk.topk_dev(x_all, idx, w, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    load = np.bincount(idx.cpu().numpy().reshape(-1), minlength=shape.E)
    blk.close()
    return load


def bench_ep(ctx, shape, steps, warmup, balanced):
    """One workload expert-parallel over the ranks of the job: experts sharded, T / world tokens per rank."""
    import torch

    from oracle.layers import make_layer
    from speedycolibri_b200 import synth
    from speedycolibri_b200.cluster import ExpertSharding, ShardedMoe, rows_per_rank
    from speedycolibri_b200.moe import Config

    world, rank, dist = ctx.world, ctx.rank, ctx.dist
    if shape.T % world:
        raise SystemExit(f"tokens {shape.T} must divide by the number of GPUs {world}")
    Tl = shape.T // world
    x_all = synth.device_tokens(shape, device=ctx.local)
    x = x_all[rank * Tl:(rank + 1) * Tl].contiguous()
    if balanced:
        sharding = ExpertSharding.balanced(world, shape.E, realised_expert_load(ctx, shape, x_all).tolist())
    else:
        sharding = ExpertSharding.new(world, shape.E)
    del x_all
    layer = synth.device_layer(shape, device=ctx.local, local_experts=sharding.local_experts(rank))
    sm = ShardedMoe(Config.from_shape(shape), layer, sharding, shape.T, ctx.local)
    out = torch.empty_like(x)
    ms_step, launches, clocks = ctx.timed_with_clocks(lambda: sm(x, out), steps, warmup, False)
    res = {"ms_per_step": ms_step, "value": shape.T / (ms_step * 1e-3), "tokens": shape.T, "gpu_launches": int(launches), "clocks": clocks,
           "placement": "balanced (LPT on the realised rows per expert, sharding.rs:87-109)" if balanced else "contiguous e*N/E (sharding.rs:197-203)",
           "l2": "per-rank weights streamed per step exceed the 126 MB L2" if shape.bytes_moved(shape.E) / world > 126e6
           else "working set may sit in L2 (no flush under torchrun)"}
    # per-stage milliseconds of rank 0 (one extra untimed pass per step, every rank takes part) and the load per rank
    res["stage_ms"] = sm.stage_ms(x, steps)
    tab = sm.block.ep_last_counts()
    rows = rows_per_rank(tab)
    res["rows_per_rank"] = {"max": int(rows.max()), "mean": float(rows.mean()), "all": rows.tolist()}
    res["dispatch_rows_per_rank"] = {"sent_max": int((tab[:, 0, :].sum(axis=1) - np.diag(tab[:, 0, :])).max()),
                                     "received_max": int((tab[:, 0, :].sum(axis=0) - np.diag(tab[:, 0, :])).max())}
    # roofline of the expert FFN stage on rank 0 (its rows, its experts)
    peaks = ctx.peaks
    ex_ms = res["stage_ms"]["experts"]
    flops = 6 * shape.H * shape.I * int(rows[0])
    byts = len(sharding.local_experts(0)) * shape.expert_bytes()
    tf, gbs = flops / (ex_ms * 1e-3) / 1e12, byts / (ex_ms * 1e-3) / 1e9
    tensor_bound = flops / (peaks["bf16_tflops"] * 1e12) > byts / (peaks["hbm_gbs"] * 1e9)
    res["roofline"] = {"bound": "tensor" if tensor_bound else "hbm", "achieved": tf if tensor_bound else gbs,
                       "peak": peaks["bf16_tflops"] if tensor_bound else peaks["hbm_gbs"], "unit": "TFLOP/s" if tensor_bound else "GB/s",
                       "frac": tf / peaks["bf16_tflops"] if tensor_bound else gbs / peaks["hbm_gbs"], "traffic": None,
                       "kernel": "expert FFN stage of rank 0 (gate+up and down)", "kernel_ms": ex_ms, "peak_source": f"of {peaks['source']}",
                       "algorithmic_bytes": byts, "algorithmic_flops": flops}
    # parity: a few tokens of every rank against the CPU oracle on rank 0
    if not ctx.args.no_parity:
        sm(x, out)
        torch.cuda.synchronize()
        per = max(1, -(-ctx.args.parity_tokens // world))
        toks = sample_tokens(Tl, per)
        idx, w = sm.block.last_routing(Tl)
        tt = torch.from_numpy(toks).to(ctx.dev)
        mine = (bits(x[tt]), bits(out[tt]), idx[toks], w[toks])
        allp = [None] * world
        dist.all_gather_object(allp, mine)
        if rank == 0:
            xb, ob, ib, wb = (np.concatenate([p[i] for p in allp]) for i in range(4))
            needed = sorted(set(ib.reshape(-1).tolist()))
            experts = [None] * shape.E
            for e in needed:  # same seeds, same quantiser: bit-identical to what the owner holds
                ex = layer.experts[e] if layer.experts[e] is not None else synth.device_expert(shape, e, ctx.local)
                experts[e] = tuple(t.export() for t in (ex.gate, ex.up, ex.down))
            shared = tuple(t.export() for t in (layer.shared.gate, layer.shared.up, layer.shared.down)) if layer.shared is not None else None
            L = make_layer(shape, layer.router, experts, shared, layer.router_bias, layer.logit_bias)
            res["parity"] = compare_with_oracle(L, xb, ob, ib, wb)
            res["parity"]["tokens_per_rank"] = int(len(toks))
        dist.barrier()
    # end to end: pinned host buffers on every rank, copies inside the timed region
    xh = torch.empty((Tl, shape.H), dtype=torch.bfloat16).pin_memory()
    oh = torch.empty((Tl, shape.H), dtype=torch.bfloat16).pin_memory()
    xh.copy_(x.cpu())
    xd = torch.empty_like(x)

    def e2e_step():
        xd.copy_(xh, non_blocking=True)
        sm(xd, out)
        oh.copy_(out, non_blocking=True)

    e2e_ms, _ = ctx.timed(e2e_step, steps, 2)
    io_bytes = Tl * shape.H * 2 * world
    res["e2e"] = {"value": shape.T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
                  "ms_per_step": e2e_ms}
    sm.close()
    return res


def run_ours(args):
    import gc

    import torch

    from speedycolibri_b200 import synth

    ctx = Ctx(args)
    world = ctx.world
    head_shape = shape_named(args.workload, args.tokens)
    if args.profile_run:
        args.workloads = "none"
    if args.workloads == "all":
        extra = ["c0", "c1_t1", "c1_t4", "c1_t8", "c2", "c4"] if world == 1 else ["c4"]
        extra = [w for w in extra if w != args.workload]
    elif args.workloads in ("none", ""):
        extra = []
    else:
        extra = [w for w in args.workloads.split(",") if w]

    layers = {}

    def layer_for(shape):  # c1_t1 / c1_t4 / c1_t8 share one set of weights
        if shape.name not in layers:
            layers.clear()
            gc.collect()
            torch.cuda.empty_cache()
            layers[shape.name] = synth.device_layer(shape, device=ctx.local)
        return layers[shape.name]

    def run(shape, headline):
        steps = args.steps if shape.T <= 8192 else max(2, min(args.steps, 5))
        if world == 1:
            return bench_single(ctx, shape, layer_for(shape), steps, args.warmup, headline)
        return bench_ep(ctx, shape, steps, args.warmup, balanced=shape.zipf_s > 0)

    head = run(head_shape, True)
    others = {}
    for name in extra:
        r = run(shape_named(name), False)
        r.pop("cpu_baseline", None)
        others[name] = r
    if ctx.rank == 0:
        line = {"metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": config_dict(head_shape, world, {"l2": head["l2"], **({"placement": head["placement"]} if "placement" in head else {})}),
                "e2e": head["e2e"], "gpu_launches": head["gpu_launches"], "clocks": head["clocks"]}
        for key in ("roofline", "cpu_baseline", "phase_ms", "stage_ms", "parity", "rows_per_rank", "dispatch_rows_per_rank"):
            if key in head:
                line[key] = head[key]
        if others:
            line["workloads"] = others
        print(json.dumps(line))
    if ctx.dist is not None:
        ctx.dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c3", help="headline workload: c0 c1 c1_t1 c1_t4 c1_t8 c2 c3 c3s c4 c4s")
    ap.add_argument("--workloads", default="all", help="other workloads reported under 'workloads': all, none, or a comma list")
    ap.add_argument("--tokens", type=int, default=0, help="override the headline workload's token count")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--parity-tokens", type=int, default=32, help="tokens checked against the CPU oracle per workload")
    ap.add_argument("--ref-tokens", type=int, default=0, help="tokens per step of the reference arm (0 = auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--profile-run", action="store_true",
                    help="for runs under ncu: only the warm-up, timed and per-phase steps of the headline workload (no clock-sample "
                         "extension, parity, end-to-end or CPU legs); implies --workloads none")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
