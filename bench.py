#!/usr/bin/env python
"""Throughput of the routed-expert MoE block: tokens/s of one block call over synthetic input.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl ours|reference]

N = 1 runs the whole block on one B200; N > 1 (launched by torch.distributed.run, one rank per
GPU) shards the experts across ranks (expert parallelism: NCCL all-gather of tokens, reduce-scatter of
partial sums) and the tokens with
them, so the total work is fixed as N grows ("strong" scaling).  Rank 0 prints ONE JSON line.

`--impl reference` times the CPU restatement of the reference's own MoE block (oracle/, the Rust
original cannot be built here) on the host cores, on a bounded token sample of the same workload.
"""
from __future__ import annotations

import argparse
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


def measured_peaks():
    """HBM GB/s and bf16 TFLOP/s measured on this pool (driver-written file), else the fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# DRAM bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum) of the expert kernels,
# keyed by (workload, tokens, kernel).  The c3 figures are the c3s capture (same matrices, 1/8 of
# the experts and tokens, so 1/8 of every stream) times 8: a full c3 launch holds too much on
# the device for a multi-pass capture.  The captures are summarised under profiles/.
NCU_TRAFFIC = {
    ("c3", 4096, "gate_up"): (8 * (663724800 + 11862528), "profiles/k_ffn_tct_c3s_full.md, c3s capture x 8"),
    ("c3", 4096, "down"): (8 * (304030720 + 24761344), "profiles/k_ffn_tct_c3s_full.md, c3s capture x 8"),
    ("c3s", 512, "gate_up"): (663724800 + 11862528, "profiles/k_ffn_tct_c3s_full.md"),
    ("c3s", 512, "down"): (304030720 + 24761344, "profiles/k_ffn_tct_c3s_full.md"),
    ("c2", 512, "gate_up"): (424864512 + 3916288, "profiles/k_ffn_tct_c2_full.md"),
    ("c2", 512, "down"): (210126336 + 5060352, "profiles/k_ffn_tct_c2_full.md"),
    ("c1", 8, "gate_up"): (92070144 + 2123008, "profiles/k_ffn_mm_c1_full.md"),
    ("c1", 8, "down"): (46130688 + 72192, "profiles/k_ffn_mm_c1_full.md"),
}


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


def shape_for(args):
    from speedycolibri_b200.configs import CONFIGS

    shape = CONFIGS[args.workload]
    if args.tokens:
        shape = shape.with_tokens(args.tokens)
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
# reference arm: the CPU restatement on the host cores
# ---------------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle
    from speedycolibri_b200 import synth

    shape = shape_for(args)
    cores = oracle.hardware_threads()
    oracle.set_threads(cores)
    # bounded sample: the block is row-independent, so tokens/s on a few tokens is the CPU rate
    per_token_gflop = 6 * shape.H * shape.I * (shape.k + (1 if shape.shared else 0)) / 1e9
    n_tok = max(1, min(shape.T, int(args.ref_tokens) if args.ref_tokens else max(1, int(2.0 / max(per_token_gflop, 1e-3)))))
    x = synth.host_tokens(shape, n_tok)
    t0 = time.perf_counter()
    from oracle.layers import host_sample_layer

    L, n_active = host_sample_layer(shape, x)
    setup_s = time.perf_counter() - t0
    for _ in range(args.warmup):
        L.moe_block(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        L.moe_block(x)
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
def cpu_baseline_sample(shape, layer, x_dev, idx_all, n_tok):
    """Time the oracle on the first n_tok tokens with the experts exported from the GPU run."""
    import torch
    from oracle import oracle
    from oracle.layers import oracle_layer_from_device

    cores = oracle.hardware_threads()
    oracle.set_threads(cores)
    needed = set(idx_all[:n_tok].reshape(-1).tolist())
    L = oracle_layer_from_device(shape, layer, needed)
    xh = x_dev[:n_tok].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    t0 = time.perf_counter()
    res = L.moe_block(xh)
    dt = time.perf_counter() - t0
    return {"value": n_tok / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"first {n_tok} of {shape.T} tokens, one pass, {len(needed)} routed experts + shared, {cores} threads"}, res


def run_ours(args):
    import torch

    from speedycolibri_b200 import _lib, backend, synth
    from speedycolibri_b200.cluster import ExpertSharding, moe_sharded, verify_peers
    from speedycolibri_b200.moe import Config, MoeBlock

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
            os.environ.pop("NCCL_DEBUG")  # its banner goes to stdout, which carries the one JSON line
        dist.init_process_group("nccl", device_id=dev)
    backend.init([local])
    shape = shape_for(args)
    peaks = measured_peaks()
    cfg = Config.from_shape(shape)
    lib = _lib.load()

    if shape.T % world:
        raise SystemExit(f"tokens {shape.T} must divide by the number of GPUs {world}")
    Tl = shape.T // world
    x_all = synth.device_tokens(shape, device=local)
    x = x_all[rank * Tl:(rank + 1) * Tl].contiguous()
    if world == 1:
        layer = synth.device_layer(shape, device=local)
        blk = MoeBlock(cfg, layer, shape.T, device=local)
        out = torch.empty_like(x)
        step = lambda: blk.forward(x, out)
    else:
        sharding = ExpertSharding.new(world, shape.E)
        verify_peers(sharding)
        layer = synth.device_layer(shape, device=local, local_experts=sharding.local_experts(rank))
        blk = MoeBlock(cfg, layer, shape.T, device=local, ep_rank=rank, ep_world=world)
        step = lambda: moe_sharded(blk, sharding, x)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # Workloads whose weights could stay in the 126 MB L2 between steps get the L2 flushed before
    # every timed step: 256 MB written, then read back so that the lines a step evicts are clean
    # (evicting dirty lines would charge the step for the flush's own write-back).
    flush_l2 = world == 1 and shape.bytes_moved(shape.E) <= 4 * 126e6
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush_l2 else None

    def flush():
        if flush_buf is not None:
            flush_buf.fill_(1)
            flush_buf.view(torch.int64).sum()

    def timed(fn, steps, warmup, flushed=False):
        for _ in range(warmup):
            fn()
        barrier()
        n0 = lib.coli_b200_launch_count()
        if flushed and flush_buf is not None:
            pairs = []
            for _ in range(steps):
                flush()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                pairs.append((a, b))
            barrier()
            ms = sum(a.elapsed_time(b) for a, b in pairs)
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1)
        launches = lib.coli_b200_launch_count() - n0
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, launches

    with ClockSampler(local) as clk:
        ms_step, launches = timed(step, args.steps, max(3, args.warmup), flushed=True)
        # nvidia-smi needs a few hundred ms to deliver its first sample: when the timed region is
        # shorter than that, the same step keeps running (untimed, same count on every rank) so
        # that the clock record still describes the GPU under this load
        spent_ms = ms_step * args.steps
        if spent_ms < 800.0:
            extra = int(min(20000, max(1, (800.0 - spent_ms) / max(ms_step, 1e-3))))
            for _ in range(extra):
                step()
            torch.cuda.synchronize()
    clocks = clk.summary()
    if spent_ms < 800.0:
        clocks["note"] = "timed region shorter than the sampler's start-up; samples include the same step repeated after it"
    value = shape.T / (ms_step * 1e-3)

    # ---- end to end: pinned host buffers, copies inside the timed region --------------------------
    xh = torch.empty((Tl, shape.H), dtype=torch.bfloat16).pin_memory()
    oh = torch.empty((Tl, shape.H), dtype=torch.bfloat16).pin_memory()
    xh.copy_(x.cpu())
    if world == 1:
        lib_stream = torch.cuda.ExternalStream(blk.stream(), device=dev)

        def e2e_run(steps):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(lib_stream)
            for _ in range(steps):
                blk.moe_ptr(xh.data_ptr(), oh.data_ptr(), Tl)  # H2D + block + D2H, synchronous
            e1.record(lib_stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / steps

        e2e_run(2)
        e2e_ms = e2e_run(args.steps)
    else:
        xd = torch.empty_like(x)

        def e2e_step():
            xd.copy_(xh, non_blocking=True)
            o = moe_sharded(blk, sharding, xd)
            oh.copy_(o, non_blocking=True)

        e2e_ms, _ = timed(e2e_step, args.steps, 2)
    io_bytes = Tl * shape.H * 2 * world
    e2e = {"value": shape.T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
           "ms_per_step": e2e_ms}

    # ---- roofline of the dominant kernel + CPU baseline (single GPU, rank 0) -------------------------
    roofline, cpu_base, phases, parity = None, None, None, None
    if world == 1:
        blk.profile(True)
        for _ in range(args.steps):
            flush()
            blk.forward(x, out)
        ms, calls = blk.phase_ms()
        blk.profile(False)
        phases = {k: v / calls for k, v in ms.items()}
        idx, _w = blk.last_routing(shape.T)
        active = len(set(idx.reshape(-1).tolist()))
        rows = shape.T * shape.k + (shape.T if shape.shared else 0)
        n_mats = active + (1 if shape.shared else 0)
        kern = {"gate_up": dict(bytes=n_mats * 2 * shape.matrix_bytes(shape.I, shape.H) + 2 * shape.T * shape.H,
                                flops=4 * shape.H * shape.I * rows),
                "down": dict(bytes=n_mats * shape.matrix_bytes(shape.H, shape.I) + 2 * shape.T * shape.H,
                             flops=2 * shape.H * shape.I * rows)}
        dom = max(kern, key=lambda k: phases[k])
        t_s = phases[dom] * 1e-3
        hbm_t = kern[dom]["bytes"] / (peaks["hbm_gbs"] * 1e9)
        tc_peak = peaks["bf16_tflops_sustained"]
        tc_t = kern[dom]["flops"] / (tc_peak * 1e12)
        if tc_t > hbm_t:
            ach = kern[dom]["flops"] / t_s / 1e12
            roofline = {"bound": "tensor", "achieved": ach, "peak": tc_peak, "unit": "TFLOP/s", "frac": ach / tc_peak}
        else:
            ach = kern[dom]["bytes"] / t_s / 1e9
            roofline = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"]}
        traffic = NCU_TRAFFIC.get((shape.name, shape.T, dom))
        roofline.update({"traffic": traffic[0] if traffic else None, "traffic_source": traffic[1] if traffic else None, "kernel": dom, "kernel_ms": phases[dom], "peak_source": f"of {peaks['source']}",
                         "algorithmic_bytes": kern[dom]["bytes"], "algorithmic_flops": kern[dom]["flops"],
                         "hbm_frac": kern[dom]["bytes"] / t_s / 1e9 / peaks["hbm_gbs"],
                         "tensor_frac_bf16": kern[dom]["flops"] / t_s / 1e12 / tc_peak, "active_experts": active})
        whole = {"bytes": shape.bytes_moved(active), "flops": shape.flops()}
        roofline["block_hbm_frac"] = whole["bytes"] / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]
        roofline["block_tensor_frac_bf16"] = whole["flops"] / (ms_step * 1e-3) / 1e12 / tc_peak
        if not args.no_cpu_baseline:
            n_tok = max(1, min(shape.T, args.cpu_tokens))
            cpu_base, res = cpu_baseline_sample(shape, layer, x, idx, n_tok)
            torch.cuda.synchronize()
            got = out[:n_tok].view(torch.int16).cpu().numpy().view(np.uint16)
            a = synth.bf16_bits_to_f32(got).astype(np.float64)
            b = synth.bf16_bits_to_f32(res["out"]).astype(np.float64)
            parity = {"routing_exact": bool(np.array_equal(idx[:n_tok], res["idx"])),
                      "rel_l2": float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)), "tokens_checked": n_tok}

    if world > 1 and os.environ.get("COLI_EP_PROFILE"):
        tm = {}
        for _ in range(args.steps):
            blk._sharded(x, timing=tm)
        if rank == 0:
            print("EP stage ms/step:", {k: round(v / args.steps, 4) for k, v in tm.items()}, file=sys.stderr)
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": config_dict(shape, world, {"l2": "L2 flushed before every timed step (256 MB written, then read)" if flush_l2
                                                     else "weights streamed per step exceed the 126 MB L2" if shape.bytes_moved(shape.E) > 4 * 126e6
                                                     else "working set may sit in L2 (no flush under torchrun)"}),
                "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks}
        if roofline:
            line["roofline"] = roofline
        if cpu_base:
            line["cpu_baseline"] = cpu_base
        if phases:
            line["phase_ms"] = phases
        if parity:
            line["parity"] = parity
        print(json.dumps(line))
    blk.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--tokens", type=int, default=0, help="override the workload's token count")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-tokens", type=int, default=2, help="tokens of the bounded CPU-baseline sample")
    ap.add_argument("--ref-tokens", type=int, default=0, help="tokens per step of the reference arm (0 = auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
