#!/usr/bin/env python
"""Benchmark of the B200 attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Default workload (`whisper_large_v3_encoder`): the attention of one Whisper large-v3 encoder pass —
32 layers x (20 heads x head_dim 64, 1500 frames, non-causal) — over a batch of 64 independent 30 s
segments per GPU.  One step = those 32 operator launches over the resident batch; the metric is
segments/s (whole job, all GPUs).  Inputs are synthetic N(0,1) F16 tensors (seed 2); one layer's Q/K/V
(737 MB) is larger than L2, so successive launches never hit in cache.  Under torchrun every rank runs
the same per-GPU batch (weak scaling, no data-path collective).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the reference operator
(oracle/) on the host cores instead; the reference's own ggml kernels are not in its tree.
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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: dict(kind, layers, units-per-gpu, H, Hkv, Tq, Lk, hd, ...)
    "whisper_large_v3_encoder": dict(kind="prefill", layers=32, units=64, H=20, Hkv=20, Tq=1500, Lk=1500, hd=64,
                                     kv="f16", seed=2, unit_name="segments"),
    "whisper_large_v3_decode_cross": dict(kind="decode", layers=32, units=64, H=20, Hkv=20, Tq=5, Lk=1500, hd=64,
                                          kv="f16", seed=1, unit_name="segment-steps"),
    "voxtral_decode_q8_0": dict(kind="decode", layers=30, units=8, H=32, Hkv=8, Tq=1, Lk=535, hd=128, kv="q8_0",
                                seed=3, unit_name="stream-steps"),
    # config 2, self-attention half: 5 beams of one segment over the pooled cell cache (448 private cells each,
    # padded to 2304), beam membership only in the F16 mask [n_kv, 5]
    "whisper_large_v3_decode_self": dict(kind="decode", layers=32, units=64, H=20, Hkv=20, Tq=5, Lk=2304, hd=64,
                                         kv="f16", seed=1, unit_name="segment-steps", beam_cells=448),
    # config 4, prefill half: 375 audio + 32 text tokens, causal, GQA 32/8 over a Q8_0 cache, 8 streams
    "voxtral_prefill_q8_0": dict(kind="prefill", layers=30, units=8, H=32, Hkv=8, Tq=407, Lk=407, hd=128, kv="q8_0",
                                 seed=3, unit_name="streams", causal=True),
    # roofline probe, not a BASELINE config: the FastConformer dims without the rel-pos bias (plain hd-128 prefill)
    "hd128_prefill_probe": dict(kind="prefill", layers=24, units=2, H=8, Hkv=8, Tq=7500, Lk=7500, hd=128, kv="f16",
                                seed=4, unit_name="utterances"),
    "parakeet_relpos_encoder": dict(kind="relpos", layers=24, units=2, H=8, Hkv=8, Tq=7500, Lk=7500, hd=128,
                                    kv="f16", seed=4, unit_name="utterances"),
}


# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel for one launch, from the ncu captures summarised
# under profiles/ (bytes, units per GPU of the captured launch).  Traffic grows in proportion to the units, so the
# bench scales it to its own launch size.
NCU_TRAFFIC = {
    "whisper_large_v3_encoder": (120.89e6, 8),
    "whisper_large_v3_decode_cross": (497.06e6, 64),
    "whisper_large_v3_decode_self": (760.78e6, 64),
    "voxtral_decode_q8_0": (310.18e6, 256),
    "parakeet_relpos_encoder": (103.11e6, 1),
    "hd128_prefill_probe": (48.61e6, 1),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tensor_burst=p["bf16_tflops"], tensor=p["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, tensor_burst=1590.0, tensor=1400.0, src="fallback")


class ClockSampler:
    """nvidia-smi clock/throttle sampling during the timed region (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs_np(w, units, rng):
    """One layer's operands for `units` units, numpy, in the workload's storage types."""
    from oracle import oracle as orc
    f16 = lambda shape, s=1.0: (rng.standard_normal(shape).astype(np.float32) * np.float32(s)).astype(np.float16)
    sc = 0.5 if w["seed"] == 1 else 1.0
    q = f16((units, w["H"], w["Tq"], w["hd"]), sc)
    if w["kv"] == "q8_0":
        k = orc.quantize_q8_0(rng.standard_normal((units, w["Hkv"], w["Lk"], w["hd"])).astype(np.float32))
        v = orc.quantize_q8_0(rng.standard_normal((units, w["Hkv"], w["Lk"], w["hd"])).astype(np.float32))
    else:
        k, v = f16((units, w["Hkv"], w["Lk"], w["hd"]), sc), f16((units, w["Hkv"], w["Lk"], w["hd"]), sc)
    extra = {}
    if w["kind"] == "relpos":
        extra["q_v"] = f16((units, w["H"], w["Tq"], w["hd"]))
        pe = orc.make_pos_enc(w["H"] * w["hd"], w["Tq"])
        wpos = (rng.standard_normal((w["H"] * w["hd"], w["H"] * w["hd"])) / 32.0).astype(np.float32)
        extra["r"] = np.ascontiguousarray((pe @ wpos).reshape(2 * w["Tq"] - 1, w["H"], w["hd"]).transpose(1, 0, 2))[None].astype(np.float16)
    return q, k, v, extra


def scale_of(w):
    if w["seed"] == 1:
        return 64 ** -0.25
    return w["hd"] ** -0.5


def algorithmic_work(w, units):
    """Per launch (one layer over `units` units): FLOPs for tensor-bound forms, bytes for HBM-bound ones."""
    if w["kind"] in ("prefill", "relpos"):
        flops = 4.0 * w["Tq"] * w["Lk"] * w["hd"] * w["H"] * units
        if w.get("causal"):
            flops = 2.0 * w["Tq"] * (w["Lk"] + 1) * w["hd"] * w["H"] * units   # lower triangle only
        return dict(bound="tensor", amount=flops, unit="TFLOP/s", div=1e12)
    row = w["hd"] * 2 if w["kv"] == "f16" else w["hd"] // 32 * 34
    rows = w["Tq"] * w["beam_cells"] if "beam_cells" in w else w["Lk"]    # valid cells only
    kv_bytes = 2.0 * rows * w["Hkv"] * row * units
    qo_bytes = units * w["H"] * w["Tq"] * w["hd"] * (2 + 4)
    return dict(bound="hbm", amount=kv_bytes + qo_bytes, unit="GB/s", div=1e9)


def oracle_kwargs(w, extra):
    from crispasr_b200 import abi
    kw = dict(scale=scale_of(w))
    if w["kv"] == "q8_0":
        kw["kv_type"] = abi.Q8_0
    if w["kind"] == "relpos":
        kw.update(q_v=extra["q_v"], r=extra["r"])
    if w.get("causal"):
        kw.update(causal=True, n_past=0)
    return kw


def host_threads():
    """Host threads this process may use.  torchrun exports OMP_NUM_THREADS=1, which would turn the CPU arm into a
    single-thread run: the thread count is passed to the oracle explicitly instead."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def gpu_local_cpus(index):
    """CPUs of the NUMA node the GPU's PCIe slot hangs off (sysfs local_cpulist), restricted to this process's
    affinity mask; None when the topology cannot be read.  Pinned staging buffers allocated by a thread bound to
    these CPUs land in the memory next to the GPU, which matters once several ranks copy at the same time."""
    try:
        import torch
        p = torch.cuda.get_device_properties(index)
        path = f"/sys/bus/pci/devices/{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0/local_cpulist"
        cpus = set()
        for part in open(path).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        return cpus or None
    except Exception:
        return None


def cpu_sample(w, budget_s, steps=None):
    """Times the oracle on one unit, layer after layer, until `budget_s` or all layers; returns
    (units/s for the full layer stack, description, threads)."""
    from oracle import oracle as orc
    rng = np.random.default_rng(w["seed"])
    q, k, v, extra = make_inputs_np(w, 1, rng)
    kw = oracle_kwargs(w, extra)
    kw["n_threads"] = host_threads()
    t0, done = time.perf_counter(), 0
    # layer after layer (every layer has the same shapes), wrapping around the stack until the budget is used
    while done < 16 * w["layers"] and (time.perf_counter() - t0 < budget_s or done == 0):
        orc.flash_attn_ext(q, k, v, **kw)
        done += 1
    dt = time.perf_counter() - t0
    per_layer = dt / done
    return (1.0 / (per_layer * w["layers"]),
            f"1 {w['unit_name'][:-1]} x {done} layer passes of a {w['layers']}-layer stack ({dt:.1f} s)", kw["n_threads"])


def run_reference(args, w, rank, world):
    """--impl reference: the CPU restatement of the reference operator on the host cores (rank 0 only)."""
    if rank != 0:
        return
    from oracle import oracle as orc
    rng = np.random.default_rng(w["seed"])
    q, k, v, extra = make_inputs_np(w, 1, rng)
    kw = oracle_kwargs(w, extra)
    kw["n_threads"] = host_threads()
    layers_per_step = w["layers"] if w["kind"] != "relpos" else 1
    def step():
        for _ in range(layers_per_step):
            orc.flash_attn_ext(q, k, v, **kw)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = 1.0 / (dt * w["layers"] / layers_per_step)
    unit = f"{w['unit_name']}/s"
    line = {
        "impl": "reference", "metric": f"attention {unit} ({args.workload})", "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 softmax/accumulate over f16/q8_0 operands",
        "data": "synthetic", "config": config_of(args, w, args.units or w["units"]),
        "cpu_baseline": {"value": value, "unit": unit, "cores": kw["n_threads"], "kind": "port",
                         "sample": f"1 {w['unit_name'][:-1]} x {layers_per_step} of {w['layers']} layers per step, scaled to the full stack"},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "reference ggml kernels are absent from the reference tree (empty submodule); this is the CPU restatement (oracle/)",
    }
    print(json.dumps(line))


def config_of(args, w, units):
    return {"workload": args.workload, "layers": w["layers"], f"{w['unit_name']}_per_gpu": units, "heads": w["H"],
            "kv_heads": w["Hkv"], "head_dim": w["hd"], "q_len": w["Tq"], "kv_len": w["Lk"], "kv_type": w["kv"],
            "q_type": "f16", "sharding": "units across GPUs, no collective", "launch": "python loop" if args.no_graph else "cuda graph of one step",
            "l2": "inputs of one launch exceed L2" if w["kind"] == "prefill" else "L2 flushed between steps"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="whisper_large_v3_encoder", choices=list(WORKLOADS))
    ap.add_argument("--units", type=int, default=0, help="units per GPU (default: the workload's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--kernel", default="auto", choices=["auto", "tile"])
    ap.add_argument("--decode-splits", type=int, default=0, help="force the split count of the split-KV decode kernel (A/B runs)")
    ap.add_argument("--no-graph", action="store_true", help="launch each layer from Python instead of replaying a CUDA graph")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return

    import torch
    import torch.distributed as dist
    import crispasr_b200 as b200
    from crispasr_b200 import abi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    b200.lib()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if args.kernel == "tile":
        b200.lib().b200_set_kernel_override(abi.KERNEL_TILE_MMA)
    if args.decode_splits:
        b200.lib().b200_set_decode_splits(args.decode_splits)

    units = args.units or w["units"]
    rng = np.random.default_rng(w["seed"] + 1000 * rank)
    # generate one unit's worth on the host and tile it with per-unit sign flips/rolls: cheap and still random-like
    gen_units = min(units, 4)
    q_np, k_np, v_np, extra = make_inputs_np(w, gen_units, rng)
    rep = -(-units // gen_units)
    def up(a):
        t = torch.from_numpy(a).to(dev)
        t = t.repeat((rep,) + (1,) * (t.dim() - 1))[:units].contiguous()
        return t
    q, k, v = up(q_np), up(k_np), up(v_np)
    if w["kind"] == "decode":
        # K/V live in cache slabs as the allocator lays them out: head-major rows, the row count per head
        # rounded up to 32 so every head starts 16-byte aligned; the op sees a view of the first Lk rows.
        ctx_rows = -(-w["Lk"] // 32) * 32
        def slab(t):
            buf = torch.zeros(t.shape[:2] + (ctx_rows, t.shape[3]), dtype=t.dtype, device=dev)
            buf[:, :, : w["Lk"]] = t
            return buf[:, :, : w["Lk"]]
        k, v = slab(k), slab(v)
    kw = dict(scale=scale_of(w))
    if w["kv"] == "q8_0":
        kw["kv_type"] = abi.Q8_0
    if w["kind"] == "relpos":
        kw["q_v"], kw["r"] = up(extra["q_v"]), torch.from_numpy(extra["r"]).to(dev)
    if w.get("causal"):
        kw["causal"], kw["n_past"] = True, 0
    mask = None
    if "beam_cells" in w:
        from oracle import oracle as orc_mask
        L, beams = w["beam_cells"], w["Tq"]
        cell_pos = np.full(w["Lk"], 10 ** 6, np.int32)
        bits = np.zeros(w["Lk"], np.uint32)
        for jb in range(beams):
            cell_pos[jb * L:(jb + 1) * L], bits[jb * L:(jb + 1) * L] = np.arange(L), 1 << jb
        m = orc_mask.whisper_beam_mask(cell_pos, bits, tok_seq=np.arange(beams), tok_pos=np.full(beams, L - 1))
        mask = torch.from_numpy(m[None, None]).to(dev)
    out = torch.empty((units, w["Tq"], w["H"], w["hd"]), dtype=torch.float32, device=dev)
    ws_bytes = b200.workspace_bytes(q, k, v, mask, **kw)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    kernel_id, n_splits = b200.plan(q, k, v, mask, **kw)
    launches_per_layer = 1 + (1 if (kernel_id == abi.KERNEL_DECODE_SPLIT and n_splits > 1) else 0)
    if kernel_id == abi.KERNEL_PREFILL_TC5 and ws_bytes:
        launches_per_layer += 2   # K and V conversion pre-pass
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if w["kind"] != "prefill" else None

    def step():
        for _ in range(w["layers"]):
            b200.flash_attn_ext(q, k, v, mask, out=out, workspace=ws, **kw)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step()                      # first call outside any capture (function attributes, tensor maps, lazy init)
    torch.cuda.synchronize()
    run_step = step
    if not args.no_graph:
        # the layer loop is launch-bound from Python for the small decode shapes: capture one step
        # (all layers) into a CUDA graph and replay it, as a runtime would
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run_step = graph.replay
    for _ in range(max(args.warmup, 0)):
        run_step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for s in range(args.steps):
        if flush is not None:
            flush.fill_(s & 0xFF)        # evict L2 between steps (outside the event pair)
        ev[s][0].record()
        run_step()
        ev[s][1].record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    step_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = float(sum(step_ms))
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = units * world / (ms_per_step * 1e-3)

    # ---- end to end: host buffers through the C-ABI host entry point, H2D + D2H inside the timed region ----
    e2e = None
    if not args.no_e2e:
        e2e_units = min(units, 16 if w["kind"] == "prefill" else units)
        affinity0 = os.sched_getaffinity(0)
        near_cpus = gpu_local_cpus(dev.index if dev.index is not None else 0)
        if near_cpus:
            os.sched_setaffinity(0, near_cpus)   # staging buffers next to the GPU; restored after the measurement
        hq, hk, hv = (x[:e2e_units].contiguous().cpu().pin_memory() for x in (q, k, v))
        hkw = dict(kw)
        if w["kind"] == "relpos":
            hkw["q_v"], hkw["r"] = kw["q_v"][:e2e_units].cpu().pin_memory(), kw["r"].cpu().pin_memory()
        hmask = mask.cpu().pin_memory() if mask is not None else None
        hout = torch.empty((e2e_units, w["Tq"], w["H"], w["hd"]), dtype=torch.float32).pin_memory()
        e2e_layers = w["layers"]
        def e2e_step():
            for _ in range(e2e_layers):
                b200.flash_attn_ext_host(hq, hk, hv, hmask, out=hout, **hkw)
        e2e_step()
        barrier()
        n_e2e = max(1, min(args.steps, 3))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / n_e2e
        if world > 1:
            t = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        h2d = sum(int(x.numel() * x.element_size()) for x in (hq, hk, hv)) + sum(
            int(hkw[n].numel() * hkw[n].element_size()) for n in ("q_v", "r") if n in hkw)
        e2e = {"value": e2e_units * world / dt, "unit": f"{w['unit_name']}/s", "h2d_bytes_per_step": h2d * e2e_layers,
               "d2h_bytes_per_step": int(hout.numel() * 4) * e2e_layers, "units_per_gpu": e2e_units,
               "api": "b200_fattn_forward_host (pinned host buffers, per-layer H2D of Q/K/V and D2H of the output)"}
        e2e["host_cpus"] = f"{len(near_cpus)} of {len(affinity0)} (NUMA-local to the GPU)" if near_cpus else f"{len(affinity0)} (topology unknown)"
        os.sched_setaffinity(0, affinity0)
        b200.lib().b200_host_arena_release()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    work = algorithmic_work(w, units)
    launch_s = (sum(step_ms) / args.steps) * 1e-3 / w["layers"]
    achieved = work["amount"] / launch_s / work["div"]
    peak = pk["tensor"] if work["bound"] == "tensor" else pk["hbm"]
    roofline = {"bound": work["bound"], "achieved": achieved, "peak": peak, "unit": work["unit"],
                "frac": achieved / peak,
                "traffic": (NCU_TRAFFIC[args.workload][0] * units / NCU_TRAFFIC[args.workload][1]
                            if args.workload in NCU_TRAFFIC else None),
                "traffic_source": "ncu capture under profiles/, scaled by units" if args.workload in NCU_TRAFFIC else None,
                "peak_source": f"{pk['src']} ({'sustained bf16 GEMM' if work['bound'] == 'tensor' else 'copy'})",
                "kernel": abi.KERNEL_NAMES[kernel_id], "launch_ms": launch_s * 1e3,
                "algorithmic_per_launch": work["amount"]}
    line = {
        "metric": f"attention {w['unit_name']}/s ({args.workload})", "value": value, "unit": f"{w['unit_name']}/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 operands, f32 softmax/accumulate" if w["kv"] == "f16" else "q8_0 KV dequantised in-kernel, f32 softmax/accumulate",
        "data": "synthetic", "config": config_of(args, w, units), "roofline": roofline, "clocks": clocks,
        "gpu_launches": launches_per_layer * w["layers"] * args.steps, "e2e": e2e,
    }
    if not args.no_cpu_baseline:
        val, sample, cores = cpu_sample(w, budget_s=12.0)
        line["cpu_baseline"] = {"value": val, "unit": f"{w['unit_name']}/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
