#!/usr/bin/env python
"""Benchmark of the B200 attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Default workload (`whisper_large_v3_encoder`): the attention of one Whisper large-v3 encoder pass —
32 layers x (20 heads x head_dim 64, 1500 frames, non-causal) — over a batch of 64 independent 30 s
segments per GPU.  One step = those 32 operator launches over the resident batch; the metric is
segments/s (whole job, all GPUs).  Inputs are synthetic N(0,1) F16 tensors (seed 2); one layer's Q/K/V
(737 MB) is larger than L2, so successive launches never hit in cache.  Under torchrun every rank runs
the same per-GPU batch (weak scaling, no data-path collective).

Prints ONE JSON line (rank 0).  Besides the headline keys it carries
  * `workloads`: the other configurations of the path (decode over F16 and Q8_0 caches, causal prefill over
    a Q8_0 cache, the fused relative-position encoder), each measured in the same process for a few steps
    with its own roofline figure and clock record (1-GPU runs only; `--no-extra` skips it);
  * `strong`: the fixed 64-segment batch partitioned over the N GPUs by the library's own scheduler
    (`b200_sched_run_batched`, one host worker thread per GPU inside ONE process), timed by wall clock on the
    host after a device synchronise — the strong-scaling counterpart of the weak-scaling headline.

`--impl reference` times the CPU restatement of the reference operator (oracle/) on the host cores instead;
the reference's own ggml kernels are not in its tree.

`--record-traffic CSV [CSV ...]` is not a benchmark: it reads ncu exports made with
    ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --print-units base --clock-control none \
        -k regex:<kernel> -s <skip> -c 1 --csv --log-file traffic_<W>_u<U>.csv python bench.py --workload W --units U \
        --steps 1 --warmup 1 --no-cpu-baseline --no-e2e --no-graph --no-extra
and rewrites the table of measured DRAM traffic per launch that `roofline.traffic` is taken from.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import re
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
    # decoder self-attention: 5 beams of one segment over the pooled cell cache (448 private cells each,
    # padded to 2304), beam membership only in the F16 mask [n_kv, 5]
    "whisper_large_v3_decode_self": dict(kind="decode", layers=32, units=64, H=20, Hkv=20, Tq=5, Lk=2304, hd=64,
                                         kv="f16", seed=1, unit_name="segment-steps", beam_cells=448),
    # the same step over a pool as a running beam search leaves it: 3584 cells, the 5 beams share a 224-token prefix
    # and own 224 private cells each, scattered over the pool.  "dense" is the reference's form (every beam row scans
    # every pooled cell through the F16 membership mask), "index" makes each beam a batch entry that gathers its own
    # 448 cells through ext->kv_index, "union" keeps the beams as query rows over ONE list of the 1344 live cells with
    # a compact mask over its entries.  Algorithmic bytes of all three: the 1344 live cells, read once.
    "whisper_large_v3_decode_self_pool_dense": dict(kind="decode", layers=32, units=64, H=20, Hkv=20, Tq=5, Lk=3584, hd=64,
                                                    kv="f16", seed=1, unit_name="segment-steps", pool=(224, 224, "dense")),
    "whisper_large_v3_decode_self_pool_union": dict(kind="decode", layers=32, units=64, H=20, Hkv=20, Tq=5, Lk=3584, hd=64,
                                                    kv="f16", seed=1, unit_name="segment-steps", pool=(224, 224, "union")),
    "whisper_large_v3_decode_self_pool_index": dict(kind="decode", layers=32, units=64, H=20, Hkv=20, Tq=5, Lk=3584, hd=64,
                                                    kv="f16", seed=1, unit_name="segment-steps", pool=(224, 224, "index")),
    # LLM prefill: 375 audio + 32 text tokens, causal, GQA 32/8 over a Q8_0 cache, 8 streams
    "voxtral_prefill_q8_0": dict(kind="prefill", layers=30, units=8, H=32, Hkv=8, Tq=407, Lk=407, hd=128, kv="q8_0",
                                 seed=3, unit_name="streams", causal=True),
    # roofline probe, not one of the path's model configurations: the FastConformer dims without the rel-pos bias
    "hd128_prefill_probe": dict(kind="prefill", layers=24, units=2, H=8, Hkv=8, Tq=7500, Lk=7500, hd=128, kv="f16",
                                seed=4, unit_name="utterances"),
    # the same for head_dim 64: the encoder kernel with 48 KV tiles per CTA instead of 12 (set-up amortised)
    "hd64_prefill_probe": dict(kind="prefill", layers=8, units=4, H=20, Hkv=20, Tq=6000, Lk=6000, hd=64, kv="f16",
                               seed=2, unit_name="utterances"),
    "parakeet_relpos_encoder": dict(kind="relpos", layers=24, units=2, H=8, Hkv=8, Tq=7500, Lk=7500, hd=128,
                                    kv="f16", seed=4, unit_name="utterances"),
}

# (workload, units per GPU or None for the workload's own) measured into the `workloads` object of a 1-GPU run
EXTRA = [("whisper_large_v3_decode_cross", None), ("whisper_large_v3_decode_self", None),
         ("whisper_large_v3_decode_self_pool_dense", None), ("whisper_large_v3_decode_self_pool_index", None),
         ("whisper_large_v3_decode_self_pool_union", None), ("voxtral_decode_q8_0", 8),
         ("voxtral_decode_q8_0", 256), ("voxtral_prefill_q8_0", None), ("parakeet_relpos_encoder", None)]

TRAFFIC_TABLE = os.path.join(ROOT, "profiles", "dram_traffic.md")


def read_traffic():
    """{workload: (dram bytes read + written per launch, units in that launch)} from the table of ncu captures."""
    out = {}
    if not os.path.exists(TRAFFIC_TABLE):
        return out
    for ln in open(TRAFFIC_TABLE):
        f = [x.strip() for x in ln.strip().strip("|").split("|")]
        if len(f) >= 5 and f[0] in WORKLOADS and f[1].isdigit():
            try:
                out[f[0]] = (float(f[3]) + float(f[4]), int(f[1]))
            except ValueError:
                pass
    return out


def record_traffic(paths):
    """Rewrites the traffic table from ncu CSV exports (see the module docstring for the capture command)."""
    rows = {}
    for path in paths:
        text = open(path, errors="replace").read()
        m = re.match(r"traffic_(\w+?)_u(\d+)\.csv$", os.path.basename(path))   # traffic_<workload>_u<units>.csv
        if not m or m.group(1) not in WORKLOADS:
            print(f"{path}: name it traffic_<workload>_u<units>.csv", file=sys.stderr)
            continue
        workload, units = m.group(1), int(m.group(2))
        start = text.find('"ID"')
        if start < 0:
            print(f"{path}: no ncu CSV table found", file=sys.stderr)
            continue
        vals, kernel = {}, ""
        for r in csv.DictReader(text[start:].splitlines()):
            name = r.get("Metric Name", "")
            if name in ("dram__bytes_read.sum", "dram__bytes_write.sum") and name not in vals:
                vals[name] = float(r["Metric Value"].replace(",", ""))
                kernel = r.get("Kernel Name", "")
        if len(vals) == 2:
            rows[workload] = (units, kernel.split("(")[0], vals["dram__bytes_read.sum"], vals["dram__bytes_write.sum"], os.path.basename(path))
    old = {}
    if os.path.exists(TRAFFIC_TABLE):
        for ln in open(TRAFFIC_TABLE):
            f = [x.strip() for x in ln.strip().strip("|").split("|")]
            if len(f) >= 6 and f[0] in WORKLOADS and f[1].isdigit():
                old[f[0]] = (int(f[1]), f[2], float(f[3]), float(f[4]), f[5])
    old.update(rows)
    with open(TRAFFIC_TABLE, "w") as f:
        f.write("# DRAM traffic per launch of each workload's dominant kernel\n\n"
                "`dram__bytes_read.sum` and `dram__bytes_write.sum` of ONE launch, from ncu captures of the command\n\n"
                "    ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --print-units base --clock-control none \\\n"
                "        -k regex:<kernel> -s <launches before it> -c 1 --csv --log-file <dir>/traffic_<workload>_u<units>.csv \\\n"
                "        python bench.py --workload <workload> --units <units> --steps 1 --warmup 1 --no-cpu-baseline --no-e2e --no-graph --no-extra\n\n"
                "written by `python bench.py --record-traffic <dir>/traffic_*.csv`.  `bench.py` scales a row to the units of\n"
                "its own launch (every unit reads its own operands once and writes its own output: traffic grows in proportion).\n\n"
                "| workload | units in the captured launch | kernel | bytes read | bytes written | capture |\n|---|---|---|---|---|---|\n")
        for name in sorted(old):
            u, k, rd, wr, src = old[name]
            f.write(f"| {name} | {u} | {k} | {rd:.0f} | {wr:.0f} | {src} |\n")
    print(f"wrote {TRAFFIC_TABLE}: {sorted(old)}")


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

    def __init__(self, index, period_ms=200):
        self.index, self.proc, self.lines, self.period_ms = index, None, [], period_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", str(self.period_ms), "-i", str(self.index)], stdout=subprocess.PIPE,
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
        sm, mx, pw, reasons = [], [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # "under load" = samples drawing at least half of the highest power seen: the sampler also runs through the
        # idle moments around the timed region, which would otherwise hide a clock that drops under the power cap
        load = [c for c, p in zip(sm, pw) if pw and p >= 0.5 * max(pw)]
        return {"sm_mhz": statistics.median(load or sm) if sm else None, "sm_mhz_min": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(pw) if pw else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(load)}


Q_TYPE = "f16"   # --q-type


def make_inputs_np(w, units, rng):
    """One layer's operands for `units` units, numpy, in the workload's storage types."""
    from oracle import oracle as orc
    f16 = lambda shape, s=1.0: (rng.standard_normal(shape).astype(np.float32) * np.float32(s)).astype(np.float16)
    sc = 0.5 if w["seed"] == 1 else 1.0
    q = f16((units, w["H"], w["Tq"], w["hd"]), sc)
    if Q_TYPE == "f32":   # the reference's graphs hand the op an F32 Q; the values stay those of the F16 draw
        q = q.astype(np.float32)
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
        # the bytes the launch has to move at least: Q once, K/V once, the F32 output once (bias operands of the
        # rel-pos form not counted); a short causal prefill over a quantised cache is bound by these, not by the FLOPs
        kv_row = w["hd"] * 2 if w["kv"] == "f16" else w["hd"] // 32 * 34
        q_bytes = 4 if Q_TYPE == "f32" else 2
        nbytes = units * (w["H"] * w["Tq"] * w["hd"] * (q_bytes + 4) + 2.0 * w["Hkv"] * w["Lk"] * kv_row)
        return dict(bound="tensor", amount=flops, unit="TFLOP/s", div=1e12, bytes=nbytes)
    row = w["hd"] * 2 if w["kv"] == "f16" else w["hd"] // 32 * 34
    rows = w["Tq"] * w["beam_cells"] if "beam_cells" in w else w["Lk"]    # valid cells only
    if "pool" in w:
        rows = w["pool"][0] + w["Tq"] * w["pool"][1]                      # live cells: the shared prefix once, every private suffix
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
            "q_type": Q_TYPE, "sharding": "units across GPUs, no collective", "launch": "python loop" if args.no_graph else "cuda graph of one step",
            "l2": "inputs of one launch exceed L2" if w["kind"] == "prefill" else "L2 flushed between steps"}


class DeviceWorkload:
    """One workload resident on one GPU: operands, output, workspace, and `step()` = one pass over the layers."""

    def __init__(self, b200, abi, torch, dev, w, units, seed_offset=0):
        self.b200, self.torch, self.w, self.units, self.dev = b200, torch, w, units, dev
        rng = np.random.default_rng(w["seed"] + seed_offset)
        # generate a few units' worth on the host and tile them: cheap and still random-like
        gen_units = min(units, 4)
        q_np, k_np, v_np, extra = make_inputs_np(w, gen_units, rng)
        rep = -(-units // gen_units)
        def up(a):
            t = torch.from_numpy(a).to(dev)
            return t.repeat((rep,) + (1,) * (t.dim() - 1))[:units].contiguous()
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
            from oracle import oracle as orc_mask   # input generation only: the beam-membership mask rule
            L, beams = w["beam_cells"], w["Tq"]
            cell_pos = np.full(w["Lk"], 10 ** 6, np.int32)
            bits = np.zeros(w["Lk"], np.uint32)
            for jb in range(beams):
                cell_pos[jb * L:(jb + 1) * L], bits[jb * L:(jb + 1) * L] = np.arange(L), 1 << jb
            m = orc_mask.whisper_beam_mask(cell_pos, bits, tok_seq=np.arange(beams), tok_pos=np.full(beams, L - 1))
            mask = torch.from_numpy(m[None, None]).to(dev)
        if "pool" in w:
            prefix, suffix, form = w["pool"]
            beams, n_cells = w["Tq"], w["Lk"]
            prng = np.random.default_rng(12345)
            slots = prng.permutation(n_cells)[:prefix + beams * suffix]
            cell_pos, bits = np.full(n_cells, -1, np.int32), np.zeros(n_cells, np.uint32)
            cell_pos[slots[:prefix]], bits[slots[:prefix]] = np.arange(prefix), (1 << beams) - 1
            for jb in range(beams):
                sl = slots[prefix + jb * suffix: prefix + (jb + 1) * suffix]
                cell_pos[sl], bits[sl] = prefix + np.arange(suffix), 1 << jb
            tok_seq, tok_pos = np.arange(beams, dtype=np.int32), np.full(beams, prefix + suffix - 1, np.int32)
            if form == "dense":
                from oracle import oracle as orc_mask   # input generation only: the beam-membership mask rule
                mask = torch.from_numpy(orc_mask.whisper_beam_mask(cell_pos, bits, tok_seq, tok_pos)[None, None]).to(dev)
            elif form == "union":
                stride = -(-(prefix + beams * suffix) // 64) * 64
                uidx, ulen, umask = np.zeros(stride, np.int32), np.zeros(1, np.int32), np.zeros((beams, stride), np.uint16)
                rc = b200.lib().b200_beam_cells_to_union(cell_pos.ctypes.data, bits.ctypes.data, n_cells, tok_seq.ctypes.data,
                                                         tok_pos.ctypes.data, beams, uidx.ctypes.data, stride, ulen.ctypes.data,
                                                         umask.ctypes.data)
                assert rc == 0
                mask = torch.from_numpy(umask.view(np.float16)[None, None]).to(dev)
                kw["kv_index"] = torch.from_numpy(np.tile(uidx[None], (units, 1))).to(dev)
                kw["kv_len"] = torch.from_numpy(np.tile(ulen, units)).to(dev)
            else:
                stride = prefix + suffix
                idx, lens = np.zeros((beams, stride), np.int32), np.zeros(beams, np.int32)
                rc = b200.lib().b200_beam_cells_to_index(cell_pos.ctypes.data, bits.ctypes.data, n_cells, tok_seq.ctypes.data,
                                                         tok_pos.ctypes.data, beams, idx.ctypes.data, stride, lens.ctypes.data)
                assert rc == 0
                # every beam of every segment is a batch entry; the beams of a segment share its pool (B / Bk = beams)
                q = q.permute(0, 2, 1, 3).reshape(units * beams, w["H"], 1, w["hd"]).contiguous()
                kw["kv_index"] = torch.from_numpy(np.tile(idx, (units, 1))).to(dev)
                kw["kv_len"] = torch.from_numpy(np.tile(lens, units)).to(dev)
        self.q, self.k, self.v, self.kw, self.mask = q, k, v, kw, mask
        self.out = torch.empty((q.shape[0], q.shape[2], w["H"], w["hd"]), dtype=torch.float32, device=dev)
        ws_bytes = b200.workspace_bytes(q, k, v, mask, **kw)
        self.ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        self.kernel_id, self.n_splits = b200.plan(q, k, v, mask, **kw)
        self.launches_per_layer = 1 + (1 if (self.kernel_id == abi.KERNEL_DECODE_SPLIT and self.n_splits > 1 and ws_bytes) else 0)
        if self.kernel_id == abi.KERNEL_PREFILL_TC5 and ws_bytes:
            self.launches_per_layer += 1   # K and V conversion pre-pass (one launch for both)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if w["kind"] != "prefill" else None

    def step(self, stream=None):
        for _ in range(self.w["layers"]):
            self.b200.flash_attn_ext(self.q, self.k, self.v, self.mask, out=self.out, workspace=self.ws, stream=stream, **self.kw)

    def measure(self, steps, warmup, graph, barrier=lambda: None):
        """CUDA-event time of `steps` steps after `warmup`; returns the per-step times in ms."""
        torch = self.torch
        self.step()                 # first call outside any capture (function attributes, tensor maps, lazy init)
        torch.cuda.synchronize()
        run_step = self.step
        if graph:
            # the layer loop is launch-bound from Python for the small decode shapes: capture one step
            # (all layers) into a CUDA graph and replay it, as a runtime would
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.step()
            run_step = g.replay
        for _ in range(max(warmup, 0)):
            run_step()
        barrier()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for s in range(steps):
            if self.flush is not None:
                self.flush.fill_(s & 0xFF)        # evict L2 between steps (outside the event pair)
            ev[s][0].record()
            run_step()
            ev[s][1].record()
        barrier()
        return [a.elapsed_time(b) for a, b in ev]


def launch_floor_us(b200, torch, n_launches=30):
    """Device time per launch of a CUDA graph of `n_launches` empty kernels: what a layer costs when it does nothing."""
    L = b200.lib()
    def step():
        st = torch.cuda.current_stream().cuda_stream
        for _ in range(n_launches):
            L.b200_test_empty_launch(st)
    step()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for _ in range(3):
        g.replay()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
    for a, b in ev:
        a.record()
        g.replay()
        b.record()
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in ev) * 1e3 / n_launches


def roofline_of(abi, w, name, units, dw, step_ms, pk, traffic):
    work = algorithmic_work(w, units)
    launch_s = statistics.fmean(step_ms) * 1e-3 / w["layers"]
    floors = None
    if "bytes" in work:   # a contraction: the bound is whichever of the two floors is the longer one for this shape
        floors = {"tensor": work["amount"] / (pk["tensor"] * 1e12) * 1e6, "hbm": work["bytes"] / (pk["hbm"] * 1e9) * 1e6}
        if floors["hbm"] > floors["tensor"]:
            work = dict(bound="hbm", amount=work["bytes"], unit="GB/s", div=1e9)
    achieved = work["amount"] / launch_s / work["div"]
    peak = pk["tensor"] if work["bound"] == "tensor" else pk["hbm"]
    t = traffic.get(name)
    return {"bound": work["bound"], "achieved": achieved, "peak": peak, "unit": work["unit"], "frac": achieved / peak,
            **({"floors_us": floors} if floors else {}),
            "traffic": (t[0] * units / t[1]) if t else None,
            "traffic_source": "ncu capture of one launch, scaled by units" if t else None,
            "peak_source": f"{pk['src']} ({'sustained bf16 GEMM' if work['bound'] == 'tensor' else 'copy'})",
            "kernel": abi.KERNEL_NAMES[dw.kernel_id], "n_splits": dw.n_splits, "launch_ms": launch_s * 1e3,
            "algorithmic_per_launch": work["amount"]}


def strong_scaling(b200, abi, torch, w, total_units, n_dev, steps, warmup):
    """The fixed batch (`total_units`) partitioned over `n_dev` GPUs by the library's scheduler inside this one
    process: each worker thread gets its contiguous share as ONE batch (one launch per layer over the share).
    Inputs are resident per device before the clock starts; value = batch / wall time of a whole pass."""
    parts = [b200.SegmentScheduler.partition(total_units, n_dev, d) for d in range(n_dev)]
    work, graphs = {}, {}
    for d, (first, count) in enumerate(parts):
        if count:
            with torch.cuda.device(d):
                work[d] = DeviceWorkload(b200, abi, torch, torch.device("cuda", d), w, count, seed_offset=first)
                work[d].step()
                torch.cuda.synchronize(d)
                # one pass over the layers as a CUDA graph, replayed by the worker thread on the scheduler's stream
                graphs[d] = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graphs[d]):
                    work[d].step()
                torch.cuda.synchronize(d)
    sched = b200.SegmentScheduler(devices=list(range(n_dev)))

    def batch(device, first, count, stream):
        assert count == work[device].units, "a worker's share arrives as one batch"
        with torch.cuda.device(device), torch.cuda.stream(torch.cuda.ExternalStream(stream, device=device)):
            graphs[device].replay()
        return 0
    times, owners = [], None
    for it in range(warmup + steps):
        for d in work:
            torch.cuda.synchronize(d)
        t0 = time.perf_counter()
        failed, owners = sched.run_batched(total_units, max(c for _, c in parts), batch, steal=False)   # returns after every worker synchronised its stream
        dt = time.perf_counter() - t0
        assert failed == 0
        if it >= warmup:
            times.append(dt)
    sched.close()
    dt = statistics.fmean(times)
    return {"value": total_units / dt, "unit": f"{w['unit_name']}/s", "batch": total_units, "n_gpus": n_dev,
            "ms_per_pass": dt * 1e3, "units_per_gpu": [c for _, c in parts], "workers_used": sorted(set(owners)),
            "timing": "host wall clock around b200_sched_run_batched (every worker synchronises its stream before it returns)",
            "api": "b200_sched_run_batched: one host thread per GPU in one process, contiguous shares, one launch per layer per share"}


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
    ap.add_argument("--no-extra", action="store_true", help="skip the `workloads` object (the other configurations)")
    ap.add_argument("--no-strong", action="store_true", help="skip the scheduler-partitioned fixed batch")
    ap.add_argument("--q-type", default="f16", choices=["f16", "f32"], help="storage type of Q (K/V follow the workload)")
    ap.add_argument("--kernel", default="auto", choices=["auto", "tile"])
    ap.add_argument("--decode-splits", type=int, default=0, help="force the split count of the split-KV decode kernel (A/B runs)")
    ap.add_argument("--no-graph", action="store_true", help="launch each layer from Python instead of replaying a CUDA graph")
    ap.add_argument("--record-traffic", nargs="+", metavar="CSV", help="rewrite the DRAM traffic table from ncu CSV exports and exit")
    args = ap.parse_args()
    global Q_TYPE
    Q_TYPE = args.q_type
    if args.record_traffic:
        record_traffic(args.record_traffic)
        return
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
    host_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        host_group = dist.new_group(backend="gloo")   # host-side barrier for the phase in which rank 0 drives every GPU
    if args.kernel == "tile":
        b200.lib().b200_set_kernel_override(abi.KERNEL_TILE_MMA)
    if args.decode_splits:
        b200.lib().b200_set_decode_splits(args.decode_splits)

    units = args.units or w["units"]
    dw = DeviceWorkload(b200, abi, torch, dev, w, units, seed_offset=1000 * rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local, period_ms=50)
    dw.step()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    step_ms = dw.measure(args.steps, args.warmup, not args.no_graph, barrier)
    clocks = sampler.stop() if rank == 0 else None
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
        e2e_units = units
        affinity0 = os.sched_getaffinity(0)
        near_cpus = gpu_local_cpus(dev.index if dev.index is not None else 0)
        if near_cpus:
            os.sched_setaffinity(0, near_cpus)   # staging buffers next to the GPU; restored after the measurement
        hq, hk, hv = (x[:e2e_units].contiguous().cpu().pin_memory() for x in (dw.q, dw.k, dw.v))
        hkw = dict(dw.kw)
        if w["kind"] == "relpos":
            hkw["q_v"], hkw["r"] = dw.kw["q_v"][:e2e_units].cpu().pin_memory(), dw.kw["r"].cpu().pin_memory()
        hmask = dw.mask.cpu().pin_memory() if dw.mask is not None else None
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
        del hq, hk, hv, hout

    # ---- strong scaling: the fixed batch over all N GPUs, driven by the library's scheduler from rank 0 alone ----
    strong = None
    if not args.no_strong and w["kind"] in ("prefill", "relpos") and not args.units:
        barrier()
        if rank == 0:
            strong = strong_scaling(b200, abi, torch, w, w["units"] if w["kind"] == "prefill" else 16, world,
                                    steps=max(1, min(args.steps, 5)), warmup=2)
        if world > 1:
            dist.barrier(group=host_group)   # the other ranks wait on the host: no kernel of theirs occupies a GPU meanwhile

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    traffic = read_traffic()
    roofline = roofline_of(abi, w, args.workload, units, dw, step_ms, pk, traffic)
    line = {
        "metric": f"attention {w['unit_name']}/s ({args.workload})", "value": value, "unit": f"{w['unit_name']}/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 operands, f32 softmax/accumulate" if w["kv"] == "f16" else "q8_0 KV dequantised in-kernel, f32 softmax/accumulate",
        "data": "synthetic", "config": config_of(args, w, units), "roofline": roofline, "clocks": clocks,
        "gpu_launches": dw.launches_per_layer * w["layers"] * args.steps, "e2e": e2e,
    }
    if strong is not None:
        line["strong"] = strong

    # ---- the other configurations of the path, a few steps each (single-GPU runs) ----
    if not args.no_extra and world == 1 and not args.units and args.workload == "whisper_large_v3_encoder":
        del dw
        torch.cuda.empty_cache()
        extra = {}
        for name, u in EXTRA:
            xw = WORKLOADS[name]
            xu = u or xw["units"]
            key = name if u is None else f"{name}@{xu}"
            try:
                xdw = DeviceWorkload(b200, abi, torch, dev, xw, xu)
                xs = ClockSampler(local, period_ms=50)
                xdw.step()
                torch.cuda.synchronize()
                xs.start()
                xms = xdw.measure(5, 3, True, torch.cuda.synchronize)
                # short workloads: keep the device busy long enough for a few clock samples
                t_end = time.perf_counter() + 0.4
                while time.perf_counter() < t_end:
                    xdw.step()
                    torch.cuda.synchronize()
                xc = xs.stop()
                xms_mean = statistics.fmean(xms)
                extra[key] = {"value": xu / (xms_mean * 1e-3), "unit": f"{xw['unit_name']}/s", "units_per_gpu": xu,
                              "ms_per_step": xms_mean, "steps": 5, "warmup": 3,
                              "roofline": roofline_of(abi, xw, name, xu, xdw, xms, pk, traffic), "clocks": xc,
                              "gpu_launches": xdw.launches_per_layer * xw["layers"] * 5}
                del xdw
                torch.cuda.empty_cache()
            except Exception as exc:   # one failing configuration must not take the headline line with it
                extra[key] = {"error": f"{type(exc).__name__}: {exc}"}
        line["workloads"] = extra
        # the short decode launches (8 streams: 9 us per layer) next to what an empty kernel per layer costs
        line["launch_floor_us_per_kernel"] = launch_floor_us(b200, torch)
    if not args.no_cpu_baseline:
        val, sample, cores = cpu_sample(w, budget_s=12.0)
        line["cpu_baseline"] = {"value": val, "unit": f"{w['unit_name']}/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
