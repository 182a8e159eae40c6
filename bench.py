#!/usr/bin/env python
"""Benchmark of the sparse DiT attention block (GEMM-Q/K/V -> block-sparse attention -> GEMM-O).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload flux_block]

A step is one pass of the block over one batch of seeded synthetic input (FLUX-like: hidden 3072,
24 heads x 128, 4608 tokens, batch 2, bf16, block density 0.5). With N > 1 the heads are partitioned
over the ranks (no traffic inside the block; strong scaling of a fixed job). Prints one JSON line.
`--impl reference` times the CPU statement of the same block (dense masked fp32 torch on the host
cores) on a bounded sample; the reference project has no CPU implementation of its own.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sparse-attn+GEMM-Q/O layer achieved TFLOPS on executed FLOPs (latency in ms_per_step)"
HID, H, D, S, B, DENSITY, SEED = 3072, 24, 128, 4608, 2, 0.5, 2024
FL_ATTN_TILE = 4 * 128 * 128 * 128
FL_GEMM_TILE = 2 * 128 * 128 * HID
# dram__bytes_read.sum + dram__bytes_write.sum per launch (ncu captures summarised in profiles/)
GEMM_TRAFFIC_BYTES = 111.0e6   # average of one step's GEMM-Q, K, V, O launches
ATTN_TRAFFIC_BYTES = 165.3e6


def block_flops(masks, hb, hc, batch=B, seq=S):
    """Executed FLOPs of one step for the head window [hb, hb+hc)."""
    from flashomni_b200 import workloads as wl
    act, _ = wl.active_pairs(masks, hb, hc)
    tiles = wl.executed_attention_tiles(masks, hb, hc)
    dense_kv = 2 * (2 * batch * seq * hc * D * HID)
    return {"gemm_q": act * FL_GEMM_TILE, "gemm_kv": dense_kv, "attention": tiles * FL_ATTN_TILE,
            "gemm_o": act * FL_GEMM_TILE, "active_pairs": act, "attn_tiles": tiles}


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs: NVML from a
    thread every few milliseconds (the timed region of the default run is only tens of milliseconds long),
    nvidia-smi at 100 ms when the NVML module is missing. Read-only queries."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.p, self.thread = gpu_index, None, None
        self.sm, self.reasons, self.mx, self.stop_flag = [], set(), None, False

    def _nvml_loop(self, nv, handle):
        bits = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                r = int(get_reasons(handle))
                for name, bit in bits.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            # NVML numbers the GPUs of the machine; CUDA_VISIBLE_DEVICES may renumber them for this process
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.idx
            if vis:
                ent = vis.split(",")[self.idx].strip()
                phys = int(ent) if ent.isdigit() else None
            handle = nv.nvmlDeviceGetHandleByIndex(phys) if phys is not None else nv.nvmlDeviceGetHandleByUUID(ent)
            self.mx = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.mx,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "source": "nvml"}
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except Exception:
            self.p.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def make_inputs(rank, world):
    from flashomni_b200 import workloads as wl
    masks = wl.flux_masks(B, H, S // 128, S // 128, DENSITY, SEED)
    hc = H // world
    hb = rank * hc
    std = HID ** -0.5
    w = {n: wl.randn_bf16((HID, HID), SEED + i, std=std) for i, n in enumerate(("wq", "wk", "wv", "wo"), 10)}
    x = wl.randn_bf16((B, S, HID), SEED + 1)
    cache = wl.randn_bf16((B, S, HID), SEED + 2)
    return masks, hb, hc, w, x, cache


def run_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    from flashomni_b200 import _native
    from flashomni_b200.layer import BlockWeights, SparseDiTAttentionBlock
    _native.load()

    masks, hb, hc, w, x_host, cache_host = make_inputs(rank, world)
    sl = slice(hb * D, (hb + hc) * D)
    weights = BlockWeights(w["wq"][sl].contiguous().to(device), w["wk"][sl].contiguous().to(device),
                           w["wv"][sl].contiguous().to(device), w["wo"][:, sl].contiguous().to(device))
    block = SparseDiTAttentionBlock(weights, H, D, B, S, hb, hc, device=device, schedule=args.schedule)
    block.cache.copy_(cache_host.to(device))
    x = x_host.to(device)
    m_host = [torch.from_numpy(a).pin_memory() for a in (masks.sparse_info, masks.sparse_kv_info, masks.info_indptr,
                                                         masks.kv_info_indptr)]
    m_dev = [t.to(device) for t in m_host]
    x_pinned = x_host.pin_memory()
    y_pinned = torch.empty((B, S, HID), dtype=torch.bfloat16).pin_memory()

    def step():
        return block.forward(x, m_dev[0], m_dev[1], m_dev[2], m_dev[3])

    # End-to-end leg: every step copies its inputs (hidden state + masks) from pinned host memory and reads
    # its result back. Three streams and double buffers pipeline step i's compute with the upload of step
    # i+1 and the download of step i-1 (the two copy directions use different copy engines).
    s_h2d, s_d2h = torch.cuda.Stream(device), torch.cuda.Stream(device)
    x_buf = [x, torch.empty_like(x)]
    m_buf = [m_dev, [torch.empty_like(t) for t in m_dev]]
    y_buf = [torch.empty((B, S, HID), dtype=torch.bfloat16, device=device) for _ in range(2)]

    def run_e2e(steps):
        cur = torch.cuda.current_stream(device)
        ev_h2d = [torch.cuda.Event() for _ in range(steps)]
        ev_cmp = [torch.cuda.Event() for _ in range(steps)]
        ev_d2h = [torch.cuda.Event() for _ in range(steps)]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_h2d.wait_stream(cur)
        s_d2h.wait_stream(cur)
        t0.record(s_h2d)
        for i in range(steps):
            k = i & 1
            with torch.cuda.stream(s_h2d):
                if i >= 2:
                    s_h2d.wait_event(ev_cmp[i - 2])      # buffer k was read by step i-2
                x_buf[k].copy_(x_pinned, non_blocking=True)
                for d, h in zip(m_buf[k], m_host):
                    d.copy_(h, non_blocking=True)
                ev_h2d[i].record(s_h2d)
            cur.wait_event(ev_h2d[i])
            if i >= 2:
                cur.wait_event(ev_d2h[i - 2])            # y buffer k was downloaded
            block.forward(x_buf[k], *m_buf[k], out=y_buf[k])
            ev_cmp[i].record(cur)
            with torch.cuda.stream(s_d2h):
                s_d2h.wait_event(ev_cmp[i])
                y_pinned.copy_(y_buf[k], non_blocking=True)
                ev_d2h[i].record(s_d2h)
        t1.record(s_d2h)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / steps

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if dist is not None:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    block.wrapper.check_status()
    graph = None
    if args.graph:
        # one CUDA graph per step (the launches of a step are fixed for fixed shapes and mask buffers)
        graph = torch.cuda.CUDAGraph()
        cs = torch.cuda.Stream(device)
        cs.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(cs):
            with torch.cuda.graph(graph, stream=cs):
                step()
        eager_step = step
        step = graph.replay  # noqa: F841
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(step, args.steps)
    clocks = sampler.stop()
    run_e2e(2)
    barrier()
    ms_e2e = run_e2e(args.steps)
    if dist is not None:
        t = torch.tensor([ms_e2e], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    block.wrapper.check_status()

    # per-op pass (same K steps, events around every op) for the roofline of the dominant kernel
    ops = {"gemm_q": [], "gemm_kv": [], "attention": [], "gemm_o": []}
    from flashomni_b200 import flashomni_gemm, flashomni_gemm_reduction
    T = B * S
    for _ in range(args.steps):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        flashomni_gemm(x, weights.wq, H, m_dev[0], m_dev[2], 0, None, out=block.q, head_begin=hb, head_dim=D)
        ev[1].record()
        flashomni_gemm(x, weights.wk, H, is_full=True, out=block.k, head_dim=D)
        flashomni_gemm(x, weights.wv, H, is_full=True, out=block.v, head_dim=D)
        ev[2].record()
        block.wrapper.run(block.q.view(T, hc, D), block.k.view(T, hc, D), block.v.view(T, hc, D), *m_dev,
                          out=block.attn.view(T, hc, D))
        ev[3].record()
        flashomni_gemm_reduction(block.attn, weights.wo, H, m_dev[0], m_dev[2], 0, block.cache, is_for_cache=False,
                                 head_begin=hb, head_dim=D, out=block.y)
        ev[4].record()
        torch.cuda.synchronize()
        for i, k in enumerate(ops):
            ops[k].append(ev[i].elapsed_time(ev[i + 1]))
    op_ms = {k: statistics.mean(v) for k, v in ops.items()}

    # Spread of the whole step (events around every single step), the same with L2 flushed before every step
    # (a 256 MB buffer is rewritten: larger than the 126 MB L2), and the mask compaction alone.
    def each_step(flush):
        ts = []
        for _ in range(args.steps):
            if flush is not None:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return {"median": round(statistics.median(ts), 4), "min": round(min(ts), 4)}

    warm_ms = each_step(None)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    cold_ms = each_step(flush_buf)
    del flush_buf
    compact_ts = []
    for _ in range(args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        block.wrapper.build_work_lists(m_dev[0], m_dev[1], m_dev[2], m_dev[3])
        e1.record()
        torch.cuda.synchronize()
        compact_ts.append(e0.elapsed_time(e1))
    block.wrapper.check_status()
    timing_detail = {"step_ms": warm_ms, "step_ms_l2_flushed": cold_ms,
                     "mask_compaction_ms": {"median": round(statistics.median(compact_ts), 4),
                                            "min": round(min(compact_ts), 4)},
                     "plan_host_ms": round(block.plan_host_ms, 3)}

    fl = block_flops(masks, hb, hc)
    fl_rank = fl["gemm_q"] + fl["gemm_kv"] + fl["attention"] + fl["gemm_o"]
    if dist is not None:
        t = torch.tensor([float(fl_rank)], device=device, dtype=torch.float64)
        dist.all_reduce(t)
        fl_total = float(t.item())
    else:
        fl_total = float(fl_rank)

    if rank == 0:
        peaks = {"bf16_tflops": 1590.0, "src": "fallback"}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                p = json.load(f)
            peaks = {"bf16_tflops": float(p["bf16_tflops_sustained"]), "burst": float(p["bf16_tflops"]), "src": "measured"}
        except Exception:
            pass
        gemm_ms = op_ms["gemm_q"] + op_ms["gemm_kv"] + op_ms["gemm_o"]
        gemm_fl = fl["gemm_q"] + fl["gemm_kv"] + fl["gemm_o"]
        dominant = "gemm" if gemm_ms >= op_ms["attention"] else "attention"
        d_fl, d_ms, launches = (gemm_fl, gemm_ms, 4) if dominant == "gemm" else (fl["attention"], op_ms["attention"], 1)
        achieved = d_fl / (d_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "gemm_kernel<bf16> / gemm_tall_kernel<bf16> (GEMM-Q, K, V, O launches)" if dominant == "gemm"
                    else "attention_kernel<bf16>", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                    "traffic": GEMM_TRAFFIC_BYTES if dominant == "gemm" else ATTN_TRAFFIC_BYTES,
                    "traffic_note": "dram read+write bytes per launch from the ncu captures summarised under profiles/",
                    "peak_source": peaks["src"] + " (sustained cuBLAS bf16; the kernel runs inside a long step)",
                    "launches_per_step": launches, "avg_launch_ms": round(d_ms / launches, 4),
                    "per_op_ms": {k: round(v, 4) for k, v in op_ms.items()},
                    "per_op_tflops": {k: round(fl[k] / (op_ms[k] * 1e-3) / 1e12, 1) for k in op_ms}}
        out = {
            "metric": METRIC, "value": round(fl_total / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
            "latency_us": round(ms * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "flux_block: hidden 3072, H=24, D=128, S=4608, batch 2, block density 0.5 "
                                   "(GEMM-Q sparse, GEMM-K/V dense, block-sparse attention, GEMM-O active heads + cache)",
                       "parallelism": f"heads/{world}", "seed": SEED, "cuda_graph": bool(args.graph),
                       "schedule": args.schedule,
                       "l2": "per-step working set (x, 4 weights, q/k/v, attention out, cache, y) is >200 MB per rank, "
                             "larger than the 126 MB L2; no explicit flush",
                       "executed_flops_per_step": fl_total, "active_pairs": fl["active_pairs"],
                       "attention_tiles": fl["attn_tiles"]},
            "e2e": {"value": round(fl_total / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e, 4),
                    "h2d_bytes_per_step": int(x_pinned.numel() * 2 + sum(t.numel() * t.element_size() for t in m_host)),
                    "d2h_bytes_per_step": int(y_pinned.numel() * 2)},
            "gpu_launches": int(args.steps * 10),
            "clocks": clocks, "roofline": roofline, "timing_detail": timing_detail,
        }
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(masks, w, x_host, cache_host, steps=40)
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_video(args):
    """Long video layer (hidden 5120, H=40, D=128, 20 frames x 3840 + 512 text = 77 312 tokens, batch 1, block
    density ~0.25) under Ulysses sequence parallelism: tokens sharded by 128-token blocks, an exchange (pulls over
    peer memory, or the NCCL all-to-all) before and after the attention. Strong scaling of a fixed job."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    from flashomni_b200 import workloads as wl
    from flashomni_b200.layer import BlockWeights, UlyssesSparseDiTAttentionBlock
    hid, Hv, frames, bpf = 5120, 40, 20, 30
    S = (4 + frames * bpf) * 128
    masks = wl.video_masks(Hv, frames, bpf, SEED)
    std = hid ** -0.5
    weights = BlockWeights(*(wl.randn_bf16((hid, hid), SEED + i, std=std).to(device) for i in range(10, 14)))
    blk = UlyssesSparseDiTAttentionBlock(weights, Hv, D, S, rank, world, device)
    x = wl.randn_bf16((1, blk.s_loc, hid), SEED + 1 + rank).to(device)
    blk.cache.copy_(wl.randn_bf16((1, blk.s_loc, hid), SEED + 100 + rank).to(device))
    m_dev = [torch.from_numpy(a).to(device) for a in (masks.sparse_info, masks.sparse_kv_info, masks.info_indptr,
                                                      masks.kv_info_indptr)]

    def step():
        return blk.forward(x, *m_dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    blk.wrapper.check_status()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    # phase breakdown of two more steps (outside the timed region), rank 0's view
    phases = {}
    for _ in range(2):
        marks = []
        blk.forward(x, *m_dev, marks=marks)
        torch.cuda.synchronize()
        if len(marks) == 8:  # peer-memory exchange: the two barriers are marked separately
            names = ("projections", "barrier", "pull_qkv", "attention", "barrier_back", "pull_o", "gemm_o")
        else:
            names = ("proj_and_exchange", "attention", "exchange_back", "gemm_o")
        phases = {n: round(marks[i].elapsed_time(marks[i + 1]), 4) for i, n in enumerate(names)}
    if dist is not None:  # slowest rank per phase
        pt = torch.tensor([phases[n] for n in phases], device=device, dtype=torch.float64)
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        phases_max = {n: round(float(v), 4) for n, v in zip(phases, pt.tolist())}
    else:
        phases_max = phases
    tiles = wl.executed_attention_tiles(masks, blk.hb, blk.hc)
    rows_blocks = blk.s_loc // 128
    fl_rank = tiles * FL_ATTN_TILE + 4 * (2 * blk.s_loc * hid * hid)
    if dist is not None:
        t = torch.tensor([ms, float(fl_rank)], device=device, dtype=torch.float64)
        tm = t.clone()
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(t)
        ms, fl_total = float(tm[0].item()), float(t[1].item())
    else:
        fl_total = float(fl_rank)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": round(fl_total / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
            "latency_us": round(ms * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "video_layer: hidden 5120, H=40, D=128, S=77312 (20 frames x 3840 + 512 text), batch 1, "
                                   "spatiotemporal-local block mask (+-1 frame + 10% random + text), Ulysses all-to-all",
                       "parallelism": f"ulysses/{world}", "exchange": blk.exchange, "seed": SEED, "executed_flops_per_step": fl_total,
                       "attention_tiles_rank0": tiles, "l2": "working set of several GB, far above the 126 MB L2",
                       "phase_ms_rank0": phases, "phase_ms_slowest_rank": phases_max},
            "gpu_launches": int(args.steps * 10), "clocks": clocks}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def cpu_sample_step(masks, w, x_host, cache_host, heads=(0, 1, 2, 3, 4, 5), row_blocks=36):
    """One bounded sample of the block on the CPU oracle: the attention of `heads` of request 0 (full
    sequence) and the four GEMMs on the first `row_blocks` 128-row blocks of request 0. Returns the
    executed FLOPs of the sample."""
    from flashomni_b200 import workloads as wl
    from oracle import attention as oa
    from oracle import gemm as og
    rows = row_blocks * 128
    xs = x_host[:1, :rows]
    q = og.gemm_q(xs, w["wq"], H, masks.sparse_info, masks.info_indptr, 0, None, None)
    og.gemm_q(xs, w["wk"], H, is_full=True)
    og.gemm_q(xs, w["wv"], H, is_full=True)
    og.gemm_o(xs, w["wo"], H, masks.sparse_info, masks.info_indptr, 0, cache_host[:1, :rows], False)
    act = int(masks.q_active[0][:row_blocks].sum())
    fl = 2 * act * FL_GEMM_TILE + 2 * (2 * rows * HID * HID)
    g = torch.Generator().manual_seed(1)
    for h in heads:
        mh = wl.pack_masks([masks.q_active[0][:, h:h + 1]], [masks.kv_kept[0][:, h:h + 1]])
        qh = torch.randn(S, 1, D, generator=g); kh = torch.randn(S, 1, D, generator=g); vh = torch.randn(S, 1, D, generator=g)
        oa.sparse_attention(qh, kh, vh, [0, S], [0, S], mh.sparse_info, mh.sparse_kv_info, mh.info_indptr, mh.kv_info_indptr)
        fl += int((masks.kv_kept[0][:, h] * masks.q_active[0][:, h:h + 1]).sum()) * FL_ATTN_TILE
    return fl, f"request 0: attention of heads {list(heads)} over all 4608 tokens + GEMM-Q/K/V/O on the first {rows} rows"


def cpu_baseline(masks, w, x_host, cache_host, steps=1):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cpu_sample_step(masks, w, x_host, cache_host, heads=(0,), row_blocks=1)  # warm-up
    t0 = time.perf_counter()
    fl = 0
    for _ in range(steps):
        f, sample = cpu_sample_step(masks, w, x_host, cache_host)
        fl += f
    dt = time.perf_counter() - t0
    return {"value": round(fl / dt / 1e12, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": sample + f"; {steps} pass(es), {dt:.1f} s; dense masked fp32 torch"}


def run_reference(args):
    """The reference has no CPU implementation of this path; its CPU statement (the oracle) is timed on
    the host cores, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    masks, hb, hc, w, x_host, cache_host = make_inputs(0, 1)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    steps = min(args.steps, 10)
    warm = min(max(args.warmup, 1), 2)
    for _ in range(warm):
        cpu_sample_step(masks, w, x_host, cache_host)
    t0 = time.perf_counter()
    fl = 0
    for _ in range(steps):
        f, sample = cpu_sample_step(masks, w, x_host, cache_host)
        fl += f
    dt = time.perf_counter() - t0
    val = round(fl / dt / 1e12, 4)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": warm,
        "ms_per_step": round(dt / steps * 1e3, 2), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "flux_block (bounded sample per step): " + sample, "seed": SEED},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="flux_block", choices=["flux_block", "video"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--schedule", default="q_first", choices=["q_first", "kv_first"],
                    help="flux_block: order of the projections and where the list kernels run")
    ap.add_argument("--graph", dest="graph", action="store_true", default=True,
                    help="replay the step from a CUDA graph (device-resident leg; the default: at 8 GPUs a step is "
                         "about 100 us of kernels and eager launches are host-bound)")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="launch the step eagerly")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "video":
        run_video(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
