#!/usr/bin/env python
"""Benchmark of the sparse DiT attention block (GEMM-Q/K/V -> block-sparse attention -> GEMM-O).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--quick] [--no-video]

A step is one pass of the block over one batch of seeded synthetic input (FLUX-like: hidden 3072,
24 heads x 128, 4608 tokens, batch 2, bf16, block density 0.5). With N > 1 the heads are partitioned
over the ranks (no traffic inside the block; strong scaling of a fixed job); the ranks' partial outputs
are summed after the block (timed on its own). Prints ONE JSON line whose `value` is that block.
The same line carries, outside the timed region of `value`:
  roofline      one entry per kernel of the step (own launch time, algorithmic work, fraction of the peak)
  sparse_trio   GEMM-Q + attention + GEMM-O alone (no dense K/V projections), replayed from a CUDA graph
  sweep         GEMM-Q at density .25/.5/.75, GEMM-O with is_for_cache True/False, attention at .25/.5/.75
  mask_path     segment_packbits and the mask compaction at the video layer's mask size, in GB/s
  baselines     the reference's own CUDA kernels (rebuilt for sm_100a) and dense library kernels, same inputs
  video         the long video layer (Ulysses sequence parallelism over the N ranks)
  parity        sampled rows of both workloads against the CPU oracle, at this N
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu captures summarised under profiles/
NCU_TRAFFIC = {"attention_kernel": 172.1e6, "gemm_kernel": 121.1e6, "gemm_tall_kernel": 233.5e6}


# ---------------------------------------------------------------------------------------------- helpers
def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"burst": float(p["bf16_tflops"]), "sustained": float(p["bf16_tflops_sustained"]),
                "hbm_gbs": float(p["hbm_gbs"]), "src": "measured"}
    except Exception:
        return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "src": "fallback"}


def block_flops(masks, hb, hc, batch=B, seq=S, hid=HID):
    """Executed FLOPs of one step for the head window [hb, hb+hc)."""
    from flashomni_b200 import workloads as wl
    act, _ = wl.active_pairs(masks, hb, hc)
    tiles = wl.executed_attention_tiles(masks, hb, hc)
    dense_kv = 2 * (2 * batch * seq * hc * D * hid)
    tile = 2 * 128 * 128 * hid
    return {"gemm_q": act * tile, "gemm_kv": dense_kv, "attention": tiles * FL_ATTN_TILE,
            "gemm_o": act * tile, "active_pairs": act, "attn_tiles": tiles}


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
            return self
        except Exception:
            self.thread = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None
        return self

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


class Ctx:
    """Rank, device and process group of this process."""

    def __init__(self):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU fallback")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # plain peer loads and rings only
            import torch.distributed as dist
            # NCCL may announce its version on stdout when the communicator comes up; stdout carries the one JSON
            # line only, so the file descriptor points at stderr until the first collective has run
            sys.stdout.flush()
            saved = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group("nccl", device_id=self.device)
                t = torch.zeros(1, device=self.device)
                dist.all_reduce(t)
                torch.cuda.synchronize()
            finally:
                sys.stdout.flush()
                os.dup2(saved, 1)
                os.close(saved)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.dist is None:
            return [float(v) for v in values]
        t = torch.tensor([float(v) for v in values], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def sum_over_ranks(self, values):
        if self.dist is None:
            return [float(v) for v in values]
        t = torch.tensor([float(v) for v in values], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t)
        return t.tolist()


def event_time(fn, steps, sync_each=False, before=None):
    """Mean (and median / min) milliseconds of fn() over `steps` calls, CUDA events on the current stream."""
    if sync_each or before is not None:
        ts = []
        for _ in range(steps):
            if before is not None:
                before()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return {"mean": statistics.mean(ts), "median": statistics.median(ts), "min": min(ts)}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"mean": ms, "median": ms, "min": ms}


def graph_time(launch, device, reps=20, on_current=False):
    """Mean milliseconds of one call of launch(stream_handle) when `reps` calls are replayed from one CUDA graph
    (for launches so short that eager calls would be bound by the host). `on_current`: the callable launches on
    torch's current stream (which is the capture stream here) and ignores the handle."""
    cs = torch.cuda.Stream(device)
    cs.wait_stream(torch.cuda.current_stream(device))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(cs):
        launch(cs.cuda_stream)
        launch(cs.cuda_stream)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=cs):
            for _ in range(reps):
                launch(cs.cuda_stream)
    for _ in range(3):
        g.replay()
    ms = event_time(g.replay, 5)["mean"] / reps
    return {"mean": ms, "median": ms, "min": ms}


def chain_time(ops, steps, pre=None):
    """Mean milliseconds of each op of a chain op_0, op_1, ... enqueued back to back, `steps` times over, with CUDA
    events between the ops and no host synchronisation inside the loop (the GPU stays busy and at its working
    clock, as inside a real step; an event pair around a lone launch after an idle period reads far longer).
    `pre` is called before every pass of the chain (work for a side stream)."""
    evs = []
    torch.cuda.synchronize()
    for _ in range(steps):
        if pre is not None:
            pre()
        row = [torch.cuda.Event(enable_timing=True) for _ in range(len(ops) + 1)]
        row[0].record()
        for i, (_name, fn) in enumerate(ops):
            fn()
            row[i + 1].record()
        evs.append(row)
    torch.cuda.synchronize()
    return {name: statistics.mean(r[i].elapsed_time(r[i + 1]) for r in evs) for i, (name, _fn) in enumerate(ops)}


def tf(flops, ms):
    return flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0


def r4(x):
    return None if x is None else round(float(x), 4)


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


# ---------------------------------------------------------------------------------------------- parity (checker)
def cmp_bf16(got, ref):
    """(max-abs, mean-abs, worst excess over the bound) of a 16-bit result against an fp32 reference value; the
    bound is max-abs 2e-2, widened to one bf16 unit in the last place of the reference where that is larger
    (|value| >= 4: the rounding step of the output format alone exceeds 2e-2 there)."""
    got, ref = got.float().cpu(), ref.float().cpu()
    diff = (got - ref).abs()
    ulp = torch.exp2(torch.floor(torch.log2(ref.abs().clamp_min(1e-30))) - 7)
    bound = torch.maximum(torch.full_like(diff, 2e-2), ulp)
    return float(diff.max()), float(diff.mean()), float((diff - bound).max())


def flux_parity(masks, w, x_host, cache_host, y_full, samples=((0, 5), (1, 0), (1, 20))):
    """Sampled 128-row blocks (request, row block) of the block's final output against the CPU oracle: for the
    heads that are active there, q = x Wq^T on the rows, K / V of the whole request, block-sparse attention over the
    kept kv blocks, and cache + sum of the active heads' output projections (each intermediate rounded to bf16 as
    the kernels store it)."""
    from flashomni_b200 import workloads as wl
    from oracle import attention as oa
    from oracle import gemm as og
    worst, mean_worst, excess = 0.0, 0.0, -1.0
    kv_of = {}
    for b, iy in samples:
        act = [h for h in range(H) if masks.q_active[b][iy, h]]
        rows = slice(iy * 128, (iy + 1) * 128)
        if b not in kv_of:
            xb = x_host[b:b + 1]
            kv_of[b] = (og.gemm_q(xb, w["wk"], H, is_full=True).to(torch.bfloat16).view(S, H, D),
                        og.gemm_q(xb, w["wv"], H, is_full=True).to(torch.bfloat16).view(S, H, D))
        kb, vb = kv_of[b]
        q = og.gemm_q(x_host[b:b + 1, rows], w["wq"], H, is_full=True).to(torch.bfloat16).view(128, H, D)
        y = cache_host[b, rows].float().clone()
        if act:
            sub = wl.pack_masks([np.ones((1, len(act)), np.uint8)], [masks.kv_kept[b][iy:iy + 1, act, :]])
            o = oa.sparse_attention(q[:, act], kb[:, act], vb[:, act], [0, 128], [0, S], sub.sparse_info,
                                    sub.sparse_kv_info, sub.info_indptr, sub.kv_info_indptr).to(torch.bfloat16)
            for i, h in enumerate(act):
                y += o[:, i].float() @ w["wo"][:, h * D:(h + 1) * D].float().T
        mx, mn, ex = cmp_bf16(y_full[b, rows], y)
        worst, mean_worst, excess = max(worst, mx), max(mean_worst, mn), max(excess, ex)
    return {"ok": bool(excess <= 0 and mean_worst <= 2e-3), "max_abs": r4(worst), "mean_abs": round(mean_worst, 5),
            "bounds": "max-abs 2e-2 (one bf16 ulp of the value where |y| >= 4), mean-abs 2e-3",
            "rows_checked": [list(s) for s in samples], "against": "oracle/ (CPU fp32 restatement)"}


# ---------------------------------------------------------------------------------------------- flux block
def run_flux(ctx, args, peaks):
    from flashomni_b200 import _native, flashomni_gemm, flashomni_gemm_reduction
    from flashomni_b200 import parallel as par
    from flashomni_b200.gemm import prepare_gemm_o_list, prepare_gemm_q_list
    from flashomni_b200.layer import BlockWeights, SparseDiTAttentionBlock
    lib = _native.load()
    world, rank, device, dist = ctx.world, ctx.rank, ctx.device, ctx.dist
    masks, hb, hc, w, x_host, cache_host = make_inputs(rank, world)
    sl = slice(hb * D, (hb + hc) * D)
    weights = BlockWeights(w["wq"][sl].contiguous().to(device), w["wk"][sl].contiguous().to(device),
                           w["wv"][sl].contiguous().to(device), w["wo"][:, sl].contiguous().to(device))
    # With one rank the block adds the cache itself; with several, every rank produces the bare sum of its heads
    # and the cache joins where the partials are summed.
    block = SparseDiTAttentionBlock(weights, H, D, B, S, hb, hc, device=device, schedule=args.schedule,
                                    add_cache=(world == 1))
    cache = cache_host.to(device)
    block.cache.copy_(cache)
    x = x_host.to(device)
    m_host = [torch.from_numpy(a).pin_memory() for a in (masks.sparse_info, masks.sparse_kv_info, masks.info_indptr,
                                                         masks.kv_info_indptr)]
    m_dev = [t.to(device) for t in m_host]
    T = B * S

    # ---- cross-rank sum of the partial outputs (N > 1): every rank owns T / N rows of the result
    px, y_part, y_ptrs, rows_per = None, None, None, T // world
    if world > 1:
        px = par.PeerExchange(None, device)
        if px.available:
            y_part, y_ptrs = [], []
            for _ in range(2):   # two buffers, alternating per step: a peer may still read the previous partial
                t, ptrs, _h = px.alloc((T, HID), torch.bfloat16)
                y_part.append(t)
                y_ptrs.append(ptrs)
        else:
            y_part = [torch.zeros((T, HID), dtype=torch.bfloat16, device=device) for _ in range(2)]
    y_slice = torch.empty((rows_per, HID), dtype=torch.bfloat16, device=device)
    cache_rows = cache.view(T, HID)[rank * rows_per:(rank + 1) * rows_per]
    reduce_mode = "none" if world == 1 else ("peer loads (fo_reduce_rows)" if px.available else "nccl reduce_scatter")
    step_no = [0]

    def step():
        return block.forward(x, m_dev[0], m_dev[1], m_dev[2], m_dev[3])

    def reduce_partials(k):
        """Sums the ranks' partials in buffer k into this rank's row slice (+ cache)."""
        if px is not None and px.available:
            px.barrier(k)
            px.reduce_rows(y_ptrs[k], rank * rows_per, rows_per, HID, torch.bfloat16, y_slice, init=cache_rows)
        else:
            dist.reduce_scatter_tensor(y_slice, y_part[k])
            y_slice.add_(cache_rows)

    def step_with_sum(xin=None, mm=None):
        k = step_no[0] & 1
        step_no[0] += 1
        mm = m_dev if mm is None else mm
        if world == 1:
            block.forward(x if xin is None else xin, *mm, out=y_slice.view(B, S, HID))
        else:
            block.forward(x if xin is None else xin, *mm, out=y_part[k].view(B, S, HID))
            reduce_partials(k)

    # ---- warm-up, launch count, optional CUDA graph
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    block.wrapper.check_status()
    n0 = lib.fo_launch_count()
    step()
    torch.cuda.synchronize()
    launches_per_step = int(lib.fo_launch_count() - n0)
    eager_step = step
    graph = None
    if args.graph:
        graph = torch.cuda.CUDAGraph()
        cs = torch.cuda.Stream(device)
        cs.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(cs):
            with torch.cuda.graph(graph, stream=cs):
                eager_step()
        step = graph.replay
        for _ in range(3):
            step()
        torch.cuda.synchronize()

    # A model captures its layers back to back; a step of a small share of the heads is launch-bound (the gap
    # between two graph launches is about 9 us), so when a step lasts under 0.27 ms a graph holds as many steps as
    # fit in about 0.65 ms (three at N = 4, four or five at N = 8; at N = 1 and 2 one step per graph measured the
    # same or faster). Every step inside a graph is the same full pass.
    steps_per_graph, graph_many = 1, None
    if graph is not None:
        est = ctx.max_over_ranks([event_time(step, 3)["mean"]])[0]
        want = args.steps_per_graph if args.steps_per_graph > 0 else (int(0.65 / max(est, 1e-3)) if est < 0.27 else 1)
        steps_per_graph = max(1, min(8, want, args.steps))
        if steps_per_graph > 1:
            graph_many = torch.cuda.CUDAGraph()
            cs.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(cs):
                with torch.cuda.graph(graph_many, stream=cs):
                    for _ in range(steps_per_graph):
                        eager_step()
            for _ in range(2):
                graph_many.replay()
            torch.cuda.synchronize()

    # ---- the timed region of `value`
    ctx.barrier()
    sampler = ClockSampler(ctx.local_rank).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps // steps_per_graph):
        (graph_many.replay if graph_many is not None else step)()
    for _ in range(args.steps % steps_per_graph if graph_many is not None else 0):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = ctx.max_over_ranks([e0.elapsed_time(e1) / args.steps])[0]
    block.wrapper.check_status()

    # ---- the cross-rank sum on its own, and block + sum
    reduce_ms = None
    if world > 1:
        for _ in range(3):
            step_with_sum()
        ctx.barrier()
        t_all = event_time(step_with_sum, args.steps)["mean"]
        ctx.barrier()
        k = step_no[0] & 1

        def only_reduce():
            step_no[0] += 1
            reduce_partials((step_no[0] - 1) & 1)
        # the partial buffers hold the last two steps' outputs: summing them again is the same work
        t_red = event_time(only_reduce, args.steps)["mean"]
        t_all, t_red = ctx.max_over_ranks([t_all, t_red])
        reduce_ms = {"block_plus_sum_ms": r4(t_all), "sum_alone_ms": r4(t_red), "mode": reduce_mode,
                     "bytes_per_rank": int(world * rows_per * HID * 2)}
        if px is not None and px.available:
            px.check_status()

    # ---- parity of the final output (after the cross-rank sum) against the oracle, sampled rows
    parity = None
    if not args.no_parity:
        step_with_sum()
        torch.cuda.synchronize()
        if world > 1:
            y_full = torch.empty((T, HID), dtype=torch.bfloat16, device=device)
            dist.all_gather_into_tensor(y_full, y_slice)
        else:
            y_full = y_slice
        if rank == 0:
            parity = flux_parity(masks, w, x_host, cache_host, y_full.view(B, S, HID))
        ctx.barrier()

    # ---- end to end: host buffers in, result back on the host, every step
    # N = 1: the hidden state and the masks go up from pinned memory, the output comes back. N > 1: every rank
    # uploads 1/N of the hidden state rows (the ranks' PCIe links work side by side), an all-gather over NVLink
    # completes it on every GPU, and after the cross-rank sum every rank downloads the rows it owns.
    s_h2d, s_d2h = torch.cuda.Stream(device), torch.cuda.Stream(device)
    x_rows_host = x_host.view(T, HID)[rank * rows_per:(rank + 1) * rows_per].contiguous().pin_memory()
    y_pinned = torch.empty((rows_per, HID), dtype=torch.bfloat16).pin_memory()
    x_buf = [torch.empty_like(x) for _ in range(2)]
    x_rows_dev = [torch.empty((rows_per, HID), dtype=torch.bfloat16, device=device) for _ in range(2)]
    m_buf = [[torch.empty_like(t) for t in m_dev] for _ in range(2)]
    y_e2e = [torch.empty((rows_per, HID), dtype=torch.bfloat16, device=device) for _ in range(2)]

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
                if world == 1:
                    x_buf[k].view(T, HID).copy_(x_rows_host, non_blocking=True)
                else:
                    x_rows_dev[k].copy_(x_rows_host, non_blocking=True)
                for d, h in zip(m_buf[k], m_host):
                    d.copy_(h, non_blocking=True)
                ev_h2d[i].record(s_h2d)
            cur.wait_event(ev_h2d[i])
            if i >= 2:
                cur.wait_event(ev_d2h[i - 2])            # result buffer k was downloaded
            if world > 1:
                dist.all_gather_into_tensor(x_buf[k].view(T, HID), x_rows_dev[k])
                kk = step_no[0] & 1
                step_no[0] += 1
                block.forward(x_buf[k], *m_buf[k], out=y_part[kk].view(B, S, HID))
                if px is not None and px.available:
                    px.barrier(kk)
                    px.reduce_rows(y_ptrs[kk], rank * rows_per, rows_per, HID, torch.bfloat16, y_e2e[k], init=cache_rows)
                else:
                    dist.reduce_scatter_tensor(y_e2e[k], y_part[kk])
                    y_e2e[k].add_(cache_rows)
            else:
                block.forward(x_buf[k], *m_buf[k], out=y_e2e[k].view(B, S, HID))
            ev_cmp[i].record(cur)
            with torch.cuda.stream(s_d2h):
                s_d2h.wait_event(ev_cmp[i])
                y_pinned.copy_(y_e2e[k], non_blocking=True)
                ev_d2h[i].record(s_d2h)
        t1.record(s_d2h)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / steps

    run_e2e(3)
    ctx.barrier()
    ms_e2e = ctx.max_over_ranks([run_e2e(args.steps)])[0]
    block.wrapper.check_status()
    if px is not None and px.available:
        px.check_status()
    h2d = int(x_rows_host.numel() * 2 + sum(t.numel() * t.element_size() for t in m_host))
    d2h = int(y_pinned.numel() * 2)
    h2d_all, d2h_all = (int(v) for v in ctx.sum_over_ranks([h2d, d2h]))

    # ---- per-kernel pass: every kernel of the step timed alone (its list prepared beforehand), this rank's view
    fl = block_flops(masks, hb, hc)
    n_local = hc * D
    q_list = prepare_gemm_q_list(B, S, n_local, H, m_dev[0], m_dev[2], 0, head_begin=hb, head_dim=D)
    o_list = prepare_gemm_o_list(B, S, n_local, H, m_dev[0], m_dev[2], 0, head_begin=hb, head_dim=D)
    kview = block.kv.view(T, 2 * hc, D) if block.fuse_kv else None

    def k_gemm_q():
        flashomni_gemm(x, weights.wq, H, m_dev[0], m_dev[2], 0, None, out=block.q, head_begin=hb, head_dim=D,
                       worklist=q_list)

    def k_gemm_kv():
        if block.fuse_kv:
            flashomni_gemm(x, block.wkv, H, is_full=True, out=block.kv, head_dim=D)
        else:
            flashomni_gemm(x, weights.wk, H, is_full=True, out=block.k, head_dim=D)
            flashomni_gemm(x, weights.wv, H, is_full=True, out=block.v, head_dim=D)

    def attn_run():
        if block.fuse_kv:
            k_, v_ = kview[:, :hc], kview[:, hc:]
        else:
            k_, v_ = block.k.view(T, hc, D), block.v.view(T, hc, D)
        block.wrapper.run(block.q.view(T, hc, D), k_, v_, *m_dev, out=block.attn.view(T, hc, D))

    def k_gemm_o():
        flashomni_gemm_reduction(block.attn, weights.wo, H, m_dev[0], m_dev[2], 0,
                                 block.cache if block.add_cache else None, is_for_cache=False, head_begin=hb,
                                 head_dim=D, out=block.y, worklist=o_list)

    def prep_masks():
        block.wrapper.prepare_masks(*m_dev)

    def compact_only():
        block.wrapper.build_work_lists(*m_dev)

    for _ in range(2):
        prep_masks(); k_gemm_q(); k_gemm_kv(); attn_run(); k_gemm_o()
    if world == 1:
        kt = chain_time([("gemm_q", k_gemm_q), ("gemm_kv", k_gemm_kv), ("attention", attn_run), ("gemm_o", k_gemm_o)],
                        args.steps, pre=prep_masks)
    else:
        # A rank's share of the step is too short for eager launches (the host's launch rate would set the intervals):
        # every kernel is replayed alone from a CUDA graph of five launches. The lists are complete by now, so the
        # GEMMs need not wait for them; the attention launch carries its list kernels, which are timed alone and
        # taken off.
        torch.cuda.synchronize()
        q_list.event = None
        o_list.event = None

        def alone(fn):
            return graph_time(lambda _s: fn(), device, reps=5, on_current=True)["mean"]

        t_lists = alone(compact_only)
        kt = {"gemm_q": alone(k_gemm_q), "gemm_kv": alone(k_gemm_kv), "attention": max(alone(attn_run) - t_lists, 0.0),
              "gemm_o": alone(k_gemm_o)}
    kt["compact"] = event_time(compact_only, args.steps)["mean"]
    kt = {k: {"mean": v} for k, v in kt.items()}
    block.wrapper.check_status()
    lists = block.wrapper.work_lists()
    compact_bytes = int(sum(t.numel() * t.element_size() for t in m_dev) + 4 * (6 * lists["n_items"] + 1)
                        + 4 * lists["total_kept"])
    dense_name = "gemm_tall_kernel" if lib.fo_gemm_dense_tile_rows(B, S, (2 if block.fuse_kv else 1) * n_local, HID, 0,
                                                                   torch.cuda.get_device_properties(device).multi_processor_count) == 256 \
        else "gemm_kernel"
    kv_launches = 1 if block.fuse_kv else 2
    step_sum_ms = sum(kt[k]["mean"] for k in ("gemm_q", "gemm_kv", "attention", "gemm_o"))

    def kentry(name, op, flops, launches):
        t = kt[op]["mean"]
        return {"kernel": name, "op": op, "launches_per_step": launches, "ms_per_step": r4(t),
                "avg_launch_ms": r4(t / launches), "flops_per_step": float(flops), "achieved_tflops": round(tf(flops, t), 1),
                "frac_of_peak": r4(tf(flops, t) / peaks["burst"]), "share_of_step": r4(t / step_sum_ms)}

    kernels = [kentry("attention_kernel<bf16>", "attention", fl["attention"], 1),
               kentry("gemm_kernel<bf16> (GEMM-Q, active tiles)", "gemm_q", fl["gemm_q"], 1),
               kentry("gemm_kernel<bf16> (GEMM-O, active heads)", "gemm_o", fl["gemm_o"], 1),
               kentry(dense_name + "<bf16> (dense K/V projection)", "gemm_kv", fl["gemm_kv"], kv_launches)]
    top = max(kernels[:3], key=lambda e: e["ms_per_step"])
    base = top["kernel"].split("<")[0]
    if world > 1:
        for e in kernels:
            e["note"] = ("this rank's share, each kernel replayed alone from a CUDA graph of five launches (eager launches "
                         "would be bound by the host at this size); at N = 1 the kernels are timed inside the step's chain")
    roofline = {"bound": "tensor", "kernel": top["kernel"], "achieved": top["achieved_tflops"], "peak": peaks["burst"],
                "unit": "TFLOP/s", "frac": top["frac_of_peak"], "traffic": NCU_TRAFFIC.get(base),
                "traffic_note": "dram read+write bytes per launch from the ncu captures summarised under profiles/",
                "peak_source": peaks["src"] + " cuBLAS bf16, the burst figure: every kernel is timed alone and the "
                               "whole step lasts well under a millisecond",
                "selection": "the kernel of the sparse path (attention, GEMM-Q, GEMM-O) with the largest share of the "
                             "step; the dense K/V projection, a plain GEMM, is listed under kernels",
                "kernels": kernels,
                "mask_compaction": {"kernel": "compact_count / compact_scan / compact_fill", "bound": "hbm",
                                    "launches_per_step": 3, "ms_per_step": r4(kt["compact"]["mean"]),
                                    "bytes": compact_bytes,
                                    "achieved_gbs": round(compact_bytes / (kt["compact"]["mean"] * 1e-3) / 1e9, 2),
                                    "peak_gbs": peaks["hbm_gbs"],
                                    "note": "a few KB of masks: launch latency, not bandwidth, sets the time here "
                                            "(see mask_path for the large mask); runs beside the projections"}}

    # ---- GEMM-Q + attention + GEMM-O alone (no dense K/V), replayed from a graph
    def trio():
        block.wrapper.prepare_masks(*m_dev)
        flashomni_gemm(x, weights.wq, H, m_dev[0], m_dev[2], 0, None, out=block.q, head_begin=hb, head_dim=D)
        attn_run()
        flashomni_gemm_reduction(block.attn, weights.wo, H, m_dev[0], m_dev[2], 0,
                                 block.cache if block.add_cache else None, is_for_cache=False, head_begin=hb,
                                 head_dim=D, out=block.y)

    for _ in range(3):
        trio()
    torch.cuda.synchronize()
    tg = torch.cuda.CUDAGraph()
    cs = torch.cuda.Stream(device)
    cs.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(cs):
        with torch.cuda.graph(tg, stream=cs):
            trio()
    for _ in range(3):
        tg.replay()
    ctx.barrier()
    t_trio = ctx.max_over_ranks([event_time(tg.replay, args.steps)["mean"]])[0]
    fl_trio = ctx.sum_over_ranks([fl["gemm_q"] + fl["attention"] + fl["gemm_o"]])[0]
    sparse_trio = {"ops": "GEMM-Q (sparse) + block-sparse attention + GEMM-O (active heads + cache), CUDA graph",
                   "ms": r4(t_trio), "executed_flops": fl_trio, "tflops": round(tf(fl_trio, t_trio), 1),
                   "frac_of_peak": r4(tf(fl_trio, t_trio) / (peaks["burst"] * world)), "peak": peaks["burst"] * world,
                   "target": 0.60}
    block.wrapper.check_status()

    # ---- spread of single steps, the same with L2 flushed, host time of plan()
    def each_step(flush):
        ts = []
        for _ in range(args.steps):
            if flush is not None:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return {"median": round(statistics.median(ts), 4), "min": round(min(ts), 4)}

    warm_ms = each_step(None)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    cold_ms = each_step(flush_buf)
    del flush_buf
    t0 = time.perf_counter()
    block.wrapper.plan(block.wrapper._qo_indptr_buf, block.wrapper._kv_indptr_buf, hc, hc, D, q_data_type=torch.bfloat16,
                       mask_num_heads=H, mask_head_begin=hb)
    replan_ms = (time.perf_counter() - t0) * 1e3
    timing_detail = {"step_ms": warm_ms, "step_ms_l2_flushed": cold_ms,
                     "per_kernel_sum_ms": r4(step_sum_ms),
                     "plan_host_ms_first": round(block.plan_host_ms, 3), "plan_host_ms_again": round(replan_ms, 3)}

    fl_rank = fl["gemm_q"] + fl["gemm_kv"] + fl["attention"] + fl["gemm_o"]
    fl_total = ctx.sum_over_ranks([fl_rank])[0]
    out = {
        "metric": METRIC, "value": round(tf(fl_total, ms), 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
        "latency_us": round(ms * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "flux_block: hidden 3072, H=24, D=128, S=4608, batch 2, block density 0.5 "
                               "(GEMM-Q sparse, GEMM-K/V dense, block-sparse attention, GEMM-O active heads + cache)",
                   "parallelism": f"heads/{world}", "seed": SEED, "cuda_graph": bool(args.graph), "steps_per_graph": steps_per_graph,
                   "schedule": args.schedule, "kv_projection": "one fused launch" if block.fuse_kv else "two launches",
                   "l2": "per-step working set (x, 4 weights, q/k/v, attention out, cache, y) is >200 MB per rank, "
                         "larger than the 126 MB L2; no explicit flush",
                   "executed_flops_per_step": fl_total, "active_pairs": fl["active_pairs"],
                   "attention_tiles": fl["attn_tiles"]},
        "e2e": {"value": round(tf(fl_total, ms_e2e), 2), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e, 4),
                "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h_all,
                "path": "pinned host -> device copy of the hidden state and masks, block, result back to pinned host"
                        + ("" if world == 1 else "; each rank uploads 1/N of the rows, all-gather over NVLink, cross-rank "
                           "sum, each rank downloads the rows it owns")},
        "gpu_launches": launches_per_step * args.steps,
        "gpu_launches_per_step": launches_per_step,
        "clocks": clocks, "roofline": roofline, "sparse_trio": sparse_trio, "timing_detail": timing_detail,
    }
    if reduce_ms is not None:
        out["cross_rank_sum"] = reduce_ms
    out["parity"] = {"flux_block": parity}
    keep = {"masks": masks, "w": w, "x_host": x_host, "cache_host": cache_host}
    return out, keep


# ---------------------------------------------------------------------------------------------- sweeps (N = 1)
def run_sweeps(ctx, args, peaks):
    """The three sparse ops on their own configurations: GEMM-Q at three densities, GEMM-O in both polarities,
    attention at three densities; each timed with CUDA events over `steps` calls (op = list kernel + GEMM as a
    caller gets it; kernel = the GEMM / attention kernel alone on a prepared list)."""
    import flashomni_b200 as fo
    from flashomni_b200 import workloads as wl
    from flashomni_b200.gemm import prepare_gemm_o_list, prepare_gemm_q_list
    device = ctx.device
    std = HID ** -0.5
    x = wl.randn_bf16((1, S, HID), SEED + 21).to(device)
    wq = wl.randn_bf16((HID, HID), SEED + 22, std=std).to(device)
    prior = wl.randn_bf16((1, S, HID), SEED + 23).to(device)
    out = {}
    gq = {}
    for dens in (0.25, 0.5, 0.75):
        m = wl.flux_masks(1, H, S // 128, S // 128, dens, SEED + 30)
        si, ip = torch.from_numpy(m.sparse_info).to(device), torch.from_numpy(m.info_indptr).to(device)
        act = int(m.q_active[0].sum())
        flops = act * FL_GEMM_TILE
        y = prior.clone()
        op = event_time(lambda: fo.flashomni_gemm(x, wq, H, si, ip, 0, None, out=y), args.steps)
        lst = prepare_gemm_q_list(1, S, HID, H, si, ip, 0)
        ker = event_time(lambda: fo.flashomni_gemm(x, wq, H, si, ip, 0, None, out=y, worklist=lst), args.steps)
        gq[str(dens)] = {"active_tiles": act, "op_us": round(op["mean"] * 1e3, 1), "kernel_us": round(ker["mean"] * 1e3, 1),
                         "kernel_tflops": round(tf(flops, ker["mean"]), 1),
                         "kernel_frac_of_peak": r4(tf(flops, ker["mean"]) / peaks["burst"])}
    out["gemm_q"] = gq
    m = wl.flux_masks(1, H, S // 128, S // 128, 0.5, SEED + 31)
    si, ip = torch.from_numpy(m.sparse_info).to(device), torch.from_numpy(m.info_indptr).to(device)
    a = wl.randn_bf16((1, S, HID), SEED + 24).to(device)
    wo = wl.randn_bf16((HID, HID), SEED + 25, std=std).to(device)
    bias1 = wl.randn_bf16((HID,), SEED + 26).to(device)
    act = int(m.q_active[0].sum())
    tot = m.q_active[0].size
    go = {}
    yo = torch.empty((1, S, HID), dtype=torch.bfloat16, device=device)
    for name, for_cache, bias, pairs in (("is_for_cache=True", True, bias1, tot - act), ("is_for_cache=False", False, prior, act)):
        flops = pairs * FL_GEMM_TILE
        op = event_time(lambda: fo.flashomni_gemm_reduction(a, wo, H, si, ip, 0, bias, is_for_cache=for_cache, out=yo),
                        args.steps)
        lst = prepare_gemm_o_list(1, S, HID, H, si, ip, 0, is_for_cache=for_cache)
        ker = event_time(lambda: fo.flashomni_gemm_reduction(a, wo, H, si, ip, 0, bias, is_for_cache=for_cache, out=yo,
                                                             worklist=lst), args.steps)
        go[name] = {"computed_pairs": pairs, "op_us": round(op["mean"] * 1e3, 1), "kernel_us": round(ker["mean"] * 1e3, 1),
                    "kernel_tflops": round(tf(flops, ker["mean"]), 1),
                    "kernel_frac_of_peak": r4(tf(flops, ker["mean"]) / peaks["burst"])}
    out["gemm_o_density_0.5"] = go
    at = {}
    filler = torch.randn(4096, 4096, device=device, dtype=torch.bfloat16)
    for dens in (0.25, 0.5, 0.75, 1.0):
        inp = wl.attention_inputs(1, H, S, D, dens, SEED + 40)
        q, k, v = (t.to(device) for t in (inp.q, inp.k, inp.v))
        mm = [torch.from_numpy(t).to(device) for t in (inp.masks.sparse_info, inp.masks.sparse_kv_info,
                                                        inp.masks.info_indptr, inp.masks.kv_info_indptr)]
        wr = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=device))
        ind = inp.qo_indptr.to(device)
        wr.plan(ind, ind, H, H, D, q_data_type=torch.bfloat16)
        o = torch.zeros_like(q)
        tiles = wl.executed_attention_tiles(inp.masks)
        flops = tiles * FL_ATTN_TILE
        for _ in range(3):
            wr.run(q, k, v, *mm, out=o)
        op = event_time(lambda: wr.run(q, k, v, *mm, out=o), args.steps)
        # the work lists are built on the side stream while a filler GEMM keeps the main stream busy, so that the
        # attention launch that follows does not wait for them
        ker = {"mean": chain_time([("fill", lambda: torch.matmul(filler, filler)),
                                   ("attn", lambda: wr.run(q, k, v, *mm, out=o))], args.steps,
                                  pre=lambda: wr.prepare_masks(*mm))["attn"]}
        wr.check_status()
        at[str(dens)] = {"tiles": tiles, "op_us": round(op["mean"] * 1e3, 1), "kernel_us": round(ker["mean"] * 1e3, 1),
                         "kernel_tflops": round(tf(flops, ker["mean"]), 1),
                         "kernel_frac_of_peak": r4(tf(flops, ker["mean"]) / peaks["burst"])}
    out["attention"] = at
    out["note"] = ("configs 1-3 on their own inputs (batch 1, 4608 tokens): op = what a caller's call costs (list or "
                   "compaction kernels included), kernel = the tensor-core kernel alone on a prepared list")
    return out


def run_mask_path(ctx, args, peaks):
    """segment_packbits and the compaction at the video layer's mask size (40 heads x 604 x 604 blocks = 14.6 M
    bits, 1.8 MB packed): algorithmic bytes / time against the measured HBM bandwidth."""
    import flashomni_b200 as fo
    from flashomni_b200 import workloads as wl
    device = ctx.device
    Hv, frames, bpf = 40, 20, 30
    n = 4 + frames * bpf
    m = wl.video_masks(Hv, frames, bpf, SEED)
    kk = torch.from_numpy(m.kv_kept[0].reshape(-1)).to(device)
    ind = torch.tensor([0, kk.numel()], dtype=torch.int32, device=device)
    for _ in range(3):
        fo.segment_packbits(kk, ind, bitorder="little")
    t = event_time(lambda: fo.segment_packbits(kk, ind, bitorder="little"), args.steps)
    pk_bytes = kk.numel() + (kk.numel() + 7) // 8
    res = {"segment_packbits": {"bits": int(kk.numel()), "bytes": int(pk_bytes), "us": round(t["mean"] * 1e3, 1),
                                "gbs": round(pk_bytes / (t["mean"] * 1e-3) / 1e9, 1),
                                "frac_of_hbm": r4(pk_bytes / (t["mean"] * 1e-3) / 1e9 / peaks["hbm_gbs"]),
                                "includes": "the cumsum of the byte indptr and its host read, as the reference's wrapper does"}}
    # the kernel alone through the C ABI
    from flashomni_b200 import _native
    lib = _native.load()
    y = torch.empty((kk.numel() + 7) // 8, dtype=torch.uint8, device=device)
    new_ind = torch.tensor([0, y.numel()], dtype=torch.int32, device=device)
    # a launch of a few microseconds through ctypes is host-bound: the launches are replayed from a CUDA graph
    # ... over twelve copies of the input in turn (175 MB, more than the 126 MB L2), so that every launch reads DRAM
    copies = [kk.clone() for _ in range(12)]
    turn = [0]

    def pack_once(s_):
        src = copies[turn[0] % len(copies)]
        turn[0] += 1
        lib.fo_segment_packbits(src.data_ptr(), ind.data_ptr(), new_ind.data_ptr(), 1, y.numel(), 1, y.data_ptr(), s_)

    tk = graph_time(pack_once, device, reps=24)
    del copies
    res["segment_packbits"]["kernel_us"] = round(tk["mean"] * 1e3, 1)
    res["segment_packbits"]["kernel_gbs"] = round(pk_bytes / (tk["mean"] * 1e-3) / 1e9, 1)
    res["segment_packbits"]["kernel_frac_of_hbm"] = r4(pk_bytes / (tk["mean"] * 1e-3) / 1e9 / peaks["hbm_gbs"])
    res["segment_packbits"]["kernel_timing"] = ("24 launches replayed from one CUDA graph over 12 copies of the input in "
                                                "turn (175 MB > L2): launch gaps included, every launch reads DRAM")
    mm = [torch.from_numpy(a).to(device) for a in (m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr)]
    wr = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=device))
    indp = torch.tensor([0, n * 128], dtype=torch.int32, device=device)
    wr.plan(indp, indp, Hv, Hv, D, q_data_type=torch.bfloat16)
    for _ in range(3):
        wr.build_work_lists(*mm)
    tc = event_time(lambda: wr.build_work_lists(*mm), args.steps)
    wr.check_status()
    lists = wr.work_lists()
    cb = int(sum(t_.numel() * t_.element_size() for t_ in mm) + 4 * (6 * lists["n_items"] + 1) + 4 * lists["total_kept"])
    res["compaction"] = {"items": lists["n_items"], "kept": lists["total_kept"], "bytes": cb,
                         "us": round(tc["mean"] * 1e3, 1), "gbs": round(cb / (tc["mean"] * 1e-3) / 1e9, 1),
                         "frac_of_hbm": r4(cb / (tc["mean"] * 1e-3) / 1e9 / peaks["hbm_gbs"]),
                         "bytes_are": "packed masks + indptrs read, items / kv_ptr / order / kv_idx written"}
    # block selection (pooled scores -> packed masks) at both mask sizes, beside the reference's torch + Triton
    # path as the fixture generator timed it on a B200 (tests/golden/make_selection_golden.py)
    ref_us = {}
    try:
        import json as _json
        z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tests", "golden", "reference_selection.npz"))
        ref_us = _json.loads(bytes(z["timing_us"]).decode())
    except Exception:
        pass
    sel = {}
    for name, Hs, ns, t2t in (("flux", 24, 36, 4), ("video", 40, 604, 4)):
        sc = torch.from_numpy((np.random.default_rng(9).standard_normal((1, Hs, ns, ns)) * 2.0).astype(np.float32)).to(device)
        for _ in range(3):
            fo.select_blocks(sc, t2t, 0.3, 0.3)
        ts = event_time(lambda: fo.select_blocks(sc, t2t, 0.3, 0.3), args.steps)
        sb = int(sc.numel() * 4 + (ns * Hs * ns + 7) // 8 + (ns * Hs + 7) // 8)
        sel[name] = {"heads": Hs, "blocks": ns, "us": round(ts["mean"] * 1e3, 1), "bytes": sb,
                     "gbs": round(sb / (ts["mean"] * 1e-3) / 1e9, 1),
                     "frac_of_hbm": r4(sb / (ts["mean"] * 1e-3) / 1e9 / peaks["hbm_gbs"]),
                     "reference_torch_triton_us": round(ref_us[name]["us"], 1) if name in ref_us else None}
    sel["bytes_are"] = "fp32 scores read, packed masks written"
    sel["reference_us_from"] = "tests/golden/reference_selection.npz (the generator's CUDA-event timing on a B200)"
    res["block_selection"] = sel
    res["peak_gbs"] = peaks["hbm_gbs"]
    return res


def run_baselines(ctx, args, keep):
    """Same inputs as the flux block: (R) the reference's own CUDA kernels rebuilt for sm_100a (the checker library
    under oracle/_ref, when it was built), (D) dense library kernels (torch SDPA, flash-attn, torch.matmul)."""
    from flashomni_b200 import workloads as wl
    device = ctx.device
    masks, w = keep["masks"], keep["w"]
    T = B * S
    x = keep["x_host"].to(device)
    m_dev = [torch.from_numpy(a).to(device) for a in (masks.sparse_info, masks.sparse_kv_info, masks.info_indptr,
                                                      masks.kv_info_indptr)]
    q = wl.randn_bf16((T, H, D), SEED + 50).to(device)
    k = wl.randn_bf16((T, H, D), SEED + 51).to(device)
    v = wl.randn_bf16((T, H, D), SEED + 52).to(device)
    wq = w["wq"].to(device)
    steps = min(args.steps, 10)
    res = {}
    try:
        from oracle import ref_cuda
        if ref_cuda.available():
            qo = torch.tensor([0, S, 2 * S], dtype=torch.int32, device=device)
            o = torch.zeros_like(q)
            plan = ref_cuda.plan_unsplit(qo.cpu().numpy(), qo.cpu().numpy(), device)
            y = torch.zeros((B, S, HID), dtype=torch.bfloat16, device=device)
            fns = {"attention_us": lambda: ref_cuda.sparse_attention(q, k, v, qo, qo, *m_dev, o, plan=plan),
                   "gemm_q_us": lambda: ref_cuda.gemm_q(x, wq, y, H, m_dev[0], m_dev[2], 0),
                   "gemm_dense_us": lambda: ref_cuda.gemm_q(x, wq, y, H, m_dev[0], m_dev[2], 0, is_full=True),
                   "gemm_o_us": lambda: ref_cuda.gemm_o(x, wq, y, H, m_dev[0], m_dev[2], 0, None, False)}
            r = {}
            for name, fn in fns.items():
                for _ in range(2):
                    fn()
                r[name] = round(event_time(fn, steps)["mean"] * 1e3, 1)
            r["what"] = ("the reference's kernels (prefill.cuh, gemm.cuh, gemm_reduction.cuh) compiled for sm_100a, "
                         "flux_block shapes, batch 2, same masks")
            res["reference_cuda"] = r
        else:
            res["reference_cuda"] = {"unavailable": "oracle/_ref/libflashomni_ref.so is not built"}
    except Exception as e:  # noqa: BLE001
        res["reference_cuda"] = {"unavailable": f"{type(e).__name__}: {e}"}
    dense = {}
    try:
        import torch.nn.functional as F
        qh = q.view(B, S, H, D).transpose(1, 2)
        kh = k.view(B, S, H, D).transpose(1, 2)
        vh = v.view(B, S, H, D).transpose(1, 2)
        for _ in range(2):
            F.scaled_dot_product_attention(qh, kh, vh)
        t = event_time(lambda: F.scaled_dot_product_attention(qh, kh, vh), steps)["mean"]
        dense_fl = B * H * (S // 128) ** 2 * FL_ATTN_TILE
        dense["sdpa_dense_us"] = round(t * 1e3, 1)
        dense["sdpa_dense_tflops"] = round(tf(dense_fl, t), 1)
    except Exception as e:  # noqa: BLE001
        dense["sdpa"] = f"unavailable: {type(e).__name__}"
    try:
        from flash_attn import flash_attn_func
        qf, kf, vf = q.view(B, S, H, D), k.view(B, S, H, D), v.view(B, S, H, D)
        for _ in range(2):
            flash_attn_func(qf, kf, vf)
        t = event_time(lambda: flash_attn_func(qf, kf, vf), steps)["mean"]
        dense["flash_attn_dense_us"] = round(t * 1e3, 1)
    except Exception as e:  # noqa: BLE001
        dense["flash_attn"] = f"unavailable: {type(e).__name__}"
    x2 = x.view(T, HID)
    for _ in range(2):
        torch.matmul(x2, wq.T)
    t = event_time(lambda: torch.matmul(x2, wq.T), steps)["mean"]
    dense["matmul_9216x3072x3072_us"] = round(t * 1e3, 1)
    dense["matmul_tflops"] = round(tf(2 * T * HID * HID, t), 1)
    dense["what"] = "dense library kernels on the flux_block shapes (all blocks computed): what the sparse path is compared with"
    res["dense_library"] = dense
    return res


# ---------------------------------------------------------------------------------------------- video layer
def run_video(ctx, args, peaks, standalone=False):
    """Long video layer (hidden 5120, H=40, D=128, 20 frames x 3840 + 512 text = 77 312 tokens, batch 1, block
    density ~0.25) under Ulysses sequence parallelism: tokens sharded by 128-token blocks, an exchange (pulls over
    peer memory, or the NCCL all-to-all) before and after the attention. Strong scaling of a fixed job."""
    from flashomni_b200 import workloads as wl
    from flashomni_b200.layer import BlockWeights, UlyssesSparseDiTAttentionBlock
    world, rank, device, dist = ctx.world, ctx.rank, ctx.device, ctx.dist
    hid, Hv, frames, bpf = 5120, 40, 20, 30
    Sv = (4 + frames * bpf) * 128
    masks = wl.video_masks(Hv, frames, bpf, SEED)
    std = hid ** -0.5
    w_host = [wl.randn_bf16((hid, hid), SEED + i, std=std) for i in range(10, 14)]
    weights = BlockWeights(*(t.to(device) for t in w_host))
    blk = UlyssesSparseDiTAttentionBlock(weights, Hv, D, Sv, rank, world, device)
    x_host = wl.randn_bf16((1, blk.s_loc, hid), SEED + 1 + rank)
    cache_host = wl.randn_bf16((1, blk.s_loc, hid), SEED + 100 + rank)
    x = x_host.to(device)
    blk.cache.copy_(cache_host.to(device))
    m_dev = [torch.from_numpy(a).to(device) for a in (masks.sparse_info, masks.sparse_kv_info, masks.info_indptr,
                                                      masks.kv_info_indptr)]
    steps = max(3, min(args.steps, 10))

    def step():
        return blk.forward(x, *m_dev)

    for _ in range(3):
        step()
    ctx.barrier()
    blk.check_status()
    sampler = ClockSampler(ctx.local_rank).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    blk.check_status()
    # phase breakdown of two more steps (outside the timed region)
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
    pm = ctx.max_over_ranks([phases[n] for n in phases])
    phases_max = {n: round(float(v), 4) for n, v in zip(phases, pm)}
    tiles = wl.executed_attention_tiles(masks, blk.hb, blk.hc)
    fl_rank = tiles * FL_ATTN_TILE + 4 * (2 * blk.s_loc * hid * hid)
    ms = ctx.max_over_ranks([ms])[0]
    fl_total = ctx.sum_over_ranks([fl_rank])[0]

    # ---- parity at this N (outside the timed region)
    parity = None
    if not args.no_parity:
        parity = video_parity(ctx, blk, masks, w_host, x_host, cache_host, hid, Hv, Sv)
    res = {"workload": "video_layer: hidden 5120, H=40, D=128, S=77312 (20 frames x 3840 + 512 text), batch 1, "
                       "spatiotemporal-local block mask (+-1 frame + 10% random + text), Ulysses sequence parallelism",
           "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": round(ms, 4),
           "tflops": round(tf(fl_total, ms), 2), "frac_of_peak": r4(tf(fl_total, ms) / (peaks["burst"] * world)),
           "executed_flops_per_step": fl_total, "parallelism": f"ulysses/{world}", "exchange": blk.exchange,
           "attention_tiles_rank0": tiles, "l2": "working set of several GB, far above the 126 MB L2",
           "phase_ms_rank0": phases, "phase_ms_slowest_rank": phases_max, "clocks": clocks, "parity": parity}
    if standalone and rank == 0:
        print(json.dumps({"metric": METRIC, "value": res["tflops"], "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
                          "warmup": 3, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": {"workload": res["workload"]},
                          "video": res}), flush=True)
    del blk
    torch.cuda.empty_cache()
    return res


def video_parity(ctx, blk, masks, w_host, x_host, cache_host, hid, Hv, Sv):
    """Checks of one step of the video layer on this rank's share, each against the CPU oracle (fp32) or, for the
    exchange, an exact integer checksum: (1) sampled local row blocks of the Q / K / V projections; (2) the
    exchange: for every (source rank, head window) the sum of the 16-bit patterns sent equals the sum received;
    (3) sampled (head, q-block) rows of the attention over their kept kv blocks; (4) a sampled local row block of
    the final output = cache + attention output (all heads) x W_o^T. Every rank checks its own share; the result is
    the worst over the ranks."""
    from flashomni_b200 import parallel as par
    from oracle import attention as oa
    from flashomni_b200 import workloads as wl
    world, rank, device, dist = ctx.world, ctx.rank, ctx.device, ctx.dist
    wq, wk, wv, wo = w_host
    worst = {"projection": 0.0, "attention": 0.0, "output": 0.0}
    mean = {"projection": 0.0, "attention": 0.0, "output": 0.0}
    excess = [-1.0]

    def note(kind, got, ref):
        mx, mn, ex = cmp_bf16(got, ref)
        worst[kind], mean[kind], excess[0] = max(worst[kind], mx), max(mean[kind], mn), max(excess[0], ex)

    torch.cuda.synchronize()
    nloc = blk.s_loc // 128
    # (1) projections on two local row blocks
    for lb in sorted({0, nloc - 1}):
        rows = slice(lb * 128, lb * 128 + 128)
        xr = x_host[0, rows].float()
        for wt, got in ((wq, blk.q), (wk, blk.k), (wv, blk.v)):
            note("projection", got[0, rows], xr @ wt.float().T)
    # (2) exchange checksum (exact): per (source rank s, destination rank r) the int64 sum of the bit patterns
    exch_ok = True
    if world > 1:
        qh = blk.heads_in[0]
        sent = torch.zeros(world, dtype=torch.int64, device=device)
        recv = torch.zeros(world, dtype=torch.int64, device=device)
        qv = blk.q[0].view(blk.s_loc, Hv, D).view(torch.int16).to(torch.int64)
        for r in range(world):
            hb_r, hc_r = par.head_window(Hv, r, world)
            sent[r] = qv[:, hb_r:hb_r + hc_r].sum()
            a, b = par.token_range(Sv, r, world)
            recv[r] = qh[a:b].view(torch.int16).to(torch.int64).sum()
        all_sent = [torch.zeros_like(sent) for _ in range(world)]
        dist.all_gather(all_sent, sent)
        for s_rank in range(world):   # what rank s_rank sent to me == what I hold of its tokens
            if int(all_sent[s_rank][rank]) != int(recv[s_rank]):
                exch_ok = False
    # (3) attention rows: local heads, sampled q-blocks, CPU oracle over the kept blocks
    if world > 1:
        qh, kh, vh = blk.heads_in
    else:
        qh, kh, vh = (t.view(Sv, Hv, D) for t in (blk.q, blk.k, blk.v))
    nblk = Sv // 128
    rng = np.random.default_rng(7 + rank)
    picks = [(0, 0), (blk.hc - 1, nblk - 1), (int(rng.integers(blk.hc)), int(rng.integers(4, nblk)))]
    for hl, qb in picks:
        kept = np.nonzero(masks.kv_kept[0][qb, blk.hb + hl])[0]
        cols = torch.from_numpy(np.concatenate([np.arange(j * 128, j * 128 + 128) for j in kept])).to(device)
        qs = qh[qb * 128:(qb + 1) * 128, hl:hl + 1].cpu()
        ks, vs = kh[cols, hl:hl + 1].cpu(), vh[cols, hl:hl + 1].cpu()
        ref = oa.sparse_attention(qs, ks, vs, [0, 128], [0, ks.shape[0]], is_full=True)
        note("attention", blk.attn[qb * 128:(qb + 1) * 128, hl], ref[:, 0])
    # (4) final output rows of one local row block: cache + o_loc W_o^T
    lb = nloc // 2
    rows = slice(lb * 128, lb * 128 + 128)
    o_loc = (blk.o_loc if (world > 1 and blk.exchange == "p2p") else None)
    if o_loc is None:
        if world > 1:
            o_loc = par.heads_to_tokens(blk.attn, Sv, blk.group)
        else:
            o_loc = blk.attn
    ref = cache_host[0, rows].float() + o_loc.view(blk.s_loc, Hv * D)[rows].float().cpu() @ wo.float().T
    note("output", blk.y[0, rows], ref)
    ok = exch_ok and excess[0] <= 0 and all(mean[k] <= 2e-3 for k in mean)
    vals = ctx.max_over_ranks([0.0 if ok else 1.0] + [worst[k] for k in ("projection", "attention", "output")]
                              + [mean[k] for k in ("projection", "attention", "output")])
    return {"ok": bool(vals[0] == 0.0), "exchange_checksum_ok": bool(exch_ok),
            "max_abs": {k: r4(v) for k, v in zip(("projection", "attention", "output"), vals[1:4])},
            "mean_abs": {k: round(v, 5) for k, v in zip(("projection", "attention", "output"), vals[4:7])},
            "bounds": "max-abs 2e-2 (one bf16 ulp where |value| >= 4), mean-abs 2e-3; worst over the ranks",
            "sampled": "2 local row blocks (projections), 3 (head, q-block) rows per rank (attention), 1 local row block "
                       "(output), exact integer checksum of every (source, destination) slice of the Q exchange",
            "against": "oracle/ (CPU fp32) and fp32 torch on the host"}


# ---------------------------------------------------------------------------------------------- CPU legs
def cpu_sample_step(masks, w, x_host, cache_host, heads=(0, 1, 2, 3, 4, 5), row_blocks=36):
    """One bounded sample of the block on the CPU oracle: the attention of `heads` of request 0 (full
    sequence) and the four GEMMs on the first `row_blocks` 128-row blocks of request 0. Returns the
    executed FLOPs of the sample."""
    from flashomni_b200 import workloads as wl
    from oracle import attention as oa
    from oracle import gemm as og
    rows = row_blocks * 128
    xs = x_host[:1, :rows]
    og.gemm_q(xs, w["wq"], H, masks.sparse_info, masks.info_indptr, 0, None, None)
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


def cpu_baseline(masks, w, x_host, cache_host, budget_s=12.0):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cpu_sample_step(masks, w, x_host, cache_host, heads=(0,), row_blocks=1)  # warm-up
    t0 = time.perf_counter()
    fl, steps = 0, 0
    while True:
        f, sample = cpu_sample_step(masks, w, x_host, cache_host)
        fl += f
        steps += 1
        if time.perf_counter() - t0 > budget_s or steps >= 40:
            break
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


def run_ours(args):
    ctx = Ctx()
    from flashomni_b200 import _native
    _native.load()
    peaks = load_peaks()
    if args.workload == "video":
        run_video(ctx, args, peaks, standalone=True)
    elif args.workload == "masks":   # the mask path alone (packing, compaction, block selection at the video mask)
        if ctx.rank == 0:
            print(json.dumps({"metric": "mask path at the video layer's mask", "unit": "GB/s", "n_gpus": 1,
                              "steps": args.steps, "mask_path": run_mask_path(ctx, args, peaks)}), flush=True)
    else:
        out, keep = run_flux(ctx, args, peaks)
        if ctx.world == 1 and not args.quick:
            out["sweep"] = run_sweeps(ctx, args, peaks)
            out["mask_path"] = run_mask_path(ctx, args, peaks)
            out["baselines"] = run_baselines(ctx, args, keep)
        if not args.no_video:
            torch.cuda.empty_cache()
            video = run_video(ctx, args, peaks)
            out["video"] = video
            out["parity"]["video"] = video.pop("parity")
        if ctx.rank == 0:
            if ctx.world == 1 and not args.no_cpu_baseline:
                out["cpu_baseline"] = cpu_baseline(keep["masks"], keep["w"], keep["x_host"], keep["cache_host"])
            print(json.dumps(out), flush=True)
    if ctx.dist is not None:
        ctx.dist.barrier()
        ctx.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="flux_block", choices=["flux_block", "video", "masks"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-video", action="store_true", help="skip the video-layer leg of the default run")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled-row parity checks")
    ap.add_argument("--quick", action="store_true", help="skip the sweeps, the mask-path figures and the baselines")
    ap.add_argument("--schedule", default="kv_first", choices=["q_first", "kv_first"],
                    help="flux_block: order of the projections and where the list kernels run")
    ap.add_argument("--graph", dest="graph", action="store_true", default=True,
                    help="replay the step from a CUDA graph (device-resident leg; the default: at 8 GPUs a step is "
                         "about 100 us of kernels and eager launches are host-bound)")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="launch the step eagerly")
    ap.add_argument("--steps-per-graph", type=int, default=0,
                    help="steps captured in one CUDA graph (0: one, or as many as fit in about 0.65 ms when a step is under 0.27 ms)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
