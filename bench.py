#!/usr/bin/env python
"""Benchmark of the quantized matmul hot path on B200.

Headline workload (N=1): the Qwen3-8B-shaped decode step at batch 1 - 36 layers of Q/K/V/O,
fused gate+up+SwiGLU and down projections plus the LM head, Q4_K_M mix (Q4_K attention
and gate/up, Q6_K down and LM head), random weights, N(0,1) f32 activations. Every
projection is one dequant-matvec through the C ABI; the step is recorded once into a
CUDA graph (zc_begin_record / zc_end_record) and replayed per token.

Metric: quantized weight bytes streamed per second (GB/s), whole job.
  value : weights, activations and outputs resident in HBM; CUDA events around blocks of K replays
          (several blocks, the median block is reported, the best beside it).
  e2e   : per token, the three activation vectors are copied from pinned host memory, the
          step runs, and the logits + hidden vector are copied back to pinned host memory,
          all through the C ABI; wall clock around K such tokens (device idle on both sides).
Each token streams 4.88 GB of distinct weights, far more than the 126 MB L2, so no cache
flush is needed between steps.

The same line carries a `workloads` object with the other parts of the metric, each timed the same
way with its own roofline and the clock samples that fell inside its timed loop: the single
Q4_K 4096 x 4096 matvec, the batched-prefill dequant-GEMM cases (TFLOP/s) and the two MoE
configurations at batch 1 and over a prefill batch. `--workload <name>` runs one of them alone and
prints one line per case.

N>1 (torchrun): tensor parallel over the ranks (strong scaling): Q/K/V, gate/up and LM
head sharded by rows, O and down along K; hidden-state sums and the logits gather over NVLink
peer memory (`--collective nccl` for the NCCL baseline). Before the timed region a small layer
stack cut from the same seeded tensors on every rank runs through the same exchange and is
compared with the unsharded step (`tp_check`); the run fails if it differs by more than 1e-4.

`--impl reference` times the CPU restatement of the reference's decode shaders (the
oracle's shader-order DMMV, all host threads) on one layer's seven projections per step.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "dmmv_weight_gbs"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
NOMINAL_BF16_TFLOPS = 2250.0
GATE_UP_KEY = "dmmv_gate_up_q4k_12288x4096"


def measured_peaks():
    """(HBM GB/s, bf16 burst TFLOP/s, bf16 sustained TFLOP/s, 'measured' | 'fallback')."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), float(p["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 6650.0, 1590.0, 1400.0, "fallback"


def ncu_traffic(kernel_key: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary
    (a line `traffic_bytes <key> <bytes>` in profiles/dmmv_q4k_warp_kernel_gate_up.txt), or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "dmmv_q4k_warp_kernel_gate_up.txt")) as f:
            for line in f:
                w = line.split()
                if len(w) == 3 and w[0] == "traffic_bytes" and w[1] == kernel_key:
                    return float(w[2])
    except Exception:
        pass
    return None


def host_threads() -> int:
    """Cores this process may run on (torchrun pins OMP_NUM_THREADS to 1, so OpenMP's own default is
    not a measure of the host)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi for the life of the run; `window(t0, t1)`
    summarises the samples taken between two wall-clock instants (none outside them are ever used)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int, period_ms: int = 50):
        self.gpu = gpu_index
        self.period_ms = period_ms
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return self
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def window(self, t0: float, t1: float):
        sm, mx, reasons = [], [], set()
        for ts, line in list(self.samples):
            if not (t0 <= ts <= t1):
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window_s": round(t1 - t0, 3)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()


class _NoSampler:
    def window(self, t0, t1):
        return None


# ---- timing helpers --------------------------------------------------------------------------------
def timed_blocks(torch, stream, replay, steps: int, barrier=None, min_total_s: float = 0.6, min_blocks: int = 5,
                 max_blocks: int = 40, fixed_blocks: int = 0):
    """Blocks of `steps` calls of replay(), each bracketed by CUDA events on `stream`. Runs at least
    min_blocks blocks and until min_total_s of device time has been timed, so that clock samples fall
    inside the region (fixed_blocks > 0: exactly that many, for ranks that must agree on the count).
    Returns (ms per step of every block, wall t0, wall t1)."""
    per = []
    if barrier:
        barrier()
    t0 = time.time()
    total_ms = 0.0
    while (len(per) < fixed_blocks if fixed_blocks else
           len(per) < min_blocks or (total_ms < min_total_s * 1e3 and len(per) < max_blocks)):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(steps):
            replay()
        ev1.record(stream)
        stream.synchronize()
        ms = ev0.elapsed_time(ev1)
        total_ms += ms
        per.append(ms / steps)
    t1 = time.time()
    if barrier:
        barrier()
    return per, t0, t1


def graph_of(torch, stream, fn):
    """fn() run once eagerly (warm-up of every kernel variant), then captured into a CUDA graph."""
    fn()
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn()
    for _ in range(3):
        g.replay()
    stream.synchronize()
    return g


def hbm_roofline(bytes_per_launch, us, peak, peak_kind, traffic=None, **extra):
    gbs = bytes_per_launch / us / 1e3
    r = {"bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": gbs / peak,
         "frac_of_nominal_8tbs": gbs / NOMINAL_HBM_GBS, "algorithmic_bytes_per_launch": bytes_per_launch,
         "us_per_launch": us, "traffic": traffic}
    r.update(extra)
    return r


# ---- CPU arms --------------------------------------------------------------------------------------
def cpu_reference_arm(args):
    """The reference's decode shaders restated on the CPU, timed on this host's cores."""
    from oracle import oracle as o
    from zinc_b200 import synth
    from zinc_b200.decode_step import QWEN3_8B as S

    mats = [(S.t_attn, S.q_dim, S.hidden), (S.t_attn, S.kv_dim, S.hidden), (S.t_attn, S.kv_dim, S.hidden),
            (S.t_attn, S.hidden, S.q_dim), (S.t_gate_up, S.ffn, S.hidden), (S.t_gate_up, S.ffn, S.hidden),
            (S.t_down, S.hidden, S.ffn)]
    g = synth.rng(2, 0)
    weights = [(t, M, K, synth.quant_matrix(g, t, M, K)) for t, M, K in mats]
    xs = {K: synth.activations(g, K) for K in (S.hidden, S.q_dim, S.ffn)}
    nbytes = sum(w.size for *_, w in weights)
    threads = host_threads()

    def step():
        for t, M, K, w in weights:
            o.dmmv_shader_order(w, t, M, K, xs[K], n_threads=threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = nbytes / dt / 1e9
    sample = (f"one layer's 7 projections ({nbytes} weight bytes) per step, shader-order CPU restatement, "
              f"{threads} host threads")
    return {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "qwen3-8b-shaped decode step, batch 1, Q4_K_M mix (CPU sample: one layer)",
                   "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def cpu_baseline_leg(torch, step, limit_s=12.0):
    """Oracle (shader-order port) timed on the host cores on layer 0's gate and down matrices."""
    import numpy as np

    from oracle import oracle as o

    S = step.shape
    lw = step.layers[0]
    g = step.world
    mats = [(S.t_gate_up, S.ffn // g, S.hidden, lw.wgate.cpu().numpy()),
            (S.t_down, S.hidden, S.ffn // g, lw.wdown.cpu().numpy())]
    xs = {S.hidden: np.random.default_rng(0).standard_normal(S.hidden).astype(np.float32),
          S.ffn // g: np.random.default_rng(1).standard_normal(S.ffn // g).astype(np.float32)}
    threads = host_threads()
    nbytes = sum(m[3].size for m in mats)

    def once():
        for t, M, K, w in mats:
            o.dmmv_shader_order(w, t, M, K, xs[K], n_threads=threads)

    once()
    t0 = time.perf_counter()
    once()
    one = time.perf_counter() - t0
    reps = max(1, min(200, int(limit_s / max(one, 1e-4))))
    t0 = time.perf_counter()
    for _ in range(reps):
        once()
    dt = (time.perf_counter() - t0) / reps
    return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"layer-0 gate (Q4_K {S.ffn // g}x{S.hidden}) + down (Q6_K {S.hidden}x{S.ffn // g}), "
                      f"{nbytes} weight bytes x {reps} repetitions"}


# ---- the other parts of the metric -------------------------------------------------------------------
def dmmv_single_results(torch, zb, dd, stream, sampler, quick):
    """One Q4_K 4096 x 4096 matvec (9 437 184 weight bytes), 64 weight copies in rotation (604 MB > L2),
    and the same on one copy (L2-hot), labelled."""
    from zinc_b200 import synth

    peak, _, _, kind = measured_peaks()
    dev = f"cuda:{torch.cuda.current_device()}"
    M = K = 4096
    copies = 64
    ws = [synth.torch_quant_matrix(zb.Q4_K, M, K, dev, 300 + i) for i in range(copies)]
    x = torch.randn(K, device=dev)
    y = torch.zeros(M, device=dev)
    wbytes = M * zb.row_bytes(zb.Q4_K, K)

    def rotating():
        for w in ws:
            dd.recordDispatch(zb.Q4_K, w, x, y, M, K)

    def hot():
        for _ in range(copies):
            dd.recordDispatch(zb.Q4_K, ws[0], x, y, M, K)

    out = []
    for label, fn in (("64 weight copies in rotation (604 MB, larger than L2)", rotating),
                      ("one weight copy, L2-hot", hot)):
        g = graph_of(torch, stream, fn)
        per, t0, t1 = timed_blocks(torch, stream, g.replay, 50, min_total_s=0.15 if quick else 0.4)
        us = statistics.median(per) * 1e3 / copies
        out.append({
            "metric": METRIC, "value": wbytes / us / 1e3, "unit": UNIT, "n_gpus": 1, "steps": len(per) * 50 * copies,
            "warmup": 4 * copies, "ms_per_step": us / 1e3, "best_ms_per_step": min(per) / copies,
            "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "single Q4_K matvec 4096x4096, f32 x", "l2": label, "weight_bytes": wbytes,
                       "reference_bytes_model": wbytes + 4 * K + 4 * M},
            "gpu_launches": len(per) * 50 * copies,
            "roofline": hbm_roofline(wbytes, us, peak, kind),
            "clocks": sampler.window(t0, t1),
        })
        g.reset()
    return out


def prefill_gemm_results(torch, zb, ctx, dd, stream, sampler, quick):
    """Batched-prefill dequant-GEMM D[T][M] = X[T][K] W[M][K]^T (bf16 activations, f32 out), one result per
    case: gate-shaped Q4_K 12288 x 4096, down-shaped Q6_K 4096 x 12288 and a GPT-OSS gate+up-shaped MXFP4
    5760 x 2880 at T = 128, 512, 2048. Each timed launch uses the next of 8 weight copies (more than L2 in
    total)."""
    from zinc_b200 import synth

    _, peak_burst, peak_sust, kind = measured_peaks()
    dev = f"cuda:{torch.cuda.current_device()}"
    copies = 8
    out = []
    for qt, name, M, K in ((zb.Q4_K, "q4_k", 12288, 4096), (zb.Q6_K, "q6_k", 4096, 12288),
                           (zb.MXFP4, "mxfp4", 5760, 2880)):
        ws = [synth.torch_quant_matrix(qt, M, K, dev, 100 + i) for i in range(copies)]
        # MXFP4 twice: weights dequantised to bf16 tiles, and (a workspace lent) as stored on the block-scaled path
        cases = [(T, path) for T in (128, 512, 2048) for path in (("bf16 tiles", "block-scaled") if qt == zb.MXFP4 else ("",))]
        for T, path in cases:
            X = torch.randn(T, K, device=dev).to(torch.bfloat16)
            D = torch.zeros(T * M, dtype=torch.float32, device=dev)
            wsp = None
            if path == "block-scaled":
                wsp = torch.empty(dd.mulMmWorkspaceBytes(qt, T, K), dtype=torch.uint8, device=dev)

            def call(wmat, wsp=wsp, X=X, D=D, T=T):
                if wsp is not None:
                    dd.recordMulMmBlockScaled(qt, wmat, X, D, M, T, K, K, M, wsp)
                else:
                    dd.recordMulMm(qt, wmat, X, D, M, T, K, K, M, 0, 0, 0, zb.BF16)

            n0 = ctx.launch_count
            for i in range(copies):
                call(ws[i])
            per_call = (ctx.launch_count - n0) // copies
            stream.synchronize()
            it = [0]

            def one():
                call(ws[it[0] % copies])
                it[0] += 1

            per, t0, t1 = timed_blocks(torch, stream, one, 24, min_total_s=0.15 if quick else 0.4, max_blocks=400)
            ctx.submit_and_wait()
            us = statistics.median(per) * 1e3
            flops = 2.0 * M * K * T
            tf = flops / us / 1e6
            wbytes = M * zb.row_bytes(qt, K)
            out.append({
                "metric": "prefill_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": len(per) * 24,
                "timed_blocks": len(per),
                "warmup": copies, "ms_per_step": us / 1e3, "best_ms_per_step": min(per), "higher_is_better": True,
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"prefill dequant-GEMM {name} {M}x{K}, T={T}, bf16 activations, f32 out",
                           **({"path": path + (" (tcgen05 kind::mxf8f6f4 with E8M0 block scales, weights as stored, two FP8 "
                                               "activation terms; the activation split kernel is inside the timed call)"
                                               if path == "block-scaled" else "")} if path else {}),
                           "l2": f"{copies} weight copies in rotation ({copies * ws[0].numel() / 1e6:.0f} MB)",
                           "bytes_per_launch": wbytes + T * K * 2 + T * M * 4},
                "gpu_launches": per_call * len(per) * 24,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": peak_burst, "peak_kind": kind + " (burst)",
                             "unit": "TFLOP/s", "frac": tf / peak_burst, "frac_of_sustained": tf / peak_sust,
                             "frac_of_nominal_dense_bf16": tf / NOMINAL_BF16_TFLOPS, "flops_per_launch": flops,
                             "us_per_launch": us, "traffic": None},
                "clocks": sampler.window(t0, t1),
            })
            del X, D, wsp
        del ws
        torch.cuda.empty_cache()
    return out


def moe_decode_results(torch, zb, ctx, dd, stream, sampler, args, rank=0, world=1, dist=None, parallelism="tp"):
    """One token through the MoE layers of the two MoE configurations at batch 1. With N ranks: the
    Qwen3.5-like configuration expert-parallel (whole experts per rank, the shared expert and the router
    replicated), the GPT-OSS-shaped one tensor-parallel (every expert's FFN dimension cut over the ranks);
    one peer all-reduce of the hidden vector per layer either way."""
    from zinc_b200.moe_step import GPT_OSS_MOE, QWEN35_MOE, MoeDecode

    peak, _, _, kind = measured_peaks()

    def allreduce(t):
        ctx.allreduce_sum(t, t.numel())

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    out = []
    for name, shape, mode in (("qwen3.5-35b-a3b-like MoE layers (256 experts top-8 + shared, Q4_K / Q6_K)", QWEN35_MOE, "ep"),
                              ("gpt-oss-20b-shaped MoE layers (32 experts top-4, MXFP4, expert biases)", GPT_OSS_MOE, "tp")):
        if args.layers:
            shape = dataclasses.replace(shape, n_layers=args.layers)
        try:
            step = MoeDecode.build(torch, dd, shape, rank=rank, world=world, allreduce=allreduce if world > 1 else None,
                                   parallel=mode, fused=args.moe_dispatch == "fused")
        except ValueError as e:
            if rank == 0:
                out.append({"metric": METRIC, "n_gpus": world, "config": {"workload": name + ", decode batch 1"},
                            "skipped": f"cut not possible: {e}"})
            continue
        launches = step.record()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step.record()
        for _ in range(4):
            graph.replay()
        per, t0, t1 = timed_blocks(torch, stream, graph.replay, 20, barrier=barrier if world > 1 else None,
                                   min_total_s=0.3, fixed_blocks=10 if world > 1 else 0)
        ms = statistics.median(per)
        if dist is not None:
            tt = torch.tensor([ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        gbs = shape.weight_bytes() / (ms * 1e-3) / 1e9
        if rank == 0:
            par = "single GPU" if world == 1 else (
                f"ep{world}: whole experts per rank, router and shared expert replicated, one peer all-reduce per layer"
                if step.parallel == "ep" else
                f"tp{world}: expert FFN dimension cut over the ranks, one peer all-reduce per layer")
            out.append({
                "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": world, "steps": len(per) * 20, "warmup": 4,
                "ms_per_step": ms, "best_ms_per_step": min(per), "higher_is_better": True, "scaling": "strong",
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": name + ", decode batch 1", "layers": shape.n_layers,
                           "weight_bytes_per_token": shape.weight_bytes(), "parallelism": par,
                           "dispatch": "router + selection / gate + up + activation / down + sum: three launches per layer"
                           if step.fused else "one launch per dispatch of the reference's sequence",
                           "l2": "weights touched per token (all layers) are larger than L2"},
                "gpu_launches": launches * len(per) * 20, "gpu_launches_per_step": launches,
                "gpu_launches_per_layer": launches / shape.n_layers,
                "roofline": hbm_roofline(shape.weight_bytes(), ms * 1e3, peak * world, kind),
                "clocks": sampler.window(t0, t1),
            })
        graph.reset()
        del graph, step
        torch.cuda.empty_cache()
    return out


def moe_prefill_results(torch, zb, ctx, dd, stream, sampler, args, per_pair=True):
    """The routed-expert matmuls of one MoE layer over a prefill batch: gate and up (one activation row per
    token, n_used experts each), activation, down (one row per (token, slot) pair) and the weighted scatter
    back to the tokens. Routing ids come from softmax_topk over N(0,1) logits, before the timed region.
    One result per configuration and path: grouped by expert on the tensor cores (with a workspace) and,
    when asked for, the per-pair kernel the reference's Vulkan path uses."""
    from zinc_b200 import synth
    from zinc_b200.moe_step import GPT_OSS_MOE, QWEN35_MOE

    peak, peak_burst, _, kind = measured_peaks()
    dev = f"cuda:{torch.cuda.current_device()}"
    out = []
    for name, S, T in (("qwen3.5-35b-a3b-like MoE layer (256 experts top-8, Q4_K gate/up, Q6_K down)", QWEN35_MOE, 512),
                       ("gpt-oss-20b-shaped MoE layer (32 experts top-4, MXFP4)", GPT_OSS_MOE, 1024)):
        T = args.tokens or T
        E, k, H, F = S.n_experts, S.top_k, S.hidden, S.ffn
        copies = 4   # layers in rotation: 2 GB (config 4) / 1.7 GB (config 5), larger than L2
        Wg = [synth.torch_quant_matrix(S.t_gate_up, E * F, H, dev, 11 + 10 * c) for c in range(copies)]
        Wu = [synth.torch_quant_matrix(S.t_gate_up, E * F, H, dev, 12 + 10 * c) for c in range(copies)]
        Wd = [synth.torch_quant_matrix(S.t_down, E * H, F, dev, 13 + 10 * c) for c in range(copies)]
        sg, sd = zb.expert_slice_bytes(S.t_gate_up, F, H), zb.expert_slice_bytes(S.t_down, H, F)
        X = torch.randn(T, H, device=dev)
        logits = torch.randn(T, E, device=dev)
        routing = torch.zeros(T * 2 * k, dtype=torch.int32, device=dev)
        dd.dispatchSoftmaxTopk(logits, routing, E, k, S.rule, T)
        ctx.submit_and_wait()
        ids = routing.view(T, 2 * k)[:, :k].contiguous()
        gate = torch.empty(T * k * F, device=dev)
        up = torch.empty(T * k * F, device=dev)
        act = torch.empty(T * k * F, device=dev)
        down = torch.empty(T * k * H, device=dev)
        hidden = torch.zeros(T * H, device=dev)
        touched = int(torch.unique(ids).numel())
        wbytes = touched * (2 * sg + sd)
        flops = 2.0 * T * k * 3 * F * H

        def layers():
            for c in range(copies):
                dd.recordMoeBatchedDispatchPair(S.t_gate_up, Wg[c], Wu[c], X, gate, up, ids, F, H, sg, E, k, T, H, k * F)
                dd.dispatchSwiglu(gate, up, act, T * k * F, oai=S.oai)
                dd.recordMoeBatchedDispatch(S.t_down, Wd[c], act, down, ids, H, F, sd, E, 1, T * k, F, H)
                dd.dispatchMoeRouteScatter(routing, down, hidden, T, H, k, 2 * k)

        ws = torch.empty(max(dd.moeGroupedWorkspaceBytes(T, k, H, E), dd.moeGroupedWorkspaceBytes(T * k, 1, F, E)),
                         dtype=torch.uint8, device=dev)
        for path in (("grouped", "per_pair") if per_pair else ("grouped",)):
            dd.setWorkspace(ws if path == "grouped" else None)
            n0 = ctx.launch_count
            layers()
            launches = (ctx.launch_count - n0) // copies
            g = graph_of(torch, stream, layers)
            per, t0, t1 = timed_blocks(torch, stream, g.replay, 4 if path == "grouped" else 1,
                                       min_total_s=0.3 if path == "grouped" else 0.0,
                                       min_blocks=5 if path == "grouped" else 2)
            ms = statistics.median(per) / copies
            gbs = wbytes / (ms * 1e-3) / 1e9
            tf = flops / (ms * 1e-3) / 1e12
            out.append({
                "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": 1, "steps": len(per) * copies, "warmup": 4,
                "ms_per_step": ms, "best_ms_per_step": min(per) / copies, "higher_is_better": True,
                "dtype": "bf16" if path == "grouped" and launches > 5 else "f32", "data": "synthetic",
                "config": {"workload": f"{name}, prefill T={T}, routed experts only", "path": path,
                           "experts_touched": touched, "weight_bytes_touched": wbytes,
                           "tokens_per_s": T / (ms * 1e-3), "tflops": tf,
                           "l2": f"{copies} layers' expert weights in rotation, larger than L2"},
                "gpu_launches": launches * len(per) * copies, "gpu_launches_per_step": launches,
                "roofline": hbm_roofline(wbytes, ms * 1e3, peak, kind, tensor_frac_of_burst=tf / peak_burst),
                "clocks": sampler.window(t0, t1),
            })
            g.reset()
        dd.setWorkspace(None)
        del Wg, Wu, Wd, ws
        torch.cuda.empty_cache()
    return out


def moe_prefill_ep_results(torch, zb, ctx, dd, stream, sampler, args, rank, world, dist):
    """N > 1: the Qwen3.5-like layer's routed experts over a prefill batch, expert-parallel: tokens and routing
    replicated, each rank groups and computes only the pairs of its own experts, one NCCL all-reduce of the
    [T][hidden] partial outputs per layer (a bandwidth-bound sum). Before the timed region a small layer cut from
    the same seeded tensors on every rank is compared with the unsharded layer (`ep_check`)."""
    from zinc_b200.moe_step import QWEN35_MOE, MoePrefill, MoeShape

    peak, peak_burst, _, kind = measured_peaks()

    def allreduce(t):
        dist.all_reduce(t)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # correctness of the partition and the sum, on a layer small enough to build unsharded everywhere
    small = MoeShape(hidden=512, n_experts=max(16, 2 * world), top_k=4, ffn=512, t_gate_up=zb.Q4_K, t_down=zb.Q6_K,
                     rule=zb.ROUTE_SOFTMAX_ALL_RENORM, shared=False, oai=False, n_layers=1)
    full = MoePrefill.build(torch, dd, small, 96, seed=13)
    dd.setWorkspace(full.workspace)
    full.record()
    ctx.submit_and_wait()
    part = MoePrefill.build(torch, dd, small, 96, seed=13, rank=rank, world=world, allreduce=allreduce)
    dd.setWorkspace(part.workspace)
    dist.barrier()
    part.record()
    ctx.submit_and_wait()
    err = float(((part.hidden.double() - full.hidden.double()).norm() / full.hidden.double().norm()).item())
    tt = torch.tensor([err], device="cuda", dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ep_check = float(tt.item())
    dd.setWorkspace(None)
    del full, part
    torch.cuda.empty_cache()
    if ep_check > 1e-4:
        raise SystemExit(f"expert-parallel prefill check failed: rel_l2 {ep_check:.3e}")

    S, T = QWEN35_MOE, args.tokens or 512
    copies = 4
    layers = [MoePrefill.build(torch, dd, S, T, seed=21 + c, rank=rank, world=world, allreduce=allreduce, local_only=True)
              for c in range(copies)]
    dd.setWorkspace(layers[0].workspace)   # same size for every copy
    launches = 0

    def run():
        nonlocal launches
        launches = sum(l.record() for l in layers) // copies

    run()
    stream.synchronize()
    g = graph_of(torch, stream, run)
    per, t0, t1 = timed_blocks(torch, stream, g.replay, 4, barrier=barrier, fixed_blocks=10)
    ms = statistics.median(per) / copies
    tt = torch.tensor([ms], device="cuda")
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms = float(tt.item())
    ids = layers[0].routing.view(T, 2 * S.top_k)[:, :S.top_k]
    touched = int(torch.unique(ids).numel())
    sg, sd = zb.expert_slice_bytes(S.t_gate_up, S.ffn, S.hidden), zb.expert_slice_bytes(S.t_down, S.hidden, S.ffn)
    wbytes = touched * (2 * sg + sd)
    flops = 2.0 * T * S.top_k * 3 * S.ffn * S.hidden
    tf = flops / (ms * 1e-3) / 1e12
    out = []
    if rank == 0:
        out.append({
            "metric": METRIC, "value": wbytes / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world, "steps": len(per) * copies,
            "warmup": 4, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"qwen3.5-35b-a3b-like MoE layer (256 experts top-8, Q4_K gate/up, Q6_K down), prefill T={T}, "
                                   "routed experts only", "path": "grouped",
                       "parallelism": f"ep{world}: whole experts per rank, tokens and routing replicated, one NCCL "
                                      "all-reduce of the [T][hidden] partial outputs per layer",
                       "experts_touched": touched, "weight_bytes_touched": wbytes, "tokens_per_s": T / (ms * 1e-3),
                       "tflops": tf, "l2": f"{copies} layers' expert weights in rotation"},
            "ep_check": {"rel_l2": ep_check, "ranks": world},
            "gpu_launches": launches * len(per) * copies, "gpu_launches_per_step": launches,
            "roofline": hbm_roofline(wbytes, ms * 1e3, peak * world, kind, tensor_frac_of_burst=tf / (peak_burst * world)),
            "clocks": sampler.window(t0, t1),
        })
    g.reset()
    dd.setWorkspace(None)
    return out


# ---- tensor-parallel correctness check (N > 1) -------------------------------------------------------------
def tp_check(torch, zb, dd, dist, rank, world, allreduce, allgather):
    """A small layer stack cut from the same seeded tensors on every rank, run through the exchange the
    timed step uses, against the unsharded step on the same GPU. Returns the worst relative L2 over the
    hidden vector and the logits, maximised over the ranks."""
    from zinc_b200.decode_step import DecodeStep, StepShape

    small = StepShape(hidden=2048, n_layers=2, q_dim=2048, kv_dim=2048, ffn=4096, vocab=8192)
    full = DecodeStep.build(torch, dd, small, rank=0, world=1, seed=77)
    part = DecodeStep.build(torch, dd, small, rank=rank, world=world, seed=77, allreduce=allreduce, allgather=allgather)
    gen = torch.Generator(device="cuda").manual_seed(4321)
    x = torch.randn(small.hidden, device="cuda", generator=gen)
    a = torch.randn(small.q_dim, device="cuda", generator=gen)
    f = torch.randn(small.ffn, device="cuda", generator=gen)
    nq, nf = small.q_dim // world, small.ffn // world
    full.x_norm.copy_(x), full.attn_out.copy_(a), full.ffn_act_in.copy_(f)
    part.x_norm.copy_(x), part.attn_out.copy_(a[rank * nq:(rank + 1) * nq]), part.ffn_act_in.copy_(f[rank * nf:(rank + 1) * nf])
    full.record()
    dist.barrier()
    part.record()
    dd.ctx.submit_and_wait()
    worst = 0.0
    for got, want in ((part.hidden, full.hidden), (part.logits, full.logits)):
        err = float(((got.double() - want.double()).norm() / want.double().norm()).item())
        worst = max(worst, err)
    tt = torch.tensor([worst], device="cuda", dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    del full, part
    torch.cuda.empty_cache()
    return float(tt.item())


def teardown_distributed(torch, dist, ctx, graphs=()):
    # A captured graph holds references on the communicator, and destroying the communicator waits for
    # them: release the graphs first. A timer ends the process if teardown still stalls (the result line
    # is already printed and flushed).
    killer = threading.Timer(30.0, lambda: os._exit(0))
    killer.daemon = True
    killer.start()
    torch.cuda.synchronize()
    for g in graphs:
        g.reset()
    dist.barrier()
    ctx.comm_destroy()
    torch.cuda.synchronize()
    dist.destroy_process_group()
    killer.cancel()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="zinc_b200", choices=["zinc_b200", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill_gemm", "dmmv_single", "moe_decode", "moe_prefill"],
                    help="decode: the headline decode step (at one GPU its line also carries the other workloads); "
                         "prefill_gemm: the batched-prefill dequant-GEMM cases; dmmv_single: one Q4_K 4096x4096 matvec; "
                         "moe_decode: the two MoE configurations at batch 1; moe_prefill: one MoE layer's routed experts "
                         "over a prefill batch")
    ap.add_argument("--moe-dispatch", default="fused", choices=["fused", "reference"],
                    help="moe_decode: fused = three launches per layer (default); reference = one launch per dispatch of "
                         "the reference's sequence")
    ap.add_argument("--collective", default="fused", choices=["fused", "peer", "nccl"],
                    help="N > 1, hidden-state sums: fused = partial rows pushed to every rank from the matvec's epilogue "
                         "and summed in the next matvec's prologue (default); peer = the library's one-kernel all-reduce; "
                         "nccl = NCCL all-reduce (the baseline)")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debug; invalidates the number)")
    ap.add_argument("--tokens", type=int, default=0, help="moe_prefill: override the prefill batch (default 512 / 1024)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="decode at one GPU: leave the `workloads` object out")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(cpu_reference_arm(args)), flush=True)
        return 0

    import torch

    import zinc_b200 as zb
    from zinc_b200.decode_step import DecodeStep, StepShape

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    if args.gpus != world and rank == 0 and world > 1:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)

    sampler = ClockSampler(local_rank).start() if rank == 0 else _NoSampler()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = zb.Context(local_rank, stream=stream.cuda_stream)
        dd = zb.DmmvDispatch(ctx)
        if world > 1:  # peer exchange of the library: IPC handles travel through the process group
            handles = [None] * world
            dist.all_gather_object(handles, ctx.comm_init(rank, world))
            ctx.comm_connect(handles)
            dist.barrier()

        if args.workload != "decode":
            if args.workload == "moe_decode":
                res = moe_decode_results(torch, zb, ctx, dd, stream, sampler, args, rank, world, dist)
            elif world > 1 and args.workload == "moe_prefill":
                res = moe_prefill_ep_results(torch, zb, ctx, dd, stream, sampler, args, rank, world, dist)
            elif world > 1:
                raise SystemExit(f"--workload {args.workload} runs on one GPU")
            elif args.workload == "prefill_gemm":
                res = prefill_gemm_results(torch, zb, ctx, dd, stream, sampler, False)
            elif args.workload == "dmmv_single":
                res = dmmv_single_results(torch, zb, dd, stream, sampler, False)
            else:
                res = moe_prefill_results(torch, zb, ctx, dd, stream, sampler, args)
            if rank == 0:
                for r in res:
                    print(json.dumps(r), flush=True)
            if isinstance(sampler, ClockSampler):
                sampler.stop()
            if dist is not None:
                teardown_distributed(torch, dist, ctx)
            return 0

        shape = StepShape() if not args.layers else StepShape(n_layers=args.layers)

        def allreduce(t):
            if args.collective == "nccl":
                dist.all_reduce(t)
            else:
                ctx.allreduce_sum(t, t.numel())

        def allgather(t, r, n):  # in place: rank r's slice is already there
            if args.collective == "nccl":
                dist.all_gather_into_tensor(t, t.narrow(0, r * n, n))
            else:
                ctx.allgather(t, t, n, src_offset=r * n * 4)

        def barrier():
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()

        if args.collective == "fused":
            allreduce = None
        check = None
        if world > 1:
            check = tp_check(torch, zb, dd, dist, rank, world, allreduce, allgather)
            if check > 1e-4:
                raise SystemExit(f"tensor-parallel check failed: relative L2 {check:.3e} over {world} ranks")

        step = DecodeStep.build(torch, dd, shape, rank=rank, world=world, allreduce=allreduce, allgather=allgather)
        gen = torch.Generator(device="cuda").manual_seed(1234)
        for buf in (step.x_norm, step.attn_out, step.ffn_act_in):
            buf.copy_(torch.randn(buf.shape, device="cuda", generator=gen))
        # pinned host staging for the end-to-end leg
        n_in = step.input_floats()
        h_in = torch.randn(n_in, generator=torch.Generator().manual_seed(7)).pin_memory()
        h_out = torch.empty(shape.vocab + shape.hidden, dtype=torch.float32).pin_memory()
        d_in = [step.x_norm, step.attn_out, step.ffn_act_in]

        # one eager token (also the warm-up of every kernel variant), then record the graph
        launches_per_step = step.record()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step.record()
        stream.synchronize()

        # ---- device-resident timing: blocks of --steps replays -------------------------------------
        for _ in range(args.warmup):
            graph.replay()
        per, t_wall0, t_wall1 = timed_blocks(torch, stream, graph.replay, args.steps, barrier=barrier,
                                             fixed_blocks=10 if world > 1 else 0)
        n_blocks = len(per)
        if dist is not None:  # slowest rank, block by block
            tt = torch.tensor(per, device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            per = [float(v) for v in tt.tolist()]
        ms_per_step = statistics.median(per)
        total_bytes = shape.weight_bytes()
        value = total_bytes / (ms_per_step * 1e-3) / 1e9
        clocks = sampler.window(t_wall0, t_wall1)

        # ---- end to end: host vectors in, logits out, per token ---------------------------------
        def e2e_token():
            off = 0
            for t in d_in:
                nb = t.numel() * 4
                ctx.upload_from_ptr(zb.Buffer.from_torch(t), h_in.data_ptr() + off, nb)
                off += nb
            graph.replay()
            ctx.download_to_ptr(h_out.data_ptr(), zb.Buffer.from_torch(step.logits), shape.vocab * 4)
            ctx.download_to_ptr(h_out.data_ptr() + shape.vocab * 4, zb.Buffer.from_torch(step.hidden),
                                shape.hidden * 4)
            ctx.submit_and_wait()

        for _ in range(3):
            e2e_token()
        e2e_steps = max(args.steps, 50)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_token()
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        if dist is not None:
            tt = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e_s = float(tt.item())
        e2e_val = total_bytes / e2e_s / 1e9

        # ---- dominant kernel alone: fused gate+up+SwiGLU (Q4_K), rotating over the layers ----------
        M, K = shape.ffn // world, shape.hidden
        kbytes = 2 * M * zb.row_bytes(shape.t_gate_up, K)

        def gate_up_pass():
            for lw in step.layers:
                dd.dispatchDmmvFusedGateUpSwiglu(shape.t_gate_up, lw.wgate, lw.wup, step.x_norm, step.act, M, K)

        kg = graph_of(torch, stream, gate_up_pass)
        kper, _, _ = timed_blocks(torch, stream, kg.replay, 3, min_total_s=0.1)
        k_us = statistics.median(kper) * 1e3 / len(step.layers)
        peak, _, _, peak_kind = measured_peaks()
        kernels = {"gate_up_q4k": {"us": k_us, "bytes": kbytes, "gbs": kbytes / k_us / 1e3, "frac": kbytes / k_us / 1e3 / peak}}

        # the step's other kernels, each alone over the layers' distinct weights (same method)
        def alone(name, nbytes, fn):
            g = graph_of(torch, stream, fn)
            p, _, _ = timed_blocks(torch, stream, g.replay, 3, min_total_s=0.05)
            us = statistics.median(p) * 1e3 / len(step.layers)
            kernels[name] = {"us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak}
            g.reset()

        s, g_ = shape, world
        alone("down_q6k", s.hidden * zb.row_bytes(s.t_down, s.ffn // g_), lambda: [
            dd.recordDispatch(s.t_down, lw.wdown, step.ffn_act_in, step.hidden, s.hidden, s.ffn // g_, acc_mode=1)
            for lw in step.layers])
        alone("qkv_q4k", (s.q_dim + 2 * s.kv_dim) // g_ * zb.row_bytes(s.t_attn, s.hidden), lambda: [
            dd.recordDispatchMulti(s.t_attn, [lw.wq, lw.wk, lw.wv], step.x_norm, [step.q, step.k, step.v],
                                   [s.q_dim // g_, s.kv_dim // g_, s.kv_dim // g_], s.hidden) for lw in step.layers])
        alone("o_q4k", s.hidden * zb.row_bytes(s.t_attn, s.q_dim // g_), lambda: [
            dd.recordDispatch(s.t_attn, lw.wo, step.attn_out, step.hidden, s.hidden, s.q_dim // g_, acc_mode=1)
            for lw in step.layers])
        kg.reset()

        cpu_base = None
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            cpu_base = cpu_baseline_leg(torch, step)

        # ---- the other workloads of the metric (one GPU) ---------------------------------------------
        extra = None
        if world == 1 and not args.no_extra and not args.layers:
            graph.reset()
            del graph, step, d_in
            torch.cuda.empty_cache()
            extra = {}
            for key, fn in (("dmmv_single", lambda: dmmv_single_results(torch, zb, dd, stream, sampler, True)),
                            ("prefill_gemm", lambda: prefill_gemm_results(torch, zb, ctx, dd, stream, sampler, True)),
                            ("moe_decode", lambda: moe_decode_results(torch, zb, ctx, dd, stream, sampler, args)),
                            ("moe_prefill", lambda: moe_prefill_results(torch, zb, ctx, dd, stream, sampler, args,
                                                                        per_pair=False))):
                try:
                    extra[key] = fn()
                except Exception as e:  # a failing side workload must not take the headline line with it
                    extra[key] = {"error": f"{type(e).__name__}: {e}"}
                torch.cuda.empty_cache()
            graph = None

    if isinstance(sampler, ClockSampler):
        sampler.stop()
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "best_ms_per_step": min(per), "timed_blocks": n_blocks,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": "qwen3-8b-shaped decode step, batch 1, Q4_K_M mix (Q4_K attn/gate/up, Q6_K down + LM head)",
                "layers": shape.n_layers, "hidden": shape.hidden, "ffn": shape.ffn, "vocab": shape.vocab,
                "weight_bytes_per_token": total_bytes,
                "parallelism": "single GPU" if world == 1 else f"tp{world} (rows: QKV/gate/up/head, K: O/down; hidden-state sums: {dict(fused='rows pushed to every rank from the matvec epilogue, summed in the next matvec prologue, over NVLink peer memory', peer='one-kernel peer all-reduce over NVLink', nccl='NCCL all-reduce')[args.collective]})",
                "l2": "inputs larger than L2: 4.88 GB of distinct weights per step, no flush needed",
                "launch": "CUDA graph replay of the recorded op sequence",
                "timing": f"{n_blocks} blocks of {args.steps} replays, CUDA events per block, median block reported",
            },
            "tok_s": 1e3 / ms_per_step,
            "frac_of_nominal_8tbs": value / NOMINAL_HBM_GBS,
            "frac_of_measured_hbm": value / (peak * world),
            "e2e": {"value": e2e_val, "unit": UNIT, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                    "h2d_bytes_per_step": n_in * 4, "d2h_bytes_per_step": (shape.vocab + shape.hidden) * 4},
            "gpu_launches": launches_per_step * args.steps * n_blocks,
            "gpu_launches_per_step": launches_per_step,
            "roofline": hbm_roofline(kbytes, k_us, peak, peak_kind,
                                     traffic=ncu_traffic(GATE_UP_KEY) if world == 1 and not args.layers else None,
                                     kernel="dmmv fused gate+up+SwiGLU (Q4_K), M=%d K=%d" % (M, K)),
            "roofline_step": {"bound": "hbm", "achieved": value, "peak": peak * world, "unit": "GB/s",
                              "frac": value / (peak * world)},
            "kernels_alone": kernels,
            "cpu_baseline": cpu_base,
            "clocks": clocks,
        }
        if check is not None:
            out["tp_check"] = {"rel_l2": check, "ranks": world, "bar": 1e-4}
        if extra is not None:
            out["workloads"] = extra
        print(json.dumps(out), flush=True)
    if dist is not None:
        teardown_distributed(torch, dist, ctx, [graph] if graph is not None else [])
    return 0


if __name__ == "__main__":
    sys.exit(main())
