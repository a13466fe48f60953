#!/usr/bin/env python
"""Benchmark of the quantized matmul hot path on B200.

Workload (N=1): the Qwen3-8B-shaped decode step at batch 1 - 36 layers of Q/K/V/O,
fused gate+up+SwiGLU and down projections plus the LM head, Q4_K_M mix (Q4_K attention
and gate/up, Q6_K down and LM head), random weights, N(0,1) f32 activations. Every
projection is one dequant-matvec through the C ABI; the step is recorded once into a
CUDA graph (zc_begin_record / zc_end_record) and replayed per token.

Metric: quantized weight bytes streamed per second (GB/s), whole job.
  value : weights, activations and outputs resident in HBM; CUDA events around K replays.
  e2e   : per token, the three activation vectors are copied from pinned host memory, the
          step runs, and the logits + hidden vector are copied back to pinned host memory,
          all through the C ABI; wall clock around K such tokens (device idle on both sides).
Each token streams 4.88 GB of distinct weights, far more than the 126 MB L2, so no cache
flush is needed between steps.

N>1 (torchrun): tensor parallel over the ranks (strong scaling): Q/K/V, gate/up and LM
head sharded by rows, O and down along K, NCCL all-reduce / all-gather over NVLink.

`--impl reference` times the CPU restatement of the reference's decode shaders (the
oracle's shader-order DMMV, all host threads) on one layer's seven projections per step.
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
sys.path.insert(0, ROOT)

METRIC = "dmmv_weight_gbs"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-3:]
        for _, line in inside:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_arm(args):
    """The reference's decode shaders restated on the CPU, timed on this host's cores."""
    import numpy as np

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
    threads = o.max_threads()

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
              f"{threads} OpenMP threads")
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
    threads = o.max_threads()
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


def _timed_graph(torch, stream, fn, reps):
    """Capture fn() once into a CUDA graph on `stream`, replay it `reps` times, return ms per replay."""
    fn()
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn()
    for _ in range(3):
        g.replay()
    stream.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(reps):
        g.replay()
    ev1.record(stream)
    stream.synchronize()
    return ev0.elapsed_time(ev1) / reps


def dmmv_single_bench(torch, zb, args, local_rank):
    """One Q4_K 4096 x 4096 matvec (9 437 184 weight bytes), 64 weight copies in rotation (604 MB > L2),
    and the same on one copy (L2-hot), labelled."""
    from zinc_b200 import synth

    peak, peak_kind = measured_peaks()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = zb.Context(local_rank, stream=stream.cuda_stream)
        dd = zb.DmmvDispatch(ctx)
        M = K = 4096
        copies = 64
        ws = [synth.torch_quant_matrix(zb.Q4_K, M, K, f"cuda:{local_rank}", 300 + i) for i in range(copies)]
        x = torch.randn(K, device="cuda")
        y = torch.zeros(M, device="cuda")
        wbytes = M * zb.row_bytes(zb.Q4_K, K)

        def rotating():
            for w in ws:
                dd.recordDispatch(zb.Q4_K, w, x, y, M, K)

        def hot():
            for _ in range(copies):
                dd.recordDispatch(zb.Q4_K, ws[0], x, y, M, K)

        reps = max(5, min(args.steps, 50))
        for label, fn in (("64 weight copies in rotation (604 MB, larger than L2)", rotating),
                          ("one weight copy, L2-hot", hot)):
            us = _timed_graph(torch, stream, fn, reps) * 1e3 / copies
            gbs = wbytes / us / 1e3
            print(json.dumps({
                "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": 1, "steps": reps * copies, "warmup": 3 * copies,
                "ms_per_step": us / 1e3, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "single Q4_K matvec 4096x4096, f32 x", "l2": label,
                           "weight_bytes": wbytes, "reference_bytes_model": wbytes + 4 * K + 4 * M},
                "gpu_launches": reps * copies,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                             "frac": gbs / peak, "traffic": None},
            }), flush=True)
    return 0


def moe_decode_bench(torch, zb, args, local_rank, rank=0, world=1, dist=None):
    """One token through the MoE layers of the two MoE configurations at batch 1. With N ranks the FFN
    dimension of every expert is cut tensor-parallel (rows of gate / up, K slice of down) and the partial
    hidden vectors are summed with the library's peer all-reduce once per layer; a configuration whose
    down projection has fewer blocks than ranks is skipped and said so."""
    import threading

    from zinc_b200.moe_step import GPT_OSS_MOE, QWEN35_MOE, MoeDecode

    peak, peak_kind = measured_peaks()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = zb.Context(local_rank, stream=stream.cuda_stream)
        dd = zb.DmmvDispatch(ctx)
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, ctx.comm_init(rank, world))
            ctx.comm_connect(handles)
            dist.barrier()

        def allreduce(t):
            ctx.allreduce_sum(t, t.numel())

        def barrier():
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()

        for name, shape in (("qwen3.5-35b-a3b-like MoE layers (256 experts top-8 + shared, Q4_K / Q6_K)", QWEN35_MOE),
                            ("gpt-oss-20b-shaped MoE layers (32 experts top-4, MXFP4)", GPT_OSS_MOE)):
            if args.layers:
                import dataclasses

                shape = dataclasses.replace(shape, n_layers=args.layers)
            try:
                step = MoeDecode.build(torch, dd, shape, rank=rank, world=world,
                                       allreduce=allreduce if world > 1 else None)
            except ValueError as e:
                if rank == 0:
                    print(json.dumps({"metric": METRIC, "n_gpus": world, "config": {"workload": name + ", decode batch 1"},
                                      "skipped": f"tensor-parallel cut not possible: {e}"}), flush=True)
                continue
            launches = step.record()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step.record()
            reps = max(20, min(args.steps, 200))
            for _ in range(4):
                graph.replay()
            barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(stream)
            for _ in range(reps):
                graph.replay()
            ev1.record(stream)
            barrier()
            ms = ev0.elapsed_time(ev1) / reps
            if dist is not None:
                tt = torch.tensor([ms], device="cuda")
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                ms = float(tt.item())
            gbs = shape.weight_bytes() / (ms * 1e-3) / 1e9
            if rank == 0:
                print(json.dumps({
                    "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": world, "steps": reps, "warmup": 4,
                    "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "dtype": "f32",
                    "data": "synthetic",
                    "config": {"workload": name + ", decode batch 1", "layers": shape.n_layers,
                               "weight_bytes_per_token": shape.weight_bytes(),
                               "parallelism": "single GPU" if world == 1 else
                               f"tp{world}: expert FFN dimension cut over the ranks, one peer all-reduce per layer",
                               "l2": "weights touched per token (all layers) are larger than L2"},
                    "gpu_launches": launches * reps, "gpu_launches_per_step": launches,
                    "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak * world, "peak_kind": peak_kind,
                                 "unit": "GB/s", "frac": gbs / (peak * world), "traffic": None},
                }), flush=True)
            graph.reset()
            del graph, step
            torch.cuda.empty_cache()
        if dist is not None:
            killer = threading.Timer(30.0, lambda: os._exit(0))
            killer.daemon = True
            killer.start()
            barrier()
            ctx.comm_destroy()
            torch.cuda.synchronize()
            dist.destroy_process_group()
            killer.cancel()
    return 0


def moe_prefill_bench(torch, zb, args, local_rank):
    """The routed-expert matmuls of one MoE layer over a prefill batch: gate and up (one activation row per
    token, n_used experts each), SwiGLU, down (one row per (token, slot) pair) and the weighted scatter
    back to the tokens. Routing ids come from softmax_topk over N(0,1) logits, before the timed region.
    One JSON line per configuration and path: grouped by expert on the tensor cores (Q4_K / Q6_K, with a
    workspace) and the per-pair kernel the reference's Vulkan path uses."""
    from zinc_b200 import synth
    from zinc_b200.moe_step import GPT_OSS_MOE, QWEN35_MOE

    peak, peak_kind = measured_peaks()
    stream = torch.cuda.Stream()
    dev = f"cuda:{local_rank}"
    with torch.cuda.stream(stream):
        ctx = zb.Context(local_rank, stream=stream.cuda_stream)
        dd = zb.DmmvDispatch(ctx)
        for name, S, T in (("qwen3.5-35b-a3b-like MoE layer (256 experts top-8, Q4_K gate/up, Q6_K down)", QWEN35_MOE, 512),
                           ("gpt-oss-20b-shaped MoE layer (32 experts top-4, MXFP4)", GPT_OSS_MOE, 1024)):
            T = args.tokens or T
            E, k, H, F = S.n_experts, S.top_k, S.hidden, S.ffn
            Wg = synth.torch_quant_matrix(S.t_gate_up, E * F, H, dev, 11)
            Wu = synth.torch_quant_matrix(S.t_gate_up, E * F, H, dev, 12)
            Wd = synth.torch_quant_matrix(S.t_down, E * H, F, dev, 13)
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

            def layer():
                dd.recordMoeBatchedDispatchPair(S.t_gate_up, Wg, Wu, X, gate, up, ids, F, H, sg, E, k, T, H, k * F)
                dd.dispatchSwiglu(gate, up, act, T * k * F, oai=S.oai)
                dd.recordMoeBatchedDispatch(S.t_down, Wd, act, down, ids, H, F, sd, E, 1, T * k, F, H)
                dd.dispatchMoeRouteScatter(routing, down, hidden, T, H, k, 2 * k)

            ws = torch.empty(max(dd.moeGroupedWorkspaceBytes(T, k, H, E), dd.moeGroupedWorkspaceBytes(T * k, 1, F, E)),
                             dtype=torch.uint8, device=dev)
            for path in ("grouped", "per_pair"):
                dd.setWorkspace(ws if path == "grouped" else None)
                n0 = ctx.launch_count
                layer()
                launches = ctx.launch_count - n0
                reps = max(5, min(args.steps, 50 if path == "grouped" else 5))
                ms = _timed_graph(torch, stream, layer, reps)
                gbs = wbytes / (ms * 1e-3) / 1e9
                print(json.dumps({
                    "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": 1, "steps": reps, "warmup": 4,
                    "ms_per_step": ms, "higher_is_better": True,
                    "dtype": "bf16" if path == "grouped" and launches > 5 else "f32", "data": "synthetic",
                    "config": {"workload": f"{name}, prefill T={T}, routed experts only", "path": path,
                               "experts_touched": touched, "weight_bytes_touched": wbytes,
                               "tokens_per_s": T / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
                               "l2": "expert weights of the layer are larger than L2"},
                    "gpu_launches": launches * reps, "gpu_launches_per_step": launches,
                    "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": peak_kind,
                                 "unit": "GB/s", "frac": gbs / peak, "traffic": None},
                }), flush=True)
            dd.setWorkspace(None)
            del Wg, Wu, Wd, ws
            torch.cuda.empty_cache()
    return 0


def prefill_gemm_bench(torch, zb, args, local_rank):
    """Batched-prefill dequant-GEMM D[T][M] = X[T][K] W[M][K]^T (bf16 activations, f32 out), one JSON
    line per case: gate-shaped Q4_K 12288 x 4096, down-shaped Q6_K 4096 x 12288 and a GPT-OSS gate+up-shaped
    MXFP4 5760 x 2880 at T = 128, 512, 2048. Each timed launch uses the next of 8 weight copies (more than L2 in total)."""
    from zinc_b200 import synth

    peak_burst = peak_sust = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        peak_burst, peak_sust = float(p["bf16_tflops"]), float(p["bf16_tflops_sustained"])
    except Exception:
        peak_burst, peak_sust = 1590.0, 1400.0
    ctx = zb.Context(local_rank, stream=torch.cuda.current_stream().cuda_stream)
    dd = zb.DmmvDispatch(ctx)
    dev = f"cuda:{local_rank}"
    copies = 8
    for qt, name, M, K in ((zb.Q4_K, "q4_k", 12288, 4096), (zb.Q6_K, "q6_k", 4096, 12288),
                           (zb.MXFP4, "mxfp4", 5760, 2880)):
        ws = [synth.torch_quant_matrix(qt, M, K, dev, 100 + i) for i in range(copies)]
        for T in (128, 512, 2048):
            X = torch.randn(T, K, device=dev).to(torch.bfloat16)
            D = torch.zeros(T * M, dtype=torch.float32, device=dev)
            n0 = ctx.launch_count
            for i in range(max(args.warmup, 3)):
                dd.recordMulMm(qt, ws[i % copies], X, D, M, T, K, K, M, 0, 0, 0, zb.BF16)
            per_call = (ctx.launch_count - n0) // max(args.warmup, 3)
            reps = max(20, min(args.steps, 200))
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for i in range(reps):
                dd.recordMulMm(qt, ws[i % copies], X, D, M, T, K, K, M, 0, 0, 0, zb.BF16)
            ev1.record()
            ctx.submit_and_wait()
            us = ev0.elapsed_time(ev1) * 1e3 / reps
            tf = 2.0 * M * K * T / us / 1e6
            print(json.dumps({
                "metric": "prefill_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": reps,
                "warmup": max(args.warmup, 3), "ms_per_step": us / 1e3, "higher_is_better": True, "dtype": "bf16",
                "data": "synthetic",
                "config": {"workload": f"prefill dequant-GEMM {name} {M}x{K}, T={T}, bf16 activations, f32 out",
                           "l2": f"{copies} weight copies in rotation ({copies * ws[0].numel() / 1e6:.0f} MB)"},
                "gpu_launches": per_call * reps,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": peak_burst, "unit": "TFLOP/s",
                             "frac": tf / peak_burst, "frac_of_sustained": tf / peak_sust, "traffic": None},
            }), flush=True)
        del ws
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="zinc_b200", choices=["zinc_b200", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill_gemm", "dmmv_single", "moe_decode", "moe_prefill"],
                    help="decode: the headline decode step; prefill_gemm: the batched-prefill dequant-GEMM cases; "
                         "dmmv_single: one Q4_K 4096x4096 matvec; moe_decode: the two MoE layers at batch 1; "
                         "moe_prefill: one MoE layer's routed experts over a prefill batch")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: the library's one-shot peer all-reduce (default) or NCCL for the hidden-state sums")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debug; invalidates the number)")
    ap.add_argument("--tokens", type=int, default=0, help="moe_prefill: override the prefill batch (default 512 / 1024)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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

    if args.workload == "prefill_gemm":
        return prefill_gemm_bench(torch, zb, args, local_rank)
    if args.workload == "dmmv_single":
        return dmmv_single_bench(torch, zb, args, local_rank)
    if args.workload == "moe_prefill":
        return moe_prefill_bench(torch, zb, args, local_rank)
    if args.workload == "moe_decode":
        return moe_decode_bench(torch, zb, args, local_rank, rank, world, dist)

    stream = torch.cuda.Stream()
    shape = StepShape() if not args.layers else StepShape(n_layers=args.layers)
    with torch.cuda.stream(stream):
        ctx = zb.Context(local_rank, stream=stream.cuda_stream)
        dd = zb.DmmvDispatch(ctx)

        if world > 1:  # peer exchange of the library: IPC handles travel through the process group
            handles = [None] * world
            dist.all_gather_object(handles, ctx.comm_init(rank, world))
            ctx.comm_connect(handles)
            dist.barrier()

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

        def barrier():
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()

        # ---- device-resident timing -------------------------------------------------------
        for _ in range(args.warmup):
            graph.replay()
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
            time.sleep(0.25)
        barrier()  # every rank enters the timed region together (a rank that starts early waits in its collectives)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_wall0 = time.time()
        ev0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        ev1.record(stream)
        barrier()
        t_wall1 = time.time()
        dev_ms = ev0.elapsed_time(ev1)
        if dist is not None:
            tt = torch.tensor([dev_ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dev_ms = float(tt.item())
        ms_per_step = dev_ms / args.steps
        total_bytes = shape.weight_bytes()
        value = total_bytes / (ms_per_step * 1e-3) / 1e9

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
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_token()
        barrier()
        e2e_s = (time.perf_counter() - t0) / args.steps
        if dist is not None:
            tt = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e_s = float(tt.item())
        e2e_val = total_bytes / e2e_s / 1e9
        clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None

        # ---- dominant kernel alone: fused gate+up+SwiGLU (Q4_K), rotating over the layers ----------
        M, K = shape.ffn // world, shape.hidden
        kbytes = 2 * M * zb.row_bytes(shape.t_gate_up, K)
        reps = 3

        def gate_up_pass():
            for lw in step.layers:
                dd.dispatchDmmvFusedGateUpSwiglu(shape.t_gate_up, lw.wgate, lw.wup, step.x_norm, step.act, M, K)

        gate_up_pass()
        kg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kg, stream=stream):
            gate_up_pass()
        kg.replay()
        stream.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(stream)
        for _ in range(reps):
            kg.replay()
        k1.record(stream)
        stream.synchronize()
        k_us = k0.elapsed_time(k1) * 1e3 / (reps * len(step.layers))
        peak, peak_kind = measured_peaks()
        achieved = kbytes / (k_us * 1e-6) / 1e9

        cpu_base = None
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            cpu_base = cpu_baseline_leg(torch, step)

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": "qwen3-8b-shaped decode step, batch 1, Q4_K_M mix (Q4_K attn/gate/up, Q6_K down + LM head)",
                "layers": shape.n_layers, "hidden": shape.hidden, "ffn": shape.ffn, "vocab": shape.vocab,
                "weight_bytes_per_token": total_bytes,
                "parallelism": "single GPU" if world == 1 else f"tp{world} (rows: QKV/gate/up/head, K: O/down; collectives: {'one-shot peer all-reduce / all-gather kernels' if args.collective == 'peer' else 'NCCL'})",
                "l2": "inputs larger than L2: 4.88 GB of distinct weights per step, no flush needed",
                "launch": "CUDA graph replay of the recorded op sequence",
            },
            "tok_s": 1e3 / ms_per_step,
            "frac_of_nominal_8tbs": value / NOMINAL_HBM_GBS,
            "frac_of_measured_hbm": value / peak,
            "e2e": {"value": e2e_val, "unit": UNIT, "ms_per_step": e2e_s * 1e3,
                    "h2d_bytes_per_step": n_in * 4, "d2h_bytes_per_step": (shape.vocab + shape.hidden) * 4},
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_per_step": launches_per_step,
            "roofline": {"bound": "hbm", "kernel": "dmmv fused gate+up+SwiGLU (Q4_K), M=%d K=%d" % (M, K),
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "us_per_launch": k_us, "algorithmic_bytes_per_launch": kbytes,
                         "traffic": ncu_traffic("dmmv_gate_up_q4k_12288x4096")},
            "roofline_step": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s",
                              "frac": value / peak},
            "cpu_baseline": cpu_base,
            "clocks": clocks,
        }
        print(json.dumps(out), flush=True)
    if dist is not None:
        # A captured graph holds references on the NCCL communicator, and destroying the communicator
        # waits for them: release the graph first. A timer ends the process if teardown still stalls
        # (the result line is already printed and flushed).
        import threading

        killer = threading.Timer(30.0, lambda: os._exit(0))
        killer.daemon = True
        killer.start()
        torch.cuda.synchronize()
        graph.reset()
        del graph
        dist.barrier()
        ctx.comm_destroy()
        torch.cuda.synchronize()
        dist.destroy_process_group()
        killer.cancel()
    return 0


if __name__ == "__main__":
    sys.exit(main())
