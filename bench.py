#!/usr/bin/env python
"""Headline benchmark: decode (and prefill) tokens/s of a Q4_K_M Qwen2.5-32B-shaped decoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload cfg2|cfg1|cfg3]

A step is one decode pass (one new token for every in-flight sequence) at context >= 2048.
With N GPUs (one process per GPU under torch.distributed.run) the model is split into N
contiguous layer ranges, one per rank, and N sequences are kept in flight so that every stage has
work in every step (the per-GPU work per step is fixed: "weak" scaling).

Prints ONE JSON line (rank 0).  Weights are synthetic: seeded N(0, 0.02) quantised on the device
to the Q4_K_M mix; tokens are seeded uniform ids.
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
sys.path.insert(0, ROOT)

WORKLOADS = {
    # the dense configurations of the benchmark list: 3B, 32B and 70B shapes
    "cfg1": dict(name="Qwen2.5-3B-shape Q4_K_M", n_layer=36, n_embd=2048, n_head=16, n_head_kv=2,
                 head_dim=128, n_ff=11008, n_vocab=151936, qkv_bias=1, rope_neox=1, rope_theta=1e6,
                 rms_eps=1e-6, prefill=512, decode=128),
    "cfg2": dict(name="Qwen2.5-32B-shape Q4_K_M", n_layer=64, n_embd=5120, n_head=40, n_head_kv=8,
                 head_dim=128, n_ff=27648, n_vocab=152064, qkv_bias=1, rope_neox=1, rope_theta=1e6,
                 rms_eps=1e-6, prefill=2048, decode=256),
    "cfg3": dict(name="Llama-3-70B-shape Q4_K_M", n_layer=80, n_embd=8192, n_head=64, n_head_kv=8,
                 head_dim=128, n_ff=28672, n_vocab=128256, qkv_bias=0, rope_neox=0, rope_theta=5e5,
                 rms_eps=1e-5, prefill=4096, decode=256),
    # the mixture-of-experts configuration; with N GPUs each rank is an independent replica holding n_expert / N experts
    "cfg4": dict(name="Qwen3-30B-A3B-shape MoE Q4_K_M", n_layer=48, n_embd=2048, n_head=32, n_head_kv=4,
                 head_dim=128, n_ff=0, n_vocab=151936, qkv_bias=0, rope_neox=1, rope_theta=1e6,
                 rms_eps=1e-6, n_expert=128, n_expert_used=8, n_ff_exp=768, prefill=1024, decode=256),
}
MODEL_KEYS = ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab", "qkv_bias",
              "rope_neox", "rope_theta", "rms_eps", "n_expert", "n_expert_used", "n_ff_exp")
BPW = {12: 144 / 256, 14: 210 / 256}
METRIC = "decode tok/s, Q4_K_M, batch 1 per stage (shape in config.workload; GEMV HBM % of peak in roofline)"


NCU_TRAFFIC_RATIO = 1.03  # DRAM bytes / algorithmic bytes of the decode GEMV, from ncu captures of isolated launches


def matmuls(w, layer):
    """(N, K, ggml type) of every quantised matmul of one layer, Q4_K_M mix"""
    h, nq, nkv, ff = w["n_embd"], w["n_head"] * w["head_dim"], w["n_head_kv"] * w["head_dim"], w["n_ff"]
    alt = 14 if layer & 1 else 12
    attn = [(nq, h, 12), (nkv, h, 12), (nkv, h, alt), (h, nq, 12)]
    if w.get("n_expert", 0):  # the experts one token activates
        fe = w["n_ff_exp"]
        return attn + w["n_expert_used"] * [(fe, h, 12), (fe, h, 12), (h, fe, alt)]
    return attn + [(ff, h, 12), (ff, h, 12), (h, ff, alt)]


def gemv_bytes(N, K, ty, M=1):
    return N * K * BPW[ty] + 4 * M * K + 4 * M * N


def step_gemv_bytes(w, l0, l1, has_output, M=1):
    b = sum(gemv_bytes(N, K, ty, M) for l in range(l0, l1) for (N, K, ty) in matmuls(w, l))
    if has_output:
        b += gemv_bytes(w["n_vocab"], w["n_embd"], 14, M)
    return b


class ClockSampler:
    """samples nvidia-smi clocks and throttle reasons while the timed region runs"""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc:
            self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ts, line in self.rows:
            if ts < t0 - 0.05 or ts > t1 + 0.15:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


_CPU_OPERANDS = {}


# ------------------------------------------------------------------------------------------------
def host_threads():
    """threads the CPU legs may really use: the cores this process is allowed on, cut to the container's CPU
    quota when there is one (more OpenMP threads than that only fight each other)"""
    n = os.cpu_count() or 1
    try:
        n = min(n, len(os.sched_getaffinity(0)))
    except Exception:
        pass
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()[:2]
        if quota != "max":
            n = min(n, max(1, int(int(quota) / int(period))))
    except Exception:
        pass
    return max(1, n)


def cpu_decode_sample(w, threads=None, reps=2):
    """times the CPU oracle on one layer of each parity (+ the LM head) at M = 1 and extrapolates
    to the full depth.  Returns (tok/s, cores, description)."""
    from oracle import binding as orc

    # all host cores, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its workers)
    orc.lib().orc_set_threads(threads or host_threads())
    cores = orc.lib().orc_get_threads()
    shapes = {}
    for layer in (0, 1):
        for (N, K, ty) in matmuls(w, layer):
            shapes[(N, K, ty)] = shapes.get((N, K, ty), 0) + w["n_layer"] / 2
    shapes[(w["n_vocab"], w["n_embd"], 14)] = 1
    total = 0.0
    for (N, K, ty), count in shapes.items():
        if (N, K, ty) not in _CPU_OPERANDS:  # random valid block bytes, made once per process
            rng = np.random.default_rng(N * 31 + K * 7 + ty)
            W = rng.integers(0, 256, size=(N, orc.row_bytes(ty, K)), dtype=np.uint8)
            x = rng.standard_normal((1, K)).astype(np.float32)
            orc.mul_mat(ty, W, x, N, K)
            _CPU_OPERANDS[(N, K, ty)] = (W, x)
        W, x = _CPU_OPERANDS[(N, K, ty)]
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.mul_mat(ty, W, x, N, K)
        total += count * (time.perf_counter() - t0) / reps
    return 1.0 / total, cores, (f"EXTRAPOLATED: CPU oracle, M=1 quantised matmuls of one even + one odd layer and the LM head "
                                f"({len(shapes)} shapes x {reps} reps, random block bytes as weights), times scaled to "
                                f"{w['n_layer']} layers; attention, norms and the argmax are not included (the figure "
                                f"favours the CPU); a CPU run timed in full is under cfg1_gpu_vs_cpu")


def run_reference(args, w):
    """--impl reference: the reference's llama.cpp CPU backend cannot be built here (sources are
    fetched at build time and are not in the tree), so the CPU port of the same arithmetic runs on
    the host cores.  A step is one bounded sample of the decode workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, wall = [], []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        toks, cores, sample = cpu_decode_sample(w, reps=1)
        if i >= args.warmup:
            vals.append(toks)
            wall.append(time.perf_counter() - t0)
    v = float(np.mean(vals))
    # value: tokens/s of a whole decode step, extrapolated from the sample (see cpu_baseline.sample);
    # ms_per_step: what one step of this arm (one sample) really took on the clock
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.mean(wall)), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int4/6 -> int32, f32 combine",
        "data": "synthetic", "config": {"workload": w["name"] + " decode, batch 1, CPU sample"},
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def micro_one(N, K, M, tname, iters):
    """One quantised matmul shape, timed with CUDA events over `iters` launches captured in a CUDA
    graph that rotates over enough weight copies to exceed L2."""
    import torch
    from mesh_llm_b200 import ops

    ty = {"q4_k": 12, "q6_k": 14}[tname.lower()]
    rb = ops.device_row_bytes(ty, K)
    copies = max(2, int(400e6 // (N * rb)) + 1)
    g = torch.Generator(device="cuda").manual_seed(1)
    Ws = [torch.randint(0, 256, (N, rb), dtype=torch.uint8, device="cuda", generator=g) for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", generator=g)
    q, d, bs = ops.quantize_act(x)
    y = torch.empty(M, N, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for W in Ws:
            ops.mul_mat_q8(ty, W, q, d, bs, N, K, out=y)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for i in range(iters):
                ops.mul_mat_q8(ty, Ws[i % copies], q, d, bs, N, K, out=y)
        graph.replay()
        torch.cuda.synchronize()
        best = 1e30
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / iters)
    sec = best * 1e-3
    out = {"micro": f"{N},{K},{M},{tname}", "us_per_launch": best * 1e3, "weight_copies": copies}
    if M <= 8:
        out["algorithmic_bytes"] = gemv_bytes(N, K, ty, M)
        out["GBps"] = out["algorithmic_bytes"] / sec / 1e9
    else:
        out["TOPps"] = 2.0 * M * N * K / sec / 1e12
    del Ws, x, q, d, bs, y, graph
    torch.cuda.empty_cache()
    return out


def run_micro(args):
    """--micro N,K,M,type: one shape of the isolated quantised-matmul sweep; also the command the committed
    ncu captures were taken with."""
    N, K, M, tname = args.micro.split(",")
    print(json.dumps(micro_one(int(N), int(K), int(M), tname, args.micro_iters)))


def run_micro_attn(args):
    """--micro-attn n_head,n_kv,pos0,T: the prefill attention kernel alone (f16 cache, head_dim 128), timed
    with CUDA events; TFLOP/s counts 4 * head_dim flops per (query, visible key, head).  Also the command
    the committed ncu capture of that kernel was taken with."""
    import torch
    from mesh_llm_b200 import ops

    nh, nkv, pos0, T = (int(v) for v in args.micro_attn.split(","))
    hd = 128
    g = torch.Generator(device="cuda").manual_seed(2)
    kc = torch.randn(pos0 + T, nkv, hd, device="cuda", generator=g).half()
    vc = torch.randn(pos0 + T, nkv, hd, device="cuda", generator=g).half()
    q = torch.randn(T, nh, hd, device="cuda", generator=g)
    for _ in range(3):
        ops.attention(q, kc, vc, pos0)
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.micro_iters):
            ops.attention(q, kc, vc, pos0)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / args.micro_iters)
    pairs = T * pos0 + T * (T + 1) // 2
    print(json.dumps({"micro_attn": args.micro_attn, "us_per_launch": best * 1e3,
                      "TFLOPps": 4.0 * hd * nh * pairs / (best * 1e-3) / 1e12}))


SWEEP_SHAPES = ((5120, 27648), (27648, 5120), (8192, 28672), (28672, 8192), (151936, 2048))
SWEEP_M = (1, 8, 64, 512, 4096)


def run_sweep(args):
    """--sweep: the isolated quantised-matmul sweep of the benchmark list: every shape x
    {Q4_K, Q6_K} x M; GB/s of algorithmic bytes for M <= 8, useful int8 TOP/s above; one JSON line each."""
    for tname in ("q4_k", "q6_k"):
        for (N, K) in SWEEP_SHAPES:
            for M in SWEEP_M:
                print(json.dumps(micro_one(N, K, M, tname, max(4, args.micro_iters // (1 + M // 64)))), flush=True)


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--layers", type=int, default=0, help="debug: truncate the model depth")
    ap.add_argument("--micro", default="", help="isolated quantised matmul instead of the model: 'N,K,M,type' "
                    "(type q4_k|q6_k); prints one line with us per launch and GB/s (M<=8) or TOP/s")
    ap.add_argument("--micro-iters", type=int, default=20)
    ap.add_argument("--micro-attn", default="", help="the prefill attention kernel alone: 'n_head,n_kv,pos0,T'")
    ap.add_argument("--balance", action="store_true", help="N > 1: split layers by weight bytes (the last stage, which "
                    "holds the output head, gets fewer layers) instead of equal layer counts")
    ap.add_argument("--handoff", default="peer", choices=["peer", "nccl"], help="N > 1: how a decode activation reaches the "
                    "next stage: the library's peer-memory kernels, or torch.distributed send/recv")
    ap.add_argument("--handoff-latency", action="store_true", help="N = 2: round trips of one [1 x n_embd] f32 row between "
                    "the two GPUs, peer-memory hand-off against send/recv; one line with the one-way latencies")
    ap.add_argument("--kv", default="f16", choices=["f16", "q8_0-q4_0", "q4_0-q4_0", "auto"],
                    help="KV-cache row types (K-V); auto = the pair mesh-llm starts a model of this size with")
    ap.add_argument("--seqs-per-stage", type=int, default=2, help="N > 1: sequences in flight per stage (every stage still "
                    "works on one sequence per tick at batch 1; with 1 the token's way back from the last stage to the "
                    "first is on every tick's critical path, with 2 it is hidden)")
    ap.add_argument("--no-extras", action="store_true", help="N = 1: skip the cfg3 / cfg4 / cfg1-against-CPU measurements "
                    "that follow the headline workload in the same run")
    ap.add_argument("--sweep", action="store_true", help="the isolated matmul sweep: all shapes x types x M")
    args = ap.parse_args()
    if args.micro:
        return run_micro(args)
    if args.micro_attn:
        return run_micro_attn(args)
    if args.sweep:
        return run_sweep(args)
    w = dict(WORKLOADS[args.workload])
    if args.layers:
        w["n_layer"] = args.layers
    if args.impl == "reference":
        return run_reference(args, w)
    if max(args.warmup, 0) < 3:
        args.warmup = 3

    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
        args.gpus = world
    if world > 1:
        from mesh_llm_b200 import pipeline
        if args.handoff_latency:
            return pipeline.bench_handoff_latency(args, w, rank, world, local)
        if w.get("n_expert", 0):
            return pipeline.bench_expert_replicas(args, w, METRIC, rank, world, local)
        return pipeline.bench_pipeline(args, w, METRIC, rank, world, local)

    torch.cuda.set_device(local)
    r = bench_single(args, w, local, full=True)
    out = {
        "metric": METRIC, "value": r["value"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int4/6 -> int32, f32 combine", "data": "synthetic",
        "config": {"workload": f"{w['name']} ({w['n_layer']} layers), decode batch 1 at context {w['prefill']}+, "
                               f"greedy, one stage on one GPU", "weight_bytes": r["weight_bytes"],
                   "l2": "each step streams all weights (>> 126 MB L2), no flush needed",
                   "sequences_in_flight": 1, "kv_cache": r["kv_cache"]},
        "e2e": {"value": r["e2e_value"], "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
        "gpu_launches": r["gpu_launches"], "clocks": r["clocks"], "roofline": r["roofline"], "cpu_baseline": None,
        "prefill_tok_s": r["prefill_tok_s"], "prefill_ubatch2048_tok_s": r["prefill_ub2048_tok_s"],
        "decode_batch8_tok_s": r["decode_batch8_tok_s"], "single_sequence_tok_s": r["value"],
        "decode_weight_stream_frac_of_hbm_peak": r["weight_stream_frac"],
    }
    if not args.no_cpu:
        v, cores, sample = cpu_decode_sample(w)
        out["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample}
    if not args.no_extras and args.workload == "cfg2" and not args.layers:
        out["prefill_gemm_roofline"] = prefill_gemm_roofline()
        # the other configurations of the benchmark list, in the same run on the same GPU
        k = max(8, min(args.steps, 24))
        r3 = bench_single(args, dict(WORKLOADS["cfg3"]), local, full=False, steps=k)
        out.update({"cfg3_decode_tok_s": r3["value"], "cfg3_e2e_tok_s": r3["e2e_value"],
                    "cfg3_single_sequence_tok_s": r3["value"], "cfg3_prefill_tok_s": r3["prefill_tok_s"],
                    "cfg3_prefill_ubatch2048_tok_s": r3["prefill_ub2048_tok_s"],
                    "cfg3_gemv_frac_of_hbm_peak": r3["roofline"]["frac"], "cfg3_workload": r3["workload"]})
        r4 = bench_single(args, dict(WORKLOADS["cfg4"]), local, full=False, steps=k)
        out.update({"cfg4_decode_tok_s": r4["value"], "cfg4_e2e_tok_s": r4["e2e_value"],
                    "cfg4_prefill_tok_s": r4["prefill_tok_s"], "cfg4_prefill_ubatch2048_tok_s": r4["prefill_ub2048_tok_s"],
                    "cfg4_decode_batch8_tok_s": r4["decode_batch8_tok_s"],
                    "cfg4_active_bytes_frac_of_hbm_peak": r4["weight_stream_frac_active"], "cfg4_workload": r4["workload"]})
        if not args.no_cpu:
            out["cfg1_gpu_vs_cpu"] = cfg1_timed_cpu_leg(local)
    print(json.dumps(out))


def bench_single(args, w, local, full=True, steps=None):
    """One workload on one GPU: prefill in ubatches of 512, device-resident greedy decode, end-to-end decode
    through pinned host memory, the GEMV-only / attention-only replays, batch-8 decode.  full = False skips
    the clock sampler and runs fewer steps (the extra configurations of a run)."""
    import ctypes as C

    import torch

    from mesh_llm_b200 import ops
    from mesh_llm_b200.capi import check, lib
    from mesh_llm_b200.stage import Stage

    steps = steps or args.steps
    warmup = args.warmup if full else 3
    model = {k: w[k] for k in MODEL_KEYS if k in w}
    n_ctx = w["prefill"] + w["decode"] + steps + warmup + 64
    n_seq = 8
    ids, names = {"f16": 1, "q4_0": 2, "q8_0": 8}, {1: "f16", 2: "q4_0", 8: "q8_0"}
    kt, vt = (1, 1) if args.kv == "auto" else [ids[t] for t in (args.kv + "-" + args.kv).split("-")[:2]]
    UB = 2048  # largest micro-batch the stage is sized for (the reference uses 512, and 2048 for vision models)
    st = Stage(**model, n_ctx=n_ctx, n_seq=n_seq, n_ubatch=UB, device=local, kv_type_k=kt, kv_type_v=vt)
    weight_bytes = st.weight_bytes()
    if args.kv == "auto" and ops.kv_types_for_model_bytes(weight_bytes) != (kt, vt):
        # the pair mesh-llm starts a model file of this size with
        kt, vt = ops.kv_types_for_model_bytes(weight_bytes)
        st.close()
        st = Stage(**model, n_ctx=n_ctx, n_seq=n_seq, n_ubatch=UB, device=local, kv_type_k=kt, kv_type_v=vt)
    st.generate(20251125)
    kv_label = names[kt] + "-" + names[vt]
    dev = torch.device("cuda", local)
    rng = np.random.default_rng(1234)

    # ---- prefill: prompt of `prefill` uniform-random tokens in ubatches of 512 (sequence 0)
    prompt = torch.from_numpy(rng.integers(0, w["n_vocab"], w["prefill"]).astype(np.int32)).to(dev)
    prefill_tok_s = prefill_ub2048 = None
    nxt = torch.zeros(1, dtype=torch.int32, device=dev)
    logits = torch.empty((1, w["n_vocab"]), dtype=torch.float32, device=dev)
    if not args.no_prefill:
        # the prompt goes through twice: the first pass is the warm-up (first launches, scratch growth), the
        # second, which rewrites the same cache rows with the same values, is the timed one
        # micro-batches of 2048 first (llama-server's --ubatch-size for vision models, launch.rs:1501-1503), then
        # the default 512, whose cache rows the decode steps continue from
        for ub, timed in ((UB, False), (UB, True), (512, False), (512, True)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for p0 in range(0, w["prefill"], ub):
                chunk = prompt[p0:p0 + ub]
                st.forward(tokens=chunk, n_seq=1, T=chunk.numel(), pos0=p0, logits=logits, next_tokens=nxt)
            e1.record()
            torch.cuda.synchronize()
            rate = w["prefill"] / (e0.elapsed_time(e1) * 1e-3)
            if timed and ub == 512:
                prefill_tok_s = rate
            elif timed:
                prefill_ub2048 = rate
            elif os.environ.get("B200_BENCH_VERBOSE"):
                print(f"[bench] warm-up prefill pass, micro-batch {ub}: {rate:.0f} tok/s", file=sys.stderr)
    pos = w["prefill"]

    # ---- decode, device resident: the stage feeds itself its own greedy token
    tok = nxt.clone()
    def decode_steps(k, pos):
        for _ in range(k):
            st.forward(tokens=tok, n_seq=1, T=1, pos0=pos, logits=logits, next_tokens=tok)
            pos += 1
        return pos
    pos = decode_steps(warmup, pos)
    torch.cuda.synchronize()
    launches0 = st.kernel_launches()
    sampler = ClockSampler(local) if full else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    pos = decode_steps(steps, pos)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    gpu_launches = st.kernel_launches() - launches0
    value = steps / (ms * 1e-3)

    # ---- decode, end to end: token ids arrive from pinned host memory, the result is read back
    h_tok = torch.zeros(1, dtype=torch.int32).pin_memory()
    h_out = torch.zeros(1, dtype=torch.int32).pin_memory()
    d_tok = torch.zeros(1, dtype=torch.int32, device=dev)
    d_out = torch.zeros(1, dtype=torch.int32, device=dev)
    h_tok[0] = int(tok.item())
    def e2e_steps(k, pos):
        for _ in range(k):
            d_tok.copy_(h_tok, non_blocking=True)
            st.forward(tokens=d_tok, n_seq=1, T=1, pos0=pos, logits=logits, next_tokens=d_out)
            h_out.copy_(d_out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            h_tok[0] = h_out[0]
            pos += 1
        return pos
    pos = e2e_steps(3, pos)
    torch.cuda.synchronize()
    tw0 = time.perf_counter()
    e0.record()
    pos = e2e_steps(steps, pos)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - tw0) * 1e3)
    e2e_value = steps / (e2e_ms * 1e-3)
    clocks = sampler.stop(t0, time.time()) if sampler else None

    # ---- the dominant kernel alone: all quantised GEMV launches of one step, replayed from a graph
    # over the real weights of every layer (GBs, so nothing is served from L2)
    ms_gemv, n_gemv = C.c_float(), C.c_int64()
    check(lib().b200_stage_profile_decode(st.h, 1, pos, 1, 10, C.byref(ms_gemv), C.byref(n_gemv)))
    ms_all, n_all = C.c_float(), C.c_int64()
    check(lib().b200_stage_profile_decode(st.h, 1, pos, 7, 10, C.byref(ms_all), C.byref(n_all)))
    ms_attn, n_attn = C.c_float(), C.c_int64()
    check(lib().b200_stage_profile_decode(st.h, 1, pos, 2, 10, C.byref(ms_attn), C.byref(n_attn)))
    algo = step_gemv_bytes(w, 0, w["n_layer"], True, 1)
    peak, peak_source = hbm_peak()
    achieved = algo / (ms_gemv.value * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "peak_source": peak_source, "unit": "GB/s",
        "frac": achieved / peak, "frac_of_nominal_8TBs": achieved / 8000.0,
        # DRAM read + write bytes per launch.  Not measured in this run: the algorithmic bytes of the step's
        # average launch times the DRAM / algorithmic ratio that ncu captures of isolated launches of the two
        # largest cfg2 matrices gave (1.02 Q4_K, 1.04 Q6_K; profiles/gemv_block_kernel_*.md)
        "traffic": NCU_TRAFFIC_RATIO * algo / max(1, n_gemv.value),
        "traffic_source": "derived: algorithmic bytes x %.2f, the DRAM / algorithmic ratio ncu measured on isolated cfg2 "
                          "launches at M = 1 (profiles/gemv_block_kernel_m1.md)" % NCU_TRAFFIC_RATIO,
        "kernel": "gemv_block_kernel (Q4_K/Q6_K x Q8 decode GEMV)",
        "launches_per_step": int(n_gemv.value), "algorithmic_bytes_per_launch": algo / max(1, n_gemv.value),
        "avg_launch_us": ms_gemv.value * 1e3 / max(1, n_gemv.value),
        "gemv_ms_per_step": ms_gemv.value, "attention_ms_per_step": ms_attn.value,
        "whole_step_graph_ms": ms_all.value,
    }

    # ---- batch-8 decode (8 slots of one server, same positions)
    b8 = None
    if n_seq >= 8:
        tok8 = torch.from_numpy(rng.integers(0, w["n_vocab"], 8).astype(np.int32)).to(dev)
        lg8 = torch.empty((8, w["n_vocab"]), dtype=torch.float32, device=dev)
        p8 = pos
        for _ in range(3):
            st.forward(tokens=tok8, n_seq=8, T=1, pos0=p8, logits=lg8, next_tokens=tok8); p8 += 1
        torch.cuda.synchronize()
        e0.record()
        k8 = max(8, steps // 4)
        for _ in range(k8):
            st.forward(tokens=tok8, n_seq=8, T=1, pos0=p8, logits=lg8, next_tokens=tok8); p8 += 1
        e1.record()
        torch.cuda.synchronize()
        b8 = 8 * k8 / (e0.elapsed_time(e1) * 1e-3)
    st.close()
    del st
    torch.cuda.empty_cache()
    active = step_gemv_bytes(w, 0, w["n_layer"], True, 1)  # bytes one token touches (experts: the selected ones)
    return {
        "value": value, "ms_per_step": ms / steps, "e2e_value": e2e_value, "gpu_launches": int(gpu_launches),
        "prefill_tok_s": prefill_tok_s, "prefill_ub2048_tok_s": prefill_ub2048, "decode_batch8_tok_s": b8, "roofline": roofline, "clocks": clocks,
        "weight_bytes": weight_bytes, "kv_cache": kv_label,
        "weight_stream_frac": None if w.get("n_expert", 0) else (weight_bytes / (ms / steps * 1e-3) / 1e9) / peak,
        "weight_stream_frac_active": (active / (ms / steps * 1e-3) / 1e9) / peak,
        "workload": f"{w['name']} ({w['n_layer']} layers), prefill {w['prefill']}, decode batch 1 at context {w['prefill']}+, "
                    f"one stage on one GPU, {steps} steps",
    }


def prefill_gemm_roofline():
    """The prefill GEMM against a tensor-core ceiling measured in the same run: the useful int8 rate
    (2 M N K per launch) of the 32B shape's FFN matmuls at M = 2048, and a bare loop of the kernel's own
    tcgen05.mma kind::i8 instruction on all SMs (b200_probe_int8_mma).  Every useful product costs two MMAs
    (the K-quant sub-block scale is folded into the weight, which then needs two int8 planes), so the
    issued rate is twice the useful one."""
    from mesh_llm_b200 import ops

    peak, _ = ops.probe_int8_mma(65536, 5)
    rows = {}
    for (N, K, t) in ((27648, 5120, "q4_k"), (5120, 27648, "q4_k"), (5120, 27648, "q6_k")):
        rows[f"{t}_{N}x{K}_m2048"] = micro_one(N, K, 2048, t, 4)["TOPps"]
    best = max(rows.values())
    return {"bound": "tensor", "achieved": best, "achieved_issued": 2 * best, "peak": peak,
            "peak_source": "measured in this run: bare tcgen05.mma.kind::i8 loop, M 128 x N 256 x K 32, one CTA per SM",
            "unit": "TOP/s", "frac": best / peak, "frac_issued": 2 * best / peak, "useful_TOPps": rows}


def hbm_peak():
    """(GB/s, where the number comes from): the driver-measured copy bandwidth of this pool's B200s"""
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(peaks["hbm_gbs"]), "MEASURED_PEAKS.json hbm_gbs"
    except Exception:
        return 6650.0, "fallback 6650 GB/s"


def cfg1_timed_cpu_leg(local, n_decode=128):
    """cfg1 (3B shape) in full on both sides with identical weights: the GPU runs the 512-token prompt and
    128 greedy steps; the CPU oracle, on all host cores, is timed on the same prompt and the same 128
    inputs (the GPU's tokens, so both see one history).  Reports tokens/s of both, top-1 agreement and the
    mean KL divergence of the logits."""
    import torch

    from mesh_llm_b200.stage import Stage
    from oracle import binding as orc

    w = dict(WORKLOADS["cfg1"])
    model = {k: w[k] for k in MODEL_KEYS if k in w}
    n_ctx = w["prefill"] + n_decode + 8
    st = Stage(**model, n_ctx=n_ctx, n_seq=1, n_ubatch=512, device=local)
    st.generate(20251125)
    orc.lib().orc_set_threads(host_threads())
    cores = orc.lib().orc_get_threads()
    m = orc.Model(**model, n_ctx=n_ctx)
    for n in m.tensor_names():  # the device-generated weights, read back in GGUF layout
        ty, data, _ = m.tensor(n)
        m.set_tensor(n, ty, st.get_tensor(n, data.size))
    dev = torch.device("cuda", local)
    prompt = np.random.default_rng(1234).integers(0, w["n_vocab"], w["prefill"]).astype(np.int32)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    logits = torch.empty((1, w["n_vocab"]), dtype=torch.float32, device=dev)
    tok = torch.zeros(1, dtype=torch.int32, device=dev)
    st.forward(tokens=torch.from_numpy(prompt).to(dev), n_seq=1, T=w["prefill"], pos0=0, logits=logits, next_tokens=tok)  # warm
    torch.cuda.synchronize()
    e0.record()
    st.forward(tokens=torch.from_numpy(prompt).to(dev), n_seq=1, T=w["prefill"], pos0=0, logits=logits, next_tokens=tok)
    e1.record()
    torch.cuda.synchronize()
    gpu_prefill = w["prefill"] / (e0.elapsed_time(e1) * 1e-3)
    inputs, gl = [], []
    n_warm = 4  # the first steps (capture of the decode graph among them) are not timed
    for i in range(n_decode):
        if i == n_warm:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
        inputs.append(tok.clone())
        lg = torch.empty((1, w["n_vocab"]), dtype=torch.float32, device=dev)
        st.forward(tokens=inputs[-1], n_seq=1, T=1, pos0=w["prefill"] + i, logits=lg, next_tokens=tok)
        gl.append(lg)
    torch.cuda.synchronize()
    gpu_decode = (n_decode - n_warm) / (time.perf_counter() - t0)
    inputs = torch.cat(inputs).cpu().numpy()
    gl = torch.cat(gl).cpu().numpy()
    st.close()
    t0 = time.perf_counter()
    m.forward(tokens=prompt, want_logits=False)
    cpu_prefill = w["prefill"] / (time.perf_counter() - t0)
    agree, kls, clear, clear_agree = 0, [], 0, 0
    t_dec = 0.0
    for i in range(n_decode):
        t0 = time.perf_counter()
        _, lref = m.forward(tokens=inputs[i:i + 1], pos0=w["prefill"] + i)
        t_dec += time.perf_counter() - t0
        a = lref[0].astype(np.float64) - lref[0].max()
        b = gl[i].astype(np.float64) - gl[i].max()
        la, lb = a - np.log(np.exp(a).sum()), b - np.log(np.exp(b).sum())
        kls.append(float((np.exp(la) * (la - lb)).sum()))
        same = int(lref[0].argmax() == gl[i].argmax())
        agree += same
        top2 = np.partition(lref[0], -2)[-2:]
        if top2[1] - top2[0] > 0.02 * np.abs(lref[0]).max():  # a clear winner on the CPU side
            clear += 1
            clear_agree += same
    m.close()
    return {"workload": f"{w['name']} ({w['n_layer']} layers), prompt {w['prefill']}, {n_decode} greedy steps, batch 1, "
                        "identical device-generated weights on both sides, CPU fed the GPU's tokens",
            "gpu_decode_tok_s": gpu_decode, "gpu_prefill_tok_s": gpu_prefill,
            "cpu_decode_tok_s": n_decode / t_dec, "cpu_prefill_tok_s": cpu_prefill, "cpu_cores": cores,
            "cpu_kind": "port (the CPU oracle timed in full, nothing extrapolated)",
            "top1_agreement": agree / n_decode, "mean_kl": float(np.mean(kls)),
            "steps_with_clear_cpu_winner": clear, "top1_agreement_on_those": (clear_agree / clear) if clear else None,
            "note": "weights are random, so most steps have near-tied top logits; 36 layers of re-quantised activations "
                    "let single rounding differences grow: a code that flips at a rounding tie moves a row by about 1e-2"}


if __name__ == "__main__":
    main()
