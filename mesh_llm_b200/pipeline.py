"""Layer-range pipeline over the GPUs of one box: one process per GPU, one stage per process.

This is mesh-llm's dense split (contiguous layer ranges per device, embeddings on the first
stage, output on the last: mesh-llm/src/inference/election.rs:3095-3114) with the reference's
ggml-RPC hand-off (third_party/llama.cpp/patches/0002 lines 544-622: device -> host -> TCP ->
host -> device) replaced by a device-to-device transfer over NVLink.  There is no collective on
the data path: the only exchange is the [rows x n_embd] f32 activation from stage g to g+1 and
the 4-byte greedy token from the last stage back to the first.

Batch-1 decode through a pipeline is serial per token, so to keep every stage busy the schedule
runs as many sequences as there are stages: at tick t stage r works on sequence (t - r) mod S.
The schedule (`Schedule`) is pure and is tested on CPU ranks with a stand-in stage.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass

import numpy as np


@dataclass
class Schedule:
    """tick <-> (sequence, decode step) for stage `rank` of `world` with `n_seq` sequences"""
    world: int
    n_seq: int

    def ticks(self, steps):
        return steps * self.n_seq + self.world - 1

    def work(self, rank, tick):
        """-> (seq, step) stage `rank` runs at `tick`, or None while the pipe fills / drains"""
        i = tick - rank
        if i < 0:
            return None
        return i % self.n_seq, i // self.n_seq


def layer_range(n_layer, world, rank, head_cost=0.0):
    """Contiguous layer range of a stage.  head_cost = 0: as equal as possible, earlier stages take the
    remainder (the equal split the benchmark configurations name).  head_cost > 0: the output head,
    which lives on the last stage, counts as that many layers and the last stage gets fewer layers, the
    way a proportional --tensor-split would place them (mesh-llm/src/inference/election.rs:3095-3114
    splits in proportion to what each device can hold, not in equal counts)."""
    if world > 1 and head_cost > 0:
        target = (n_layer + head_cost) / world
        last = int(round(target - head_cost))
        last = max(1, min(last, n_layer - (world - 1)))
        if rank == world - 1:
            return n_layer - last, n_layer
        n_layer, world = n_layer - last, world - 1
    base, rem = divmod(n_layer, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class Transport:
    """Point-to-point moves between neighbouring stages over torch.distributed.

    Sends never block the sender: at tick t the first stage sends a hidden state forward while the
    last stage sends a token back, and with rendezvous sends on one channel those two would wait
    for each other.  So sends are posted with isend, the forward (hidden) and backward (token)
    traffic use separate process groups (separate NCCL streams on GPUs), and a send buffer is only
    reused after the send posted from it two ticks earlier has completed.
    """

    def __init__(self, dist, rank, world, pg_fwd=None, pg_tok=None):
        self.dist, self.rank, self.world = dist, rank, world
        self.pg_fwd, self.pg_tok = pg_fwd, pg_tok
        self.pending = {}

    def _post(self, key, t, dst, pg):
        self.pending[key] = self.dist.isend(t, dst, group=pg)

    def wait_slot(self, key):
        w = self.pending.pop(key, None)
        if w is not None:
            w.wait()

    def send_hidden(self, t, slot):
        self._post(("h", slot), t, self.rank + 1, self.pg_fwd)

    def recv_hidden(self, t):
        self.dist.recv(t, self.rank - 1, group=self.pg_fwd)

    def send_token(self, t, slot):
        self._post(("t", slot), t, 0, self.pg_tok)

    def recv_token(self, t):
        self.dist.recv(t, self.world - 1, group=self.pg_tok)

    def drain(self):
        for k in list(self.pending):
            self.wait_slot(k)


class PeerTransport:
    """Transport's interface with the moves done by kernels of libb200kq.so: the sender writes the
    payload into the receiving stage's landing ring through the NVLink peer mapping and publishes its
    number; the receiver's kernel acquires it and copies it to the stage's input (handoff.py).  No
    rendezvous and no host involvement per token; buffers are reused in stream order, so wait_slot
    has nothing to wait for.  Endpoints: every stage but the first receives hidden states, the first
    receives the greedy tokens of the last."""

    def __init__(self, dist, rank, world, hidden_bytes, n_slots=16):
        from .handoff import Endpoint, Sender

        self.rank, self.world = rank, world
        self.rx_h = Endpoint(hidden_bytes, n_slots) if rank > 0 else None
        self.rx_t = Endpoint(16, n_slots) if rank == 0 and world > 1 else None
        mine = {"h": self.rx_h.handle() if self.rx_h else None, "t": self.rx_t.handle() if self.rx_t else None}
        handles = [None] * world
        dist.all_gather_object(handles, mine)
        self.tx_h = Sender.open(handles[rank + 1]["h"], hidden_bytes, n_slots) if rank < world - 1 else None
        self.tx_t = Sender.open(handles[0]["t"], 16, n_slots) if rank == world - 1 and world > 1 else None

    def wait_slot(self, key):
        pass

    def send_hidden(self, t, slot):
        self.tx_h.send(t)

    def recv_hidden(self, t):
        self.rx_h.wait(t)

    def send_token(self, t, slot):
        self.tx_t.send(t)

    def recv_token(self, t):
        self.rx_t.wait(t)

    def drain(self):
        pass

    def check(self):
        """after the stream has been synchronised: raises if any bounded wait gave up"""
        for o in (self.rx_h, self.rx_t, self.tx_h, self.tx_t):
            if o is not None:
                o.raise_on_timeout()

    def close_senders(self):
        """unmap the peers' rings; every rank does this (and a barrier) before any ring is freed"""
        for o in (self.tx_h, self.tx_t):
            if o is not None:
                o.close()

    def close(self):
        self.close_senders()
        for o in (self.rx_h, self.rx_t):
            if o is not None:
                o.close()


def run_decode(stage_step, sched, rank, steps, transport, hidden_in, hidden_out, token_in, token_out,
               first_tokens, on_token=None, on_input=None):
    """Generic pipelined greedy decode.

    stage_step(seq, step, token_or_None, hidden_in_or_None, out) runs this rank's layers for one
    token of `seq` and writes `out`: one of the two `hidden_out` buffers (not the last stage) or one
    of the two `token_out` buffers (last stage).  `first_tokens[seq]` feeds step 0 on the first
    stage.  on_token(seq, step, token) is called on the last stage after each token, on_input(token)
    on the first stage before each token is consumed.
    """
    last = rank == sched.world - 1
    n = 0
    for tick in range(sched.ticks(steps)):
        w = sched.work(rank, tick)
        if w is None or w[1] >= steps:
            continue
        seq, step = w
        slot = n & 1
        n += 1
        if last:
            transport.wait_slot(("t", slot))
        else:
            transport.wait_slot(("h", slot))
        out = token_out[slot] if last else hidden_out[slot]
        if rank == 0:
            if step == 0:
                token_in.copy_(first_tokens[seq:seq + 1])
            else:
                transport.recv_token(token_in)  # greedy token of (seq, step - 1) from the last stage
            if on_input is not None:
                on_input(token_in)
            stage_step(seq, step, token_in, None, out)
        else:
            transport.recv_hidden(hidden_in)
            stage_step(seq, step, None, hidden_in, out)
        if last:
            if on_token is not None:
                on_token(seq, step, out)
            if sched.world > 1 and step + 1 < steps:
                transport.send_token(out, slot)
        else:
            transport.send_hidden(out, slot)
    transport.drain()


# ------------------------------------------------------------------------------------------------
def bench_pipeline(args, w, metric, rank, world, local):
    """bench.py body for N > 1: N stages, N sequences in flight, value = all tokens / max time."""
    import torch
    import torch.distributed as dist

    from .stage import Stage

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pg_fwd = dist.new_group(backend="nccl")
    pg_tok = dist.new_group(backend="nccl")
    model_keys = ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab", "qkv_bias",
                  "rope_neox", "rope_theta", "rms_eps")
    model = {k: w[k] for k in model_keys}
    head_cost = 0.0
    if getattr(args, "balance", False):  # the output head in units of an average layer's weight bytes
        from bench import gemv_bytes, matmuls

        layer_b = sum(gemv_bytes(N, K, ty) for l in (0, 1) for (N, K, ty) in matmuls(w, l)) / 2
        head_cost = gemv_bytes(w["n_vocab"], w["n_embd"], 14) / layer_b
    lo, hi = layer_range(w["n_layer"], world, rank, head_cost)
    n_seq = world
    steps, warm = args.steps, max(3, args.warmup)
    n_ctx = w["prefill"] + 2 * (steps + warm) + 72
    ids, names = {"f16": 1, "q4_0": 2, "q8_0": 8}, {1: "f16", 2: "q4_0", 8: "q8_0"}
    kv = getattr(args, "kv", "f16")
    if kv == "auto":  # the pair mesh-llm starts a model file of this size with
        from bench import step_gemv_bytes
        from .ops import kv_types_for_model_bytes

        kt, vt = kv_types_for_model_bytes(step_gemv_bytes(w, 0, w["n_layer"], True) + w["n_vocab"] * w["n_embd"] * 0.5625)
    else:
        kt, vt = [ids[t] for t in (kv + "-" + kv).split("-")[:2]]
    st = Stage(**model, layer_begin=lo, layer_end=hi, has_embd=int(rank == 0), has_output=int(rank == world - 1),
               n_ctx=n_ctx, n_seq=n_seq, n_ubatch=512, device=local, kv_type_k=kt, kv_type_v=vt)
    st.generate(20251125)
    tr = Transport(dist, rank, world, pg_fwd, pg_tok)
    sched = Schedule(world, n_seq)
    h = w["n_embd"]
    # decode hand-off: peer-memory kernels unless --handoff nccl asks for send/recv; prefill ubatches (MBs) use send/recv
    peer = getattr(args, "handoff", "peer") == "peer"
    tr_dec = tr
    if peer:
        # every rank must end up on the same transport: if mapping a neighbour's ring fails anywhere, all use send / recv
        try:
            tr_dec = PeerTransport(dist, rank, world, h * 4)
            ok = torch.ones(1, device=dev)
        except Exception as e:  # noqa: BLE001 - reported, then the collective below decides for everybody
            print(f"[rank {rank}] peer-memory hand-off unavailable ({e}); using send / recv", flush=True)
            ok = torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            if tr_dec is not tr:
                tr_dec.close()
            tr_dec, peer = tr, False
    rng = np.random.default_rng(1234)
    prompts = torch.from_numpy(rng.integers(0, w["n_vocab"], (n_seq, w["prefill"])).astype(np.int32)).to(dev)
    hid_big = torch.empty((512, h), dtype=torch.float32, device=dev)
    hid_out = torch.empty((512, h), dtype=torch.float32, device=dev)
    first = torch.zeros(n_seq, dtype=torch.int32, device=dev)
    tok1 = torch.zeros(1, dtype=torch.int32, device=dev)
    logits = torch.empty((1, w["n_vocab"]), dtype=torch.float32, device=dev) if rank == world - 1 else None
    last = rank == world - 1

    # ---- prefill: every sequence's prompt flows through the stages in ubatches of 512
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if not args.no_prefill:
        for s in range(n_seq):
            for p0 in range(0, w["prefill"], 512):
                T = min(512, w["prefill"] - p0)
                hin = None
                if rank > 0:
                    tr.recv_hidden(hid_big[:T])
                    hin = hid_big[:T]
                st.forward(tokens=prompts[s, p0:p0 + T] if rank == 0 else None, hidden_in=hin, n_seq=1, T=T,
                           pos0=p0, seq0=s, hidden_out=None if last else hid_out[:T], logits=logits,
                           next_tokens=first[s:s + 1] if last else None)
                if not last:
                    tr.send_hidden(hid_out[:T], 0)
                    tr.wait_slot(("h", 0))
    e1.record()
    torch.cuda.synchronize()
    t_prefill = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t_prefill, op=dist.ReduceOp.MAX)
    dist.broadcast(first, world - 1)  # first decode tokens come from the last stage
    pos_base = w["prefill"]

    hid1_in = torch.empty((1, h), dtype=torch.float32, device=dev)
    hid1_out = [torch.empty((1, h), dtype=torch.float32, device=dev) for _ in range(2)]
    tok_out = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(2)]

    def make_step(base):
        def stage_step(seq, step, token, hidden_in, out):
            st.forward(tokens=token, hidden_in=hidden_in, n_seq=1, T=1, pos0=base + step, seq0=seq,
                       hidden_out=None if last else out, logits=logits, next_tokens=out if last else None)
        return stage_step

    h_tok = torch.zeros(1, dtype=torch.int32).pin_memory()

    def via_host(token):  # the id is read on the host and comes back from pinned host memory
        h_tok.copy_(token, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        token.copy_(h_tok, non_blocking=True)

    def decode(k, base, first_tokens, e2e=False):
        run_decode(make_step(base), sched, rank, k, tr_dec, hid1_in, hid1_out, tok1, tok_out, first_tokens,
                   on_token=(lambda s_, k_, t_: via_host(t_)) if (e2e and last) else None,
                   on_input=via_host if (e2e and rank == 0) else None)

    decode(warm, pos_base, first)
    torch.cuda.synchronize()
    dist.barrier()
    launches0 = st.kernel_launches()
    from bench import ClockSampler

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.time()
    e0.record()
    decode(steps, pos_base + warm, first)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t1 = time.time()
    tt = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms = float(tt.item())
    launches = torch.tensor([st.kernel_launches() - launches0], device=dev, dtype=torch.int64)
    dist.all_reduce(launches)

    # ---- end to end: result token crosses to the host and back every step
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    decode(steps, pos_base + warm + steps, first, e2e=True)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    te = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    if peer:
        tr_dec.check()

    if rank == 0:
        total = steps * n_seq
        print(json.dumps({
            "metric": metric, "value": total / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int4/6 -> int32, f32 combine", "data": "synthetic",
            "config": {"split": "weighted by bytes (output head counted)" if head_cost > 0 else "equal layer counts",
                       "workload": f"{w['name']} ({w['n_layer']} layers) split into {world} contiguous layer ranges, "
                                   f"one per GPU; {n_seq} sequences in flight, decode batch 1 per stage at context "
                                   f"{w['prefill']}+; f32 [1 x {h}] activation handed to the next stage over NVLink",
                       "sequences_in_flight": n_seq, "kv_cache": names[kt] + "-" + names[vt],
                       "l2": "each stage streams its weights every tick (>> 126 MB L2), no flush needed"},
            "e2e": {"value": total / (float(te.item()) * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 4 * n_seq,
                    "d2h_bytes_per_step": 4 * n_seq},
            "gpu_launches": int(launches.item()), "clocks": clocks,
            "prefill_tok_s": None if args.no_prefill else n_seq * w["prefill"] / (float(t_prefill.item()) * 1e-3),
            "handoff": "peer-memory landing ring written by the sending stage's kernel over NVLink (prefill ubatches: "
                       "torch.distributed send/recv)" if peer else "torch.distributed send/recv (NCCL P2P over NVLink)",
        }))
    if peer:
        tr_dec.close_senders()
    dist.barrier()
    if peer:
        tr_dec.close()
    dist.destroy_process_group()


def bench_handoff_latency(args, w, rank, world, local):
    """One [1 x n_embd] f32 row bounced between ranks 0 and 1 `iters` times inside one stream on each side,
    no host synchronisation in between: half the round trip is the one-way cost of a hand-off as a stage
    sees it (launch of the send, the link, the wait).  Measured for the peer-memory kernels and for
    torch.distributed send / recv; rank 0 prints one JSON line."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    h = w["n_embd"]
    x = torch.randn(1, h, device=dev)
    y = torch.empty_like(x)
    iters = max(200, args.steps * 8)
    out = {}
    if rank < 2:
        from .handoff import Endpoint, Sender

        rx = Endpoint(h * 4, 16)
    else:
        rx = None
    handles = [None] * world
    dist.all_gather_object(handles, rx.handle() if rx else None)
    tx = Sender.open(handles[1 - rank], h * 4, 16) if rank < 2 else None

    def bounce_peer(n):
        for _ in range(n):
            if rank == 0:
                tx.send(x)
                rx.wait(y)
            elif rank == 1:
                rx.wait(y)
                tx.send(y)

    def bounce_nccl(n):
        for _ in range(n):
            if rank == 0:
                dist.send(x, 1)
                dist.recv(y, 1)
            elif rank == 1:
                dist.recv(y, 0)
                dist.send(y, 0)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, fn in (("peer", bounce_peer), ("nccl", bounce_nccl)):
        fn(20)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        fn(iters)
        e1.record()
        torch.cuda.synchronize()
        out[name + "_one_way_us"] = e0.elapsed_time(e1) * 1e3 / iters / 2
        if rank == 0 and name == "peer":
            assert torch.equal(x, y), "the row did not come back bit for bit"
    if rank < 2:
        rx.raise_on_timeout()
        tx.raise_on_timeout()
        tx.close()
    dist.barrier()
    if rx:
        rx.close()
    if rank == 0:
        print(json.dumps({"handoff_latency": out, "payload_bytes": h * 4, "round_trips": iters, "n_gpus": world,
                          "method": "CUDA events on rank 0 around the whole loop, no host synchronisation inside"}))
    dist.destroy_process_group()


def bench_expert_replicas(args, w, metric, rank, world, local):
    """bench.py body for an MoE model at N > 1: N independent replicas, rank r holding the trunk and
    experts [r*E/N, (r+1)*E/N) with the router rows of those experts (the layout the reference's
    expert shards have: patches/0003 llama-moe-split, mesh-llm/src/inference/moe.rs).  No data-path
    traffic between ranks; every rank decodes its own sequence; value = all tokens / max time."""
    import torch
    import torch.distributed as dist

    from .stage import Stage

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    keys = ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab", "qkv_bias", "rope_neox",
            "rope_theta", "rms_eps", "n_ff_exp")
    model = {k: w[k] for k in keys}
    e_local = w["n_expert"] // world
    model["n_expert"] = e_local
    model["n_expert_used"] = min(w["n_expert_used"], e_local)
    steps, warm = args.steps, max(3, args.warmup)
    st = Stage(**model, n_ctx=w["prefill"] + 2 * (steps + warm) + 72, n_seq=1, n_ubatch=512, device=local)
    st.generate(20251125 + rank)
    rng = np.random.default_rng(1234 + rank)
    prompt = torch.from_numpy(rng.integers(0, w["n_vocab"], w["prefill"]).astype(np.int32)).to(dev)
    tok = torch.zeros(1, dtype=torch.int32, device=dev)
    logits = torch.empty((1, w["n_vocab"]), dtype=torch.float32, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn):
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def prefill():
        for p0 in range(0, w["prefill"], 512):
            chunk = prompt[p0:p0 + 512]
            st.forward(tokens=chunk, n_seq=1, T=chunk.numel(), pos0=p0, logits=logits, next_tokens=tok)

    t_prefill = None if args.no_prefill else timed(prefill)
    pos = [w["prefill"]]

    def decode(k):
        for _ in range(k):
            st.forward(tokens=tok, n_seq=1, T=1, pos0=pos[0], logits=logits, next_tokens=tok)
            pos[0] += 1

    h_tok = torch.zeros(1, dtype=torch.int32).pin_memory()

    def decode_e2e(k):
        for _ in range(k):
            h_tok.copy_(tok, non_blocking=True)  # result to the host ...
            torch.cuda.current_stream().synchronize()
            tok.copy_(h_tok, non_blocking=True)  # ... and back in as the next input
            st.forward(tokens=tok, n_seq=1, T=1, pos0=pos[0], logits=logits, next_tokens=tok)
            pos[0] += 1

    decode(warm)
    from bench import ClockSampler

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = st.kernel_launches()
    t0 = time.time()
    ms = timed(lambda: decode(steps))
    t1 = time.time()
    launches = torch.tensor([st.kernel_launches() - launches0], device=dev, dtype=torch.int64)
    dist.all_reduce(launches)
    te = timed(lambda: decode_e2e(steps))
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    if rank == 0:
        total = steps * world
        print(json.dumps({
            "metric": metric, "value": total / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int4/6 -> int32, f32 combine", "data": "synthetic",
            "config": {"workload": f"{w['name']} ({w['n_layer']} layers): {world} replicas, each the trunk plus "
                                   f"{e_local} of {w['n_expert']} experts (top-{model['n_expert_used']}), one sequence "
                                   f"per replica, decode batch 1 at context {w['prefill']}+; no traffic between GPUs",
                       "sequences_in_flight": world,
                       "l2": "active weights per token exceed L2 only in aggregate; experts change every token"},
            "e2e": {"value": total / (te * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 4 * world,
                    "d2h_bytes_per_step": 4 * world},
            "gpu_launches": int(launches.item()), "clocks": clocks,
            "prefill_tok_s": None if t_prefill is None else world * w["prefill"] / (t_prefill * 1e-3),
        }))
    dist.destroy_process_group()
