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
    token of `seq` and writes `out`: one of the `hidden_out` buffers (not the last stage) or one of
    the `token_out` buffers (last stage), used in rotation.  Over a transport whose sends complete
    only when received (send / recv), two hidden buffers are enough, and the last stage needs as many
    token buffers as there are sequences: with more sequences than stages its tokens wait for the
    first stage to come round to them.  `first_tokens[seq]` feeds step 0 on the first
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
        slot = n % (len(token_out) if last else len(hidden_out))
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


class _RawDeviceFloats:
    """lets torch view device memory it does not own (a landing slot of the hand-off ring)"""

    def __init__(self, address, n_floats):
        self.__cuda_array_interface__ = {"shape": (n_floats,), "typestr": "<f4", "data": (int(address), False), "version": 3}


class PrefillPeerLink:
    """Micro-batches of a prefill between neighbouring stages through peer memory: a ring of three
    landing slots of [512 x n_embd] f32 in the receiver's HBM.  The sender's stream reserves a slot,
    copies with a whole grid over NVLink and publishes; the receiver's stream acquires the slot, runs
    its layers on it in place and releases it.  Nobody waits on the host, so micro-batch u + 1 is
    computed while u crosses and while the next stage works on u."""

    def __init__(self, dist, rank, world, slot_bytes, n_slots=3):
        from .handoff import Endpoint, Sender

        self.rx = Endpoint(slot_bytes, n_slots) if rank > 0 else None
        handles = [None] * world
        dist.all_gather_object(handles, self.rx.handle() if self.rx else None)
        self.tx = Sender.open(handles[rank + 1], slot_bytes, n_slots) if rank < world - 1 else None

    def send(self, t):
        self.tx.send(t)

    def recv_in_place(self, rows, h, device):
        """-> (tensor [rows, h] over the landing slot, payload number to release after use)"""
        import torch

        addr, seqno = self.rx.wait_in_place(rows * h * 4)
        return torch.as_tensor(_RawDeviceFloats(addr, rows * h), device=device).view(rows, h), seqno

    def release(self, seqno):
        self.rx.release(seqno)

    def check(self):
        for o in (self.rx, self.tx):
            if o is not None:
                o.raise_on_timeout()

    def close_senders(self):
        if self.tx is not None:
            self.tx.close()

    def close(self):
        self.close_senders()
        if self.rx is not None:
            self.rx.close()


# ------------------------------------------------------------------------------------------------
MODEL_KEYS = ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab", "qkv_bias",
              "rope_neox", "rope_theta", "rms_eps")


def run_pipeline(args, w, rank, world, local, pg_fwd, pg_tok, steps, warm, full=True):
    """One dense workload over `world` stages: prefill, pipelined decode with `seqs_per_stage * world` sequences in flight
    (device-timed and end to end), one sequence alone through all stages, the slowest stage's GEMV-only
    replay, and a replay of sequence 0 on a single stage holding the whole model (rank 0) whose tokens
    must equal the pipeline's.  Returns the measurements on every rank."""
    import ctypes as C

    import torch
    import torch.distributed as dist

    from bench import ClockSampler, gemv_bytes, hbm_peak, matmuls, step_gemv_bytes

    from .capi import check, lib
    from .stage import Stage

    dev = torch.device("cuda", local)
    model = {k: w[k] for k in MODEL_KEYS}
    head_cost = 0.0
    if getattr(args, "balance", False):  # the output head in units of an average layer's weight bytes
        layer_b = sum(gemv_bytes(N, K, ty) for l in (0, 1) for (N, K, ty) in matmuls(w, l)) / 2
        head_cost = gemv_bytes(w["n_vocab"], w["n_embd"], 14) / layer_b
    lo, hi = layer_range(w["n_layer"], world, rank, head_cost)
    spp = max(1, int(getattr(args, "seqs_per_stage", 1)))
    if getattr(args, "handoff", "peer") != "peer":
        spp = 1  # rendezvous sends: a token that waits for its receiver would stall the last stage
    n_seq = world * spp
    n_ctx = w["prefill"] + 4 * (steps + warm) + 72
    ids, names = {"f16": 1, "q4_0": 2, "q8_0": 8}, {1: "f16", 2: "q4_0", 8: "q8_0"}
    kv = getattr(args, "kv", "f16")
    if kv == "auto":  # the pair mesh-llm starts a model file of this size with
        from .ops import kv_types_for_model_bytes

        kt, vt = kv_types_for_model_bytes(step_gemv_bytes(w, 0, w["n_layer"], True) + w["n_vocab"] * w["n_embd"] * 0.5625)
    else:
        kt, vt = [ids[t] for t in (kv + "-" + kv).split("-")[:2]]
    last = rank == world - 1
    st = Stage(**model, layer_begin=lo, layer_end=hi, has_embd=int(rank == 0), has_output=int(last),
               n_ctx=n_ctx, n_seq=n_seq, n_ubatch=512, device=local, kv_type_k=kt, kv_type_v=vt)
    st.generate(20251125)
    tr = Transport(dist, rank, world, pg_fwd, pg_tok)
    h = w["n_embd"]
    # hand-off: peer-memory kernels unless --handoff nccl asks for send / recv
    peer = getattr(args, "handoff", "peer") == "peer"
    tr_dec, big = tr, None
    if peer:
        # every rank must end up on the same transport: if mapping a neighbour's ring fails anywhere, all use send / recv
        try:
            tr_dec = PeerTransport(dist, rank, world, h * 4)
            big = PrefillPeerLink(dist, rank, world, 512 * h * 4)
            ok = torch.ones(1, device=dev)
        except Exception as e:  # noqa: BLE001 - reported, then the collective below decides for everybody
            print(f"[rank {rank}] peer-memory hand-off unavailable ({e}); using send / recv", flush=True)
            ok = torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            for o in (tr_dec if tr_dec is not tr else None, big):
                if o is not None:
                    o.close()
            tr_dec, big, peer = tr, None, False
            spp, n_seq = 1, world
    sched = Schedule(world, n_seq)
    rng = np.random.default_rng(1234)
    prompts = torch.from_numpy(rng.integers(0, w["n_vocab"], (n_seq, w["prefill"])).astype(np.int32)).to(dev)
    hid_big = torch.empty((512, h), dtype=torch.float32, device=dev)
    hid_out = [torch.empty((512, h), dtype=torch.float32, device=dev) for _ in range(2)]
    first = torch.zeros(n_seq, dtype=torch.int32, device=dev)
    tok1 = torch.zeros(1, dtype=torch.int32, device=dev)
    logits = torch.empty((1, w["n_vocab"]), dtype=torch.float32, device=dev) if last else None

    # ---- prefill: every sequence's prompt flows through the stages in micro-batches of 512
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if not args.no_prefill:
        u = 0
        for s in range(n_seq):
            for p0 in range(0, w["prefill"], 512):
                T = min(512, w["prefill"] - p0)
                hin, held = None, None
                if rank > 0:
                    if big is not None:
                        hin, held = big.recv_in_place(T, h, dev)
                    else:
                        tr.recv_hidden(hid_big[:T])
                        hin = hid_big[:T]
                out = hid_out[u & 1][:T]
                if big is None and not last:
                    tr.wait_slot(("h", u & 1))  # the send posted from this buffer two micro-batches ago
                st.forward(tokens=prompts[s, p0:p0 + T] if rank == 0 else None, hidden_in=hin, n_seq=1, T=T,
                           pos0=p0, seq0=s, hidden_out=None if last else out, logits=logits,
                           next_tokens=first[s:s + 1] if last else None)
                if held is not None:
                    big.release(held)
                if not last:
                    if big is not None:
                        big.send(out)
                    else:
                        tr.send_hidden(out, u & 1)
                u += 1
        tr.drain()
    e1.record()
    torch.cuda.synchronize()
    t_prefill = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t_prefill, op=dist.ReduceOp.MAX)
    dist.broadcast(first, world - 1)  # first decode tokens come from the last stage
    pos_base = w["prefill"]

    hid1_in = torch.empty((1, h), dtype=torch.float32, device=dev)
    hid1_out = [torch.empty((1, h), dtype=torch.float32, device=dev) for _ in range(2)]
    tok_out = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(2)]
    seq0_tokens = []  # last stage: the greedy tokens of sequence 0, in the order they were produced

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

    def keep(seq, step, token):
        if seq == 0:
            seq0_tokens.append(token.clone())

    def decode(k, base, first_tokens, e2e=False, sch=None, record=False):
        def on_token(s_, k_, t_):
            if record:
                keep(s_, k_, t_)
            if e2e:
                via_host(t_)
        run_decode(make_step(base), sch or sched, rank, k, tr_dec, hid1_in, hid1_out, tok1, tok_out, first_tokens,
                   on_token=on_token if (last and (e2e or record)) else None,
                   on_input=via_host if (e2e and rank == 0) else None)

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

    decode(warm, pos_base, first, record=True)
    torch.cuda.synchronize()
    dist.barrier()
    launches0 = st.kernel_launches()
    sampler = ClockSampler(local) if (full and rank == 0) else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    t0 = time.time()
    ms = timed(lambda: decode(steps, pos_base + warm, first, record=True))
    t1 = time.time()
    launches = torch.tensor([st.kernel_launches() - launches0], device=dev, dtype=torch.int64)
    dist.all_reduce(launches)
    # ---- end to end: result token crosses to the host and back every step
    te = timed(lambda: decode(steps, pos_base + warm + steps, first, e2e=True))
    clocks = sampler.stop(t0, t1) if sampler else None
    # ---- one sequence alone through all stages: the latency-bound batch-1 figure
    k1 = max(4, steps // 2)
    t_single = timed(lambda: decode(k1, pos_base + warm + 2 * steps, first, sch=Schedule(world, 1)))
    # ---- one sequence per stage in flight: every tick then also waits for the token's way back to the first stage
    t_one = None
    if spp > 1:
        t_one = timed(lambda: decode(k1, pos_base + warm + 2 * steps + k1, first, sch=Schedule(world, world)))
    if peer:
        tr_dec.check()
        big.check()

    # ---- this stage's GEMV launches alone; the slowest stage bounds the pipeline
    ms_gemv, n_gemv = C.c_float(), C.c_int64()
    check(lib().b200_stage_profile_decode(st.h, 1, pos_base, 1, 10, C.byref(ms_gemv), C.byref(n_gemv)))
    peak, peak_source = hbm_peak()
    algo = step_gemv_bytes(w, lo, hi, last, 1)
    mine = torch.tensor([ms_gemv.value, algo, float(n_gemv.value)], device=dev, dtype=torch.float64)
    allr = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allr, mine)
    per_stage = [(float(t[0]), float(t[1]), int(t[2])) for t in allr]
    slow = max(range(world), key=lambda r: per_stage[r][0])
    s_ms, s_algo, s_n = per_stage[slow]
    roofline = {
        "bound": "hbm", "achieved": s_algo / (s_ms * 1e-3) / 1e9, "peak": peak, "peak_source": peak_source, "unit": "GB/s",
        "frac": s_algo / (s_ms * 1e-3) / 1e9 / peak, "stage": slow,
        "per_stage_frac": [a / (m * 1e-3) / 1e9 / peak for (m, a, _) in per_stage],
        "traffic": None, "kernel": "gemv_block_kernel (Q4_K/Q6_K x Q8 decode GEMV), the slowest stage's launches of one step",
        "launches_per_step": s_n, "algorithmic_bytes_per_launch": s_algo / max(1, s_n),
        "avg_launch_us": s_ms * 1e3 / max(1, s_n), "gemv_ms_per_step": s_ms,
    }

    # ---- outputs must match: sequence 0 replayed on one stage holding the whole model
    n_tok = warm + steps
    toks = torch.stack(seq0_tokens).reshape(-1).to(torch.int32) if last else torch.zeros(n_tok, dtype=torch.int32, device=dev)
    dist.broadcast(toks, world - 1)
    match = torch.ones(1, device=dev)
    if peer:
        tr_dec.close_senders()
        big.close_senders()
    dist.barrier()
    if peer:
        tr_dec.close()
        big.close()
    st.close()
    del st
    torch.cuda.empty_cache()
    if rank == 0 and not getattr(args, "no_match", False):
        one = Stage(**model, n_ctx=n_ctx, n_seq=1, n_ubatch=512, device=local, kv_type_k=kt, kv_type_v=vt)
        one.generate(20251125)
        lg = torch.empty((1, w["n_vocab"]), dtype=torch.float32, device=dev)
        t_ = torch.zeros(1, dtype=torch.int32, device=dev)
        for p0 in range(0, w["prefill"], 512):
            T = min(512, w["prefill"] - p0)
            one.forward(tokens=prompts[0, p0:p0 + T], n_seq=1, T=T, pos0=p0, logits=lg, next_tokens=t_)
        got = []
        ok = bool(int(t_.item()) == int(first[0].item()))
        for (k, base) in ((warm, pos_base), (steps, pos_base + warm)):
            cur = first[0:1].clone()
            for i in range(k):
                nx = torch.zeros(1, dtype=torch.int32, device=dev)
                one.forward(tokens=cur, n_seq=1, T=1, pos0=base + i, logits=lg, next_tokens=nx)
                got.append(nx)
                cur = nx
        got = torch.cat(got)
        ok = ok and bool(torch.equal(got, toks))
        match.fill_(1.0 if ok else 0.0)
        one.close()
    dist.broadcast(match, 0)
    total = steps * n_seq
    return {
        "value": total / (ms * 1e-3), "ms_per_step": ms / steps, "e2e_value": total / (te * 1e-3),
        "gpu_launches": int(launches.item()), "clocks": clocks, "n_seq": n_seq,
        "prefill_tok_s": None if args.no_prefill else n_seq * w["prefill"] / (float(t_prefill.item()) * 1e-3),
        "single_sequence_tok_s": k1 / (t_single * 1e-3),
        "one_sequence_per_stage_tok_s": None if t_one is None else k1 * world / (t_one * 1e-3),
        "tokens_match_single_stage": None if getattr(args, "no_match", False) else bool(match.item() == 1.0),
        "tokens_compared": 1 + n_tok, "roofline": roofline, "kv_cache": names[kt] + "-" + names[vt], "peer": peer,
        "split": "weighted by bytes (output head counted)" if head_cost > 0 else "equal layer counts",
    }


def bench_pipeline(args, w, metric, rank, world, local):
    """bench.py body for N > 1: N stages, `--seqs-per-stage` x N sequences in flight (one sequence per stage and tick,
    batch 1), value = all tokens / max time."""
    import torch
    import torch.distributed as dist

    from bench import WORKLOADS, cpu_decode_sample, host_threads

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pg_fwd = dist.new_group(backend="nccl")
    pg_tok = dist.new_group(backend="nccl")
    steps, warm = args.steps, max(3, args.warmup)
    r = run_pipeline(args, w, rank, world, local, pg_fwd, pg_tok, steps, warm, full=True)
    extra = {}
    if not getattr(args, "no_extras", False) and not getattr(args, "balance", False) and not args.layers:
        # the same workload with the layers split by weight bytes (the last stage also holds the output head)
        import copy

        args_b = copy.copy(args)
        args_b.balance = True
        rb = run_pipeline(args_b, w, rank, world, local, pg_fwd, pg_tok, max(8, min(steps, 16)), 3, full=False)
        extra.update({"balanced_split_decode_tok_s": rb["value"], "balanced_split_e2e_tok_s": rb["e2e_value"],
                      "balanced_split": rb["split"], "balanced_split_tokens_match_single_stage": rb["tokens_match_single_stage"]})
    if not getattr(args, "no_extras", False) and args.workload == "cfg2" and not args.layers:
        # the 70B shape over the same N stages, in the same run
        w3 = dict(WORKLOADS["cfg3"])
        r3 = run_pipeline(args, w3, rank, world, local, pg_fwd, pg_tok, max(8, min(steps, 16)), 3, full=False)
        extra.update({"cfg3_decode_tok_s": r3["value"], "cfg3_e2e_tok_s": r3["e2e_value"],
                 "cfg3_single_sequence_tok_s": r3["single_sequence_tok_s"], "cfg3_prefill_tok_s": r3["prefill_tok_s"],
                 "cfg3_one_sequence_per_stage_tok_s": r3["one_sequence_per_stage_tok_s"],
                 "cfg3_tokens_match_single_stage": r3["tokens_match_single_stage"],
                 "cfg3_gemv_frac_of_hbm_peak": r3["roofline"]["frac"],
                 "cfg3_workload": f"{w3['name']} ({w3['n_layer']} layers) over {world} stages, {r3['n_seq']} sequences in flight, "
                                  f"prefill {w3['prefill']}, decode at context {w3['prefill']}+"})
    cpu = None
    if rank == 0 and not args.no_cpu:
        # the other ranks wait for this one in a barrier, each spinning on a core: one OpenMP thread more than
        # there are free cores makes every parallel loop wait for a descheduled thread (measured at 2 ranks on 24
        # cores: 24 threads 0.28 tok/s, 16 threads 1.56, 24 threads with the other rank asleep 2.36)
        v, cores, sample = cpu_decode_sample(w, threads=max(1, host_threads() - world))
        cpu = {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample}
    h = w["n_embd"]
    bad = (r["tokens_match_single_stage"] is False or extra.get("cfg3_tokens_match_single_stage") is False or
           extra.get("balanced_split_tokens_match_single_stage") is False)
    if rank == 0:
        out = {
            "metric": metric, "value": r["value"], "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int4/6 -> int32, f32 combine", "data": "synthetic",
            "config": {"split": r["split"],
                       "workload": f"{w['name']} ({w['n_layer']} layers) split into {world} contiguous layer ranges, "
                                   f"one per GPU; {r['n_seq']} sequences in flight, decode batch 1 per stage at context "
                                   f"{w['prefill']}+; f32 [1 x {h}] activation handed to the next stage over NVLink",
                       "sequences_in_flight": r["n_seq"], "kv_cache": r["kv_cache"],
                       "l2": "each stage streams its weights every tick (>> 126 MB L2), no flush needed"},
            "e2e": {"value": r["e2e_value"], "unit": "tok/s", "h2d_bytes_per_step": 4 * r["n_seq"],
                    "d2h_bytes_per_step": 4 * r["n_seq"]},
            "gpu_launches": r["gpu_launches"], "clocks": r["clocks"], "roofline": r["roofline"], "cpu_baseline": cpu,
            "prefill_tok_s": r["prefill_tok_s"], "single_sequence_tok_s": r["single_sequence_tok_s"],
            "one_sequence_per_stage_tok_s": r["one_sequence_per_stage_tok_s"],
            "tokens_match_single_stage": r["tokens_match_single_stage"], "tokens_compared": r["tokens_compared"],
            "handoff": "peer-memory landing rings written by the sending stage's kernels over NVLink (decode rows and "
                       "prefill micro-batches)" if r["peer"] else "torch.distributed send/recv (NCCL P2P over NVLink)",
        }
        out.update(extra)
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if bad:
        raise SystemExit("the pipeline's tokens differ from the single stage's")


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
