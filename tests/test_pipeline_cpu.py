"""Multi-rank host logic of the layer-range pipeline on CPU ranks (gloo, world_size 2 and 3).

A stand-in stage does exact integer arithmetic, so the pipelined greedy decode must reproduce the
sequential single-stage result token for token (the reference's own end-to-end check is
"1 server vs 2 servers give the same greedy tokens", third_party/llama.cpp/patches/0002 lines
827-972, where a difference is only a warning; here it is a hard assert).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mesh_llm_b200.pipeline import Schedule, Transport, layer_range, run_decode

N_LAYER, VOCAB = 7, 101


def layer_fn(l, v):
    return (v * (2 * l + 3) + l + 1) % 1009


def full_step(tok):
    v = int(tok) * 7 + 1
    for l in range(N_LAYER):
        v = layer_fn(l, v)
    return v % VOCAB


def test_schedule_and_layer_ranges():
    assert [layer_range(64, 8, r) for r in range(8)] == [(8 * r, 8 * r + 8) for r in range(8)]
    assert [layer_range(7, 3, r) for r in range(3)] == [(0, 3), (3, 5), (5, 7)]
    assert layer_range(80, 1, 0) == (0, 80)
    # weighted: the head of the 32B shape weighs 2.2 layers, of the 70B shape 1.7
    assert [layer_range(64, 8, r, 2.2) for r in range(8)] == [(0, 9), (9, 18), (18, 26), (26, 34), (34, 42), (42, 50),
                                                                (50, 58), (58, 64)]
    assert [layer_range(64, 2, r, 2.2) for r in range(2)] == [(0, 33), (33, 64)]
    assert [b - a for a, b in (layer_range(80, 8, r, 1.7) for r in range(8))] == [11, 10, 10, 10, 10, 10, 10, 9]
    assert layer_range(64, 1, 0, 2.2) == (0, 64)
    s = Schedule(4, 4)
    assert s.work(0, 0) == (0, 0) and s.work(3, 2) is None and s.work(3, 3) == (0, 0)
    assert s.work(0, 4) == (0, 1) and s.work(1, 4) == (3, 0)
    # every (seq, step) is visited exactly once per stage, in pipeline order
    for r in range(4):
        seen = [s.work(r, t) for t in range(s.ticks(3)) if s.work(r, t) and s.work(r, t)[1] < 3]
        assert sorted(seen) == [(q, k) for q in range(4) for k in range(3)]
    # two sequences per stage in flight: the same, and a sequence's next step comes up on the first stage
    # world + 1 ticks after the last stage has produced its token
    s2 = Schedule(4, 8)
    for r in range(4):
        seen = [s2.work(r, t) for t in range(s2.ticks(3)) if s2.work(r, t) and s2.work(r, t)[1] < 3]
        assert sorted(seen) == [(q, k) for q in range(8) for k in range(3)]
    t_last = next(t for t in range(64) if s2.work(3, t) == (0, 0))
    t_first = next(t for t in range(64) if s2.work(0, t) == (0, 1))
    assert t_first - t_last == 8 - 4 + 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, steps, first, q, n_seq):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = layer_range(N_LAYER, world, rank)
    last = rank == world - 1
    hin = torch.zeros(1, dtype=torch.int64)
    hout = [torch.zeros(1, dtype=torch.int64) for _ in range(2)]
    tok = torch.zeros(1, dtype=torch.int64)
    tout = [torch.zeros(1, dtype=torch.int64) for _ in range(max(2, n_seq))]
    got = {}

    def stage_step(seq, step, token, hidden_in, out):
        v = int(token.item()) * 7 + 1 if hidden_in is None else int(hidden_in.item())
        for l in range(lo, hi):
            v = layer_fn(l, v)
        out[0] = v % VOCAB if last else v

    run_decode(stage_step, Schedule(world, n_seq), rank, steps, Transport(dist, rank, world), hin, hout, tok,
               tout, torch.tensor(first, dtype=torch.int64),
               on_token=(lambda s, k, t: got.__setitem__((s, k), int(t.item()))) if last else None)
    if last:
        q.put(got)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_seq", [(2, 2), (3, 3), (2, 4), (3, 5)])
def test_pipelined_decode_equals_sequential(world, n_seq):
    """n_seq > world: more sequences in flight than stages (the token's way back is then off the critical path)"""
    steps = 5
    first = [3 + 11 * s for s in range(n_seq)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, steps, first, q, n_seq)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for s in range(n_seq):
        t = first[s]
        for k in range(steps):
            t = full_step(t)
            assert got[(s, k)] == t, (s, k)
