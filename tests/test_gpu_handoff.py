"""Peer-memory stage hand-off: byte exactness, ordering, back-pressure and bounded waits.

The exactness cases are the ones the reference pushes between two servers
(third_party/llama.cpp/patches/0002 test_direct_push, lines 1612-1745: forward and reverse byte
patterns, a partial window, a 16 MB payload), taken from tests/golden/handoff_pattern.npz.  On one GPU
the send is ordered before the wait on one stream, so no kernel ever waits for another one; the
time-out cases wait for something that nothing sends, with a limit of a few milliseconds, and read the
status the kernel left.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden", "handoff_pattern.npz")
MS = 1_000_000


def test_patterns_arrive_byte_exact_and_in_order():
    import torch
    from mesh_llm_b200.handoff import Endpoint

    g = np.load(GOLD)
    ep = Endpoint(4096, n_slots=4)
    tx = ep.local_sender()
    fwd, rev = torch.from_numpy(g["forward"]).cuda(), torch.from_numpy(g["reverse"]).cuda()
    off, size = int(g["partial_offset"]), int(g["partial_size"])
    out = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    # full forward, full reverse, then a partial window into the middle of a zeroed buffer
    tx.send(fwd)
    ep.wait(out)
    assert torch.equal(out, fwd)
    tx.send(rev)
    ep.wait(out)
    assert torch.equal(out, rev)
    out.zero_()
    tx.send(fwd[off:off + size])
    ep.wait(out[off:off + size])
    torch.cuda.synchronize()
    assert torch.equal(out[off:off + size], fwd[off:off + size]) and not out[:off].any() and not out[off + size:].any()
    # several payloads queued before the first is taken: they come out in order, through the wrap of the ring
    rows = [torch.full((4096,), i, dtype=torch.uint8, device="cuda") for i in range(1, 11)]
    got = []
    for i in range(0, 10, 2):
        tx.send(rows[i])
        tx.send(rows[i + 1])
        for _ in range(2):
            o = torch.empty(4096, dtype=torch.uint8, device="cuda")
            ep.wait(o)
            got.append(o)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(got, rows))
    assert ep.status() == 0 and tx.status() == 0


def test_large_payload_and_activation_rows():
    import torch
    from mesh_llm_b200.handoff import Endpoint

    n = int(np.load(GOLD)["large_bytes"])
    ep = Endpoint(n, n_slots=2)
    tx = ep.local_sender()
    src = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda")
    dst = torch.empty_like(src)
    tx.send(src)
    ep.wait(dst)
    torch.cuda.synchronize()
    assert torch.equal(src, dst)
    # the decode hand-off itself: one f32 row of n_embd values, bit for bit
    ep2 = Endpoint(5120 * 4, n_slots=16)
    tx2 = ep2.local_sender()
    x = torch.randn(1, 5120, device="cuda")
    y = torch.empty_like(x)
    for _ in range(40):
        tx2.send(x)
        ep2.wait(y)
    torch.cuda.synchronize()
    assert torch.equal(x, y) and ep2.status() == 0 and tx2.status() == 0
    # and the 4-byte greedy token that goes back to the first stage (a view at an odd word of a larger tensor)
    ep3 = Endpoint(16, n_slots=4)
    tx3 = ep3.local_sender()
    toks = torch.arange(100, 108, dtype=torch.int32, device="cuda")
    back = torch.zeros(8, dtype=torch.int32, device="cuda")
    for i in range(8):
        tx3.send(toks[i:i + 1])
        ep3.wait(back[i:i + 1])
    torch.cuda.synchronize()
    assert torch.equal(toks, back) and ep3.status() == 0


def test_payload_read_in_place_then_released():
    import torch
    from mesh_llm_b200.capi import check, cur_stream, lib, ptr
    from mesh_llm_b200.handoff import Endpoint

    ep = Endpoint(1024, n_slots=2)
    tx = ep.local_sender()
    zeros = torch.zeros(256, device="cuda")
    for i in range(5):  # more payloads than slots: each slot must be released before it is reused
        src = torch.full((256,), float(i), device="cuda")
        tx.send(src, limit_ns=50 * MS)
        addr, seq = ep.wait_in_place(1024, limit_ns=50 * MS)
        view = torch.empty(256, device="cuda")
        check(lib().b200_add(addr, ptr(zeros), 256, ptr(view), cur_stream()))  # an op reads the slot where it landed
        ep.release(seq)
        torch.cuda.synchronize()
        assert torch.equal(view, src)
    assert ep.status() == 0 and tx.status() == 0


def test_a_wait_for_nothing_gives_up_and_reports():
    import torch
    from mesh_llm_b200.handoff import Endpoint, HandoffTimeout

    ep = Endpoint(256, n_slots=2)
    dst = torch.full((64,), 7.0, device="cuda")
    ep.wait(dst, limit_ns=2 * MS)  # nothing was sent
    torch.cuda.synchronize()
    assert ep.status() == 2
    assert (dst == 7.0).all()  # untouched
    with pytest.raises(HandoffTimeout):
        ep.raise_on_timeout()
    # the context is still usable
    assert float((dst + 1).sum()) == 64 * 8.0


def test_a_send_into_a_full_ring_gives_up_and_reports():
    import torch
    from mesh_llm_b200.handoff import Endpoint

    ep = Endpoint(256, n_slots=2)
    tx = ep.local_sender()
    a, b, c = (torch.full((64,), v, device="cuda") for v in (1.0, 2.0, 3.0))
    tx.send(a, limit_ns=2 * MS)
    tx.send(b, limit_ns=2 * MS)
    tx.send(c, limit_ns=2 * MS)  # both slots hold payloads nobody took
    torch.cuda.synchronize()
    assert tx.status() == 1
    out = torch.empty(64, device="cuda")
    ep.wait(out, limit_ns=2 * MS)
    torch.cuda.synchronize()
    assert torch.equal(out, a)  # the payload in the slot was not overwritten by the refused send
    ep.wait(out, limit_ns=2 * MS)
    torch.cuda.synchronize()
    assert torch.equal(out, b) and ep.status() == 0


def test_between_two_devices_of_one_process():
    import torch
    from mesh_llm_b200.handoff import Endpoint

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with torch.cuda.device(1):
        ep = Endpoint(5120 * 4, n_slots=8)
    with torch.cuda.device(0):
        tx = ep.local_sender()
        xs = [torch.randn(1, 5120, device="cuda:0") for _ in range(6)]
        for x in xs:
            tx.send(x)
        torch.cuda.synchronize()
    with torch.cuda.device(1):
        for x in xs:
            y = torch.empty(1, 5120, device="cuda:1")
            ep.wait(y)
            torch.cuda.synchronize()
            assert torch.equal(x.to("cuda:1"), y)
        assert ep.status() == 0
    with torch.cuda.device(0):
        assert tx.status() == 0


def test_bad_arguments_are_refused():
    import torch
    from mesh_llm_b200.capi import B200Error
    from mesh_llm_b200.handoff import Endpoint

    with pytest.raises(B200Error):
        Endpoint(102)  # not a multiple of 4
    ep = Endpoint(256, n_slots=2)
    tx = ep.local_sender()
    with pytest.raises(B200Error):
        tx.send(torch.zeros(128, device="cuda"))  # 512 bytes into 256-byte slots
    with pytest.raises(B200Error):
        ep.wait(torch.zeros(128, device="cuda"))


def test_micro_batches_cross_in_place_through_a_three_slot_ring():
    """What the pipelined prefill does at a stage boundary: payloads of megabytes (reserve, grid-wide copy,
    publish on the sender's stream), read in place by the receiver through a tensor view of the landing
    slot and released afterwards; five payloads through three slots."""
    import torch
    from mesh_llm_b200.handoff import Endpoint
    from mesh_llm_b200.pipeline import _RawDeviceFloats

    rows, h = 256, 1024  # 1 MB
    ep = Endpoint(rows * h * 4, n_slots=3)
    tx = ep.local_sender()
    for i in range(5):
        src = torch.randn(rows, h, device="cuda") + i
        tx.send(src, limit_ns=50 * MS)
        addr, seq = ep.wait_in_place(rows * h * 4, limit_ns=50 * MS)
        view = torch.as_tensor(_RawDeviceFloats(addr, rows * h), device="cuda").view(rows, h)
        got = view.clone()  # the stage's kernels would read the slot here
        ep.release(seq)
        torch.cuda.synchronize()
        assert torch.equal(got, src), i
    assert ep.status() == 0 and tx.status() == 0
