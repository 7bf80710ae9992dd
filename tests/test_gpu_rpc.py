"""Worker front end on the GPU, through the wire: the reference's own exactness cases for direct
tensor pushes (third_party/llama.cpp/patches/0002: test_direct_push lines 1612-1745 -- full copy,
partial window offset 1024 size 2048 with untouched surroundings, reverse direction; test_large_push
16 MB; test_fallback_on_failed_push -- a push to a dead endpoint returns 0 and the caller relays),
plus graph_compute, the local-GGUF load and the spawned executable."""
import os
import socket
import subprocess
import time

import numpy as np
import pytest
import torch

from oracle import binding as orc
from rpc_client import Client, Server, make_tensor

pytestmark = pytest.mark.gpu
DATA_SIZE = 4096


def pattern(n, seed):
    return ((np.arange(n, dtype=np.uint32) * 2654435761 + seed) >> 13).astype(np.uint8)


def setup_pair(dev_b=0, size=DATA_SIZE):
    sa, sb = Server(), Server()
    a, b = Client(sa.port), Client(sb.port)
    assert a.register_peer(1, sb.endpoint) == 1 and b.register_peer(0, sa.endpoint) == 1
    ha, sza = a.alloc_buffer(0, size)
    hb, szb = b.alloc_buffer(dev_b, size)
    assert ha and hb and sza >= size and szb >= size
    ta = make_tensor(ha, a.buffer_get_base(ha), (size // 4,))
    tb = make_tensor(hb, b.buffer_get_base(hb), (size // 4,))
    return sa, sb, a, b, ta, tb


def second_device():
    return 1 if torch.cuda.device_count() > 1 else 0


def test_direct_push_full_partial_reverse():
    sa, sb, a, b, ta, tb = setup_pair(second_device())
    try:
        src = pattern(DATA_SIZE, 1)
        a.set_tensor(ta, 0, src)
        assert a.push_tensor_to_peer(1, ta, tb, 0, DATA_SIZE) == 1
        assert np.array_equal(np.frombuffer(b.get_tensor(tb, 0, DATA_SIZE), np.uint8), src)
        # partial window: only [1024, 3072) may change
        b.set_tensor(tb, 0, bytes(DATA_SIZE))
        assert a.push_tensor_to_peer(1, ta, tb, 1024, 2048) == 1
        got = np.frombuffer(b.get_tensor(tb, 0, DATA_SIZE), np.uint8)
        assert not got[:1024].any() and not got[3072:].any() and np.array_equal(got[1024:3072], src[1024:3072])
        # reverse direction
        back = pattern(DATA_SIZE, 77)
        b.set_tensor(tb, 0, back)
        assert b.push_tensor_to_peer(0, tb, ta, 0, DATA_SIZE) == 1
        assert np.array_equal(np.frombuffer(a.get_tensor(ta, 0, DATA_SIZE), np.uint8), back)
    finally:
        a.close(); b.close(); sa.stop(); sb.stop()


def test_large_push_16_mb():
    n = 16 << 20
    sa, sb, a, b, ta, tb = setup_pair(second_device(), n)
    try:
        data = pattern(n, 5)
        a.set_tensor(ta, 0, data)
        assert a.push_tensor_to_peer(1, ta, tb, 0, n) == 1
        assert np.array_equal(np.frombuffer(b.get_tensor(tb, 0, n), np.uint8), data)
    finally:
        a.close(); b.close(); sa.stop(); sb.stop()


def test_fallback_on_failed_push():
    sa, sb, a, b, ta, tb = setup_pair()
    try:
        assert a.register_peer(1, "127.0.0.1:59999") == 1  # nobody listens there
        data = pattern(DATA_SIZE, 9)
        a.set_tensor(ta, 0, data)
        assert a.push_tensor_to_peer(1, ta, tb, 0, DATA_SIZE) == 0  # the command itself succeeds
        relay = a.get_tensor(ta, 0, DATA_SIZE)  # the caller's fall-back: get + set
        b.set_tensor(tb, 0, relay)
        assert np.array_equal(np.frombuffer(b.get_tensor(tb, 0, DATA_SIZE), np.uint8), data)
        bad = make_tensor(tb.buffer, tb.data + DATA_SIZE - 16, (DATA_SIZE // 4,))  # runs past its buffer
        assert a.register_peer(1, sb.endpoint) == 1
        assert a.push_tensor_to_peer(1, ta, bad, 0, DATA_SIZE) == 0  # refused by the receiving server
    finally:
        a.close(); b.close(); sa.stop(); sb.stop()


def test_push_between_devices_of_one_server_is_a_device_copy():
    with Server() as s:
        c = Client(s.port)
        assert c.device_count() == torch.cuda.device_count()
        assert c.register_peer(3, s.endpoint) == 1  # the peer is this server
        h0, _ = c.alloc_buffer(0, DATA_SIZE)
        h1, _ = c.alloc_buffer(second_device(), DATA_SIZE)
        t0 = make_tensor(h0, c.buffer_get_base(h0), (DATA_SIZE // 4,))
        t1 = make_tensor(h1, c.buffer_get_base(h1), (DATA_SIZE // 4,))
        data = pattern(DATA_SIZE, 21)
        c.set_tensor(t0, 0, data)
        assert c.buffer_clear(h1, 0)
        assert c.push_tensor_to_peer(3, t0, t1, 1024, 2048) == 1
        got = np.frombuffer(c.get_tensor(t1, 0, DATA_SIZE), np.uint8)
        assert not got[:1024].any() and not got[3072:].any() and np.array_equal(got[1024:3072], data[1024:3072])
        assert c.free_buffer(h0) and c.free_buffer(h1)
        c.close()


@pytest.mark.parametrize("ty,M", [(orc.TYPE_Q4_K, 1), (orc.TYPE_Q6_K, 3), (orc.TYPE_Q4_K, 16)])
def test_graph_compute_and_recompute_over_the_wire(ty, M):
    rng = np.random.default_rng(8)
    N, K = 384, 1024
    W = orc.quantize_weights(ty, (rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((M, K)).astype(np.float32)
    with Server() as s:
        c = Client(s.port)
        h, size = c.alloc_buffer(0, 1 << 22)
        base = c.buffer_get_base(h)
        off = [0]

        def place(nbytes):
            p = base + off[0]
            off[0] += (nbytes + 255) & ~255
            return p

        tw = make_tensor(h, place(W.nbytes + 4096), (K, N), type_=ty, nb0=144 if ty == orc.TYPE_Q4_K else 210, name="W", id_=11)
        tx = make_tensor(h, place(x.nbytes), (K, M), name="x", id_=12)
        ty_ = make_tensor(h, place(M * N * 4), (N, M), name="y", id_=13, op=1, src=(11, 12))  # MUL_MAT
        c.set_tensor(tw, 0, W.tobytes())
        c.set_tensor(tx, 0, x.tobytes())
        c.graph_compute(0, [13], [tw, tx, ty_])
        got = np.frombuffer(c.get_tensor(ty_, 0, M * N * 4), np.float32).reshape(M, N)
        ref = orc.mul_mat(ty, W, x, N, K)
        assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
        x2 = rng.standard_normal((M, K)).astype(np.float32)
        c.set_tensor(tx, 0, x2.tobytes())
        c.graph_recompute(0)
        got2 = np.frombuffer(c.get_tensor(ty_, 0, M * N * 4), np.float32).reshape(M, N)
        ref2 = orc.mul_mat(ty, W, x2, N, K)
        assert np.abs(got2 - ref2).max() <= 1e-3 * np.abs(ref2).max()
        c.close()


def test_set_tensor_gguf_loads_from_the_servers_file(tmp_path):
    from gguf_util import write_model_gguf

    cfg = dict(n_layer=1, n_embd=512, n_head=4, n_head_kv=2, head_dim=128, n_ff=512, n_vocab=512, n_ctx=32)
    m = orc.Model(**cfg)
    m.generate(6)
    path = tmp_path / "m.gguf"
    write_model_gguf(path, m)
    with Server(path) as s:
        c = Client(s.port)
        h, _ = c.alloc_buffer(0, 1 << 22)
        base = c.buffer_get_base(h)
        for name, nb0 in (("blk.0.attn_q.weight", 144), ("blk.0.ffn_down.weight", 210), ("blk.0.attn_norm.weight", 4)):
            ty, data, ne = m.tensor(name)
            t = make_tensor(h, base, (ne[0], ne[1]), type_=ty, nb0=nb0, name=name)
            assert c.set_tensor_gguf(t) == 1
            assert np.array_equal(np.frombuffer(c.get_tensor(t, 0, data.size), np.uint8), data), name
        t = make_tensor(h, base, (512, 4), name="blk.9.nope.weight")
        assert c.set_tensor_gguf(t) == 0  # not in the file: the client sends the bytes itself
        c.close()
    with Server() as s:  # no file configured
        c = Client(s.port)
        h, _ = c.alloc_buffer(0, 4096)
        assert c.set_tensor_gguf(make_tensor(h, c.buffer_get_base(h), (16,), name="blk.0.attn_norm.weight")) == 0
        c.close()


def test_spawned_worker_executable():
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "mesh_llm_b200", "b200-rpc-server")
    assert os.path.exists(exe), "build it with python -m mesh_llm_b200.build"
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    proc = subprocess.Popen([exe, "-d", "B200_0", "-H", "127.0.0.1", "-p", str(port)], stdout=subprocess.PIPE,
                            stderr=subprocess.STDOUT)
    try:
        c = None
        for _ in range(100):
            try:
                c = Client(port)
                break
            except OSError:
                time.sleep(0.1)
        assert c is not None, "worker did not start listening"
        assert c.device_count() >= 1
        h, size = c.alloc_buffer(0, 1 << 20)
        t = make_tensor(h, c.buffer_get_base(h), (1 << 18,))
        data = pattern(1 << 20, 3)
        c.set_tensor(t, 0, data)
        assert np.array_equal(np.frombuffer(c.get_tensor(t, 0, 1 << 20), np.uint8), data)
        assert c.free_buffer(h)
        c.close()
    finally:
        proc.terminate()
        assert proc.wait(timeout=20) == 0
    assert subprocess.run([exe, "-d", "CUDA0", "-p", str(port)], capture_output=True).returncode == 2  # unknown device name


def test_copy_tensor_of_a_size_that_is_no_multiple_of_256():
    """COPY_TENSOR copies the tensor's own byte count: 100 floats, read back exactly."""
    with Server() as s:
        c = Client(s.port)
        h, _ = c.alloc_buffer(0, 1 << 16)
        base = c.buffer_get_base(h)
        src = make_tensor(h, base, (100,), name="src")
        dst = make_tensor(h, base + 4096, (100,), name="dst")
        data = np.random.default_rng(31).standard_normal(100).astype(np.float32)
        c.set_tensor(src, 0, data.tobytes())
        assert c.buffer_clear(h, 0)
        c.set_tensor(src, 0, data.tobytes())
        assert c.copy_tensor(src, dst) == 1
        got = np.frombuffer(c.get_tensor(dst, 0, 400), np.float32)
        np.testing.assert_array_equal(got, data)
        # the bytes behind the destination were not touched
        tail = make_tensor(h, base + 4096 + 400, (64,), name="tail")
        assert not np.frombuffer(c.get_tensor(tail, 0, 256), np.uint8).any()
        assert c.free_buffer(h)
        c.close()


def test_graph_with_a_too_small_destination_over_the_wire_writes_nothing():
    """GRAPH_COMPUTE has no response; a node whose destination cannot hold the op's result is refused
    by the backend before anything is launched: the server drops the connection and the memory behind
    the destination is unchanged."""
    with Server() as s:
        c = Client(s.port)
        h, _ = c.alloc_buffer(0, 1 << 20)
        base = c.buffer_get_base(h)
        T, n = 8, 512
        x = np.random.default_rng(32).standard_normal((T, n)).astype(np.float32)
        tx = make_tensor(h, base, (n, T), name="x", id_=21)
        small = make_tensor(h, base + 65536, (n, 1), name="small", id_=22, op=3, src=(21,))  # RMS_NORM of 8 rows into 1
        small.op_params[0] = int(np.float32(1e-6).view(np.int32))
        guard = make_tensor(h, base + 65536 + n * 4, (n, T - 1), name="guard", id_=23)
        c.set_tensor(tx, 0, x.tobytes())
        sentinel = np.full((T - 1, n), 3.5, np.float32)
        c.set_tensor(guard, 0, sentinel.tobytes())
        c.graph_compute(0, [22], [tx, small])
        with pytest.raises((ConnectionError, OSError)):  # a failed command ends the connection, as in the reference
            c.get_tensor(guard, 0, 16)
        c.close()
        c2 = Client(s.port)  # buffers belong to the server, not to the connection
        got = np.frombuffer(c2.get_tensor(guard, 0, sentinel.nbytes), np.float32).reshape(T - 1, n)
        np.testing.assert_array_equal(got, sentinel)
        assert c2.free_buffer(h)
        c2.close()
