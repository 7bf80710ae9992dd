"""Worker front end, protocol level, no GPU: handshake, framing, peer registration rules and
connection churn — the device-free cases of the reference's own RPC test program
(third_party/llama.cpp/patches/0002 lines 1558-1616 test_peer_registration, 1885-1915
test_rapid_connect_disconnect)."""
import socket
import struct

import pytest

from rpc_client import (ALLOC_BUFFER, BUFFER_GET_BASE, Client, DEVICE_COUNT, GET_ALIGNMENT, HELLO, REGISTER_PEER,
                        Server)


@pytest.fixture
def server():
    with Server() as s:
        yield s


def test_hello_reports_protocol_4_1(server):
    c = Client(server.port, hello=False)
    assert c.hello() == (4, 1, 0)
    assert c.call(GET_ALIGNMENT, struct.pack("<I", 0)) == struct.pack("<Q", 256)
    assert isinstance(c.device_count(), int)
    c.close()


def test_first_command_must_be_hello(server):
    c = Client(server.port, hello=False)
    c.send(DEVICE_COUNT)
    with pytest.raises((ConnectionError, socket.timeout, OSError)):
        c.recv()
    c.close()
    c2 = Client(server.port)  # the server itself is unharmed
    assert c2.hello()[0] == 4
    c2.close()


def test_malformed_requests_close_only_their_connection(server):
    for cmd, payload in ((ALLOC_BUFFER, b"\x00" * 3), (BUFFER_GET_BASE, struct.pack("<Q", 0xDEADBEEF)), (99, b""),
                         (REGISTER_PEER, b"\x00" * 5)):
        c = Client(server.port)
        c.send(cmd, payload)
        with pytest.raises((ConnectionError, socket.timeout, OSError)):
            c.recv()
        c.close()
    c = Client(server.port, hello=False)
    c.s.sendall(struct.pack("<BQ", HELLO, 1 << 40))  # absurd payload size
    with pytest.raises((ConnectionError, socket.timeout, OSError)):
        c.recv()
    c.close()
    ok = Client(server.port)
    assert ok.hello() == (4, 1, 0)
    ok.close()


def test_peer_registration_rules(server):
    with Server() as other:
        a, b = Client(server.port), Client(other.port)
        assert a.register_peer(1, other.endpoint) == 1
        assert b.register_peer(0, server.endpoint) == 1
        assert a.register_peer(99, "") == 0  # empty endpoint
        assert a.register_peer(7, "nocolon") == 0 and a.register_peer(7, ":5000") == 0 and a.register_peer(7, "host:") == 0
        assert a.register_peer(1, "127.0.0.1:59998") == 1  # the same id again replaces the endpoint
        assert a.register_peer(50, "h" * 120 + ":1") == 1  # long endpoint
        a.close()
        b.close()


def test_unknown_peer_push_reports_failure_without_closing(server):
    from rpc_client import make_tensor

    c = Client(server.port)
    t = make_tensor(0, 0, (4,))
    assert c.push_tensor_to_peer(42, t, t, 0, 16) == 0
    assert c.hello() == (4, 1, 0)
    c.close()


def test_rapid_connect_disconnect(server):
    ok = 0
    for i in range(50):
        try:
            c = Client(server.port, hello=(i % 2 == 0))
            c.close()
            ok += 1
        except OSError:
            pass
    assert ok >= 45
    c = Client(server.port)
    assert c.hello() == (4, 1, 0)
    c.close()


def test_stop_with_open_connections():
    s = Server()
    c = Client(s.port)
    s.stop()
    with pytest.raises((ConnectionError, socket.timeout, OSError)):
        c.send(HELLO, bytes(24))
        c.recv()
    c.close()
