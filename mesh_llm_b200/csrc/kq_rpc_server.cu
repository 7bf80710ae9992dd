// A worker front end that speaks the ggml RPC wire protocol (version 4.1) and serves it from this
// library's backend, so that a mesh-llm host can use a B200 stage exactly as it uses the
// `rpc-server -d DEV -p PORT --gguf PATH` processes it spawns (mesh-llm/src/inference/launch.rs:
// 887-933).  Host code only.
//
// Wire format (third_party/llama.cpp/patches/0002, test client lines 1172-1230): a request is
// | cmd u8 | size u64 | payload |, a response | size u64 | payload |; SET_TENSOR and GRAPH_COMPUTE
// have no response.  Command ids and the packed message structs are those of patches/0002 lines
// 1042-1146 and patches/0001 lines 49-63; the 296-byte tensor record is b200_tensor.  Commands whose
// message layout is not visible in those patches (GET_ALIGNMENT, GET_MAX_SIZE, BUFFER_CLEAR,
// COPY_TENSOR, INIT_TENSOR, GET_DEVICE_MEMORY, DEVICE_COUNT, SET_TENSOR_HASH, the GRAPH_COMPUTE
// payload | device u32 | n_nodes u32 | node ids u64[] | n_tensors u32 | tensors[] |) follow the public
// protocol description of that version.
//
// Like the patched reference server, one server object is shared by all connections (a thread
// per connection) and every backend call runs under one mutex (patches/0002 lines 320-337).  A
// tensor record arriving from the wire is only handed to the backend after its buffer handle has
// been found in the set of live buffers.  A peer push between two devices of this server is one
// NVLink copy; to any other endpoint it travels as PEER_TENSOR_DATA over TCP, as in the reference.
#include "kq_common.cuh"

#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

namespace {

enum Cmd : uint8_t {
    ALLOC_BUFFER = 0, GET_ALIGNMENT, GET_MAX_SIZE, BUFFER_GET_BASE, FREE_BUFFER, BUFFER_CLEAR, SET_TENSOR,
    SET_TENSOR_HASH, GET_TENSOR, COPY_TENSOR, GRAPH_COMPUTE, GET_DEVICE_MEMORY, INIT_TENSOR, GET_ALLOC_SIZE,
    HELLO, DEVICE_COUNT, GRAPH_RECOMPUTE, SET_TENSOR_GGUF, REGISTER_PEER, PUSH_TENSOR_TO_PEER, PEER_TENSOR_DATA,
    CMD_COUNT
};
constexpr uint8_t PROTO_MAJOR = 4, PROTO_MINOR = 1, PROTO_PATCH = 0;
constexpr size_t CAPS = 24, TSZ = sizeof(b200_tensor);
constexpr uint64_t MAX_PAYLOAD = 1ull << 32; // larger requests are refused and the connection closed

#pragma pack(push, 1)
struct HelloRsp { uint8_t major, minor, patch, padding, caps[CAPS]; };
struct AllocReq { uint32_t device; uint64_t size; };
struct AllocRsp { uint64_t remote_ptr, remote_size; };
struct GetTensorReq { b200_tensor tensor; uint64_t offset, size; };
struct RegisterPeerReq { uint32_t peer_id; char endpoint[128]; };
struct PushReq { uint32_t peer_id; b200_tensor src, dst; uint64_t offset, size; };
struct SetGgufReq { b200_tensor tensor; uint64_t offset; };
struct AllocSizeReq { uint32_t device; b200_tensor tensor; b200_tensor srcs[10]; };
struct CopyReq { b200_tensor src, dst; };
struct ClearReq { uint64_t remote_ptr; uint8_t value; };
struct HashReq { b200_tensor tensor; uint64_t offset, hash; };
#pragma pack(pop)

bool send_all(int fd, const void *p, size_t n) {
    const char *c = (const char *)p;
    while (n > 0) {
        const ssize_t w = send(fd, c, n, MSG_NOSIGNAL);
        if (w <= 0) return false;
        c += w;
        n -= (size_t)w;
    }
    return true;
}
bool recv_all(int fd, void *p, size_t n) {
    char *c = (char *)p;
    while (n > 0) {
        const ssize_t r = recv(fd, c, n, 0);
        if (r <= 0) return false;
        c += r;
        n -= (size_t)r;
    }
    return true;
}
bool send_rsp(int fd, const void *p, uint64_t n) { return send_all(fd, &n, 8) && (n == 0 || send_all(fd, p, (size_t)n)); }

int connect_endpoint(const std::string &ep) {
    const size_t colon = ep.rfind(':');
    if (colon == std::string::npos) return -1;
    const std::string host = ep.substr(0, colon), port = ep.substr(colon + 1);
    struct addrinfo hints = {}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(host.c_str(), port.c_str(), &hints, &res) != 0 || !res) return -1;
    const int fd = socket(res->ai_family, res->ai_socktype, res->ai_protocol);
    if (fd < 0 || connect(fd, res->ai_addr, res->ai_addrlen) != 0) {
        if (fd >= 0) close(fd);
        freeaddrinfo(res);
        return -1;
    }
    freeaddrinfo(res);
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    return fd;
}

} // namespace

struct b200_rpc_server {
    int listen_fd = -1, port = 0;
    std::string host, self_endpoint;
    std::atomic<bool> stopping{false};
    std::thread acceptor;
    std::mutex backend_mutex; // every backend call
    std::mutex conn_mutex;    // the connection table
    std::set<int> conn_fds;
    std::atomic<int> live_threads{0};
    std::set<b200_buffer *> buffers;
    std::map<int, b200_backend *> backends;
    struct Peer { std::string endpoint; int fd = -1; };
    std::map<uint32_t, Peer> peers;
    std::mutex peer_mutex;
    b200_gguf *gguf = nullptr;
    int n_devices = 0;
    struct StoredGraph { std::vector<uint64_t> nodes; std::vector<b200_tensor> tensors; bool valid = false; };
    std::map<uint32_t, StoredGraph> graphs;

    bool live(uint64_t handle) const { return handle != 0 && buffers.count((b200_buffer *)(uintptr_t)handle) != 0; }
    // a tensor record may be used only if it names a live buffer (or none, for an op result placeholder)
    bool tensor_ok(const b200_tensor &t) const { return t.buffer == 0 || live(t.buffer); }
    b200_backend *backend(uint32_t dev) {
        auto it = backends.find((int)dev);
        if (it != backends.end()) return it->second;
        b200_backend *be = nullptr;
        if (b200_backend_init((int)dev, &be) != B200_OK) return nullptr;
        backends[(int)dev] = be;
        return be;
    }
};

namespace {

// returns false when the connection must be closed
bool handle(b200_rpc_server *s, int fd, uint8_t cmd, std::vector<uint8_t> &in) {
    auto need = [&](size_t n) { return in.size() == n; };
    switch (cmd) {
    case HELLO: {
        if (!(in.size() == CAPS || in.empty())) return false;
        HelloRsp r = {PROTO_MAJOR, PROTO_MINOR, PROTO_PATCH, 0, {0}};
        return send_rsp(fd, &r, sizeof(r));
    }
    case DEVICE_COUNT: {
        const uint32_t n = (uint32_t)s->n_devices;
        return send_rsp(fd, &n, 4);
    }
    case GET_ALIGNMENT: {
        if (!need(4)) return false;
        const uint64_t a = b200_buft_alignment();
        return send_rsp(fd, &a, 8);
    }
    case GET_MAX_SIZE: {
        if (!need(4)) return false;
        uint32_t dev;
        memcpy(&dev, in.data(), 4);
        if ((int)dev >= s->n_devices) return false;
        const uint64_t m = b200_buft_max_size((int)dev);
        return send_rsp(fd, &m, 8);
    }
    case GET_DEVICE_MEMORY: {
        if (!need(4)) return false;
        uint32_t dev;
        memcpy(&dev, in.data(), 4);
        if ((int)dev >= s->n_devices) return false;
        size_t fr = 0, tot = 0;
        {
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            if (b200_dev_memory((int)dev, &fr, &tot) != B200_OK) return false;
        }
        const uint64_t r[2] = {fr, tot};
        return send_rsp(fd, r, 16);
    }
    case ALLOC_BUFFER: {
        if (!need(sizeof(AllocReq))) return false;
        AllocReq q;
        memcpy(&q, in.data(), sizeof(q));
        AllocRsp r = {0, 0};
        if ((int)q.device < s->n_devices) {
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            b200_buffer *b = nullptr;
            if (b200_buffer_alloc((int)q.device, (size_t)q.size, &b) == B200_OK && b) {
                s->buffers.insert(b);
                r.remote_ptr = (uint64_t)(uintptr_t)b;
                r.remote_size = b200_buffer_get_size(b);
            }
        }
        return send_rsp(fd, &r, sizeof(r)); // remote_ptr 0 tells the client the allocation failed
    }
    case BUFFER_GET_BASE: {
        if (!need(8)) return false;
        uint64_t h;
        memcpy(&h, in.data(), 8);
        std::lock_guard<std::mutex> lock(s->backend_mutex);
        if (!s->live(h)) return false;
        const uint64_t base = (uint64_t)(uintptr_t)b200_buffer_get_base((b200_buffer *)(uintptr_t)h);
        return send_rsp(fd, &base, 8);
    }
    case FREE_BUFFER: {
        if (!need(8)) return false;
        uint64_t h;
        memcpy(&h, in.data(), 8);
        {
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            if (!s->live(h)) return false;
            s->buffers.erase((b200_buffer *)(uintptr_t)h);
            for (auto &g : s->graphs) g.second.valid = false; // stored graphs may reference it
            b200_buffer_free((b200_buffer *)(uintptr_t)h);
        }
        return send_rsp(fd, nullptr, 0);
    }
    case BUFFER_CLEAR: {
        if (!need(sizeof(ClearReq))) return false;
        ClearReq q;
        memcpy(&q, in.data(), sizeof(q));
        {
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            if (!s->live(q.remote_ptr)) return false;
            if (b200_buffer_clear((b200_buffer *)(uintptr_t)q.remote_ptr, q.value) != B200_OK) return false;
        }
        return send_rsp(fd, nullptr, 0);
    }
    case SET_TENSOR:
    case PEER_TENSOR_DATA: {
        bool ok = in.size() >= TSZ + 8;
        if (ok) {
            b200_tensor t;
            uint64_t off;
            memcpy(&t, in.data(), TSZ);
            memcpy(&off, in.data() + TSZ, 8);
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            ok = s->live(t.buffer) && b200_buffer_set_tensor((b200_buffer *)(uintptr_t)t.buffer, &t, in.data() + TSZ + 8,
                                                             (size_t)off, in.size() - TSZ - 8) == B200_OK;
        }
        if (cmd == PEER_TENSOR_DATA) {
            const uint8_t r = ok ? 1 : 0;
            return send_rsp(fd, &r, 1);
        }
        return ok; // no response; a refused write ends the connection, as an out-of-bounds write does upstream
    }
    case GET_TENSOR: {
        if (!need(sizeof(GetTensorReq))) return false;
        GetTensorReq q;
        memcpy(&q, in.data(), sizeof(q));
        if (q.size > MAX_PAYLOAD) return false;
        std::vector<uint8_t> out((size_t)q.size);
        {
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            if (!s->live(q.tensor.buffer)) return false;
            if (b200_buffer_get_tensor((b200_buffer *)(uintptr_t)q.tensor.buffer, &q.tensor, out.data(), (size_t)q.offset,
                                       (size_t)q.size) != B200_OK)
                return false;
        }
        return send_rsp(fd, out.data(), out.size());
    }
    case COPY_TENSOR: {
        if (!need(sizeof(CopyReq))) return false;
        CopyReq q;
        memcpy(&q, in.data(), sizeof(q));
        uint8_t r = 0;
        {
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            if (!s->live(q.src.buffer) || !s->live(q.dst.buffer)) return false;
            // the tensor's exact byte count (the allocation size is rounded up and would be refused)
            const uint64_t rows = (uint64_t)q.src.ne[1] * q.src.ne[2] * q.src.ne[3];
            const size_t bytes = q.src.type == B200_TYPE_I32 ? (size_t)(rows * q.src.ne[0] * 4)
                                                             : (size_t)(rows * (uint64_t)b200_row_bytes(q.src.type, q.src.ne[0]));
            r = b200_buffer_cpy_tensor(&q.src, &q.dst, 0, bytes) == 1 ? 1 : 0;
        }
        return send_rsp(fd, &r, 1);
    }
    case INIT_TENSOR: {
        if (!need(TSZ)) return false;
        b200_tensor t;
        memcpy(&t, in.data(), TSZ);
        {
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            if (!s->live(t.buffer)) return false;
            if (b200_buffer_init_tensor((b200_buffer *)(uintptr_t)t.buffer, &t) != B200_OK) return false;
        }
        return send_rsp(fd, nullptr, 0);
    }
    case GET_ALLOC_SIZE: {
        if (!need(sizeof(AllocSizeReq))) return false;
        AllocSizeReq *q = (AllocSizeReq *)in.data();
        const uint64_t n = b200_buft_alloc_size(q->tensor.type, q->tensor.ne);
        return send_rsp(fd, &n, 8);
    }
    case SET_TENSOR_HASH: {
        if (!need(sizeof(HashReq))) return false;
        const uint8_t r = 0; // no content cache here: the client sends the bytes with SET_TENSOR
        return send_rsp(fd, &r, 1);
    }
    case SET_TENSOR_GGUF: {
        if (!need(sizeof(SetGgufReq))) return false;
        SetGgufReq q;
        memcpy(&q, in.data(), sizeof(q));
        uint8_t r = 0;
        if (s->gguf) {
            char name[65];
            memcpy(name, q.tensor.name, 64);
            name[64] = 0;
            const int64_t idx = b200_gguf_find_tensor(s->gguf, name);
            b200_gguf_tensor info;
            if (idx >= 0 && b200_gguf_tensor_info(s->gguf, idx, &info) == B200_OK && info.nbytes > 0) {
                std::vector<uint8_t> data((size_t)info.nbytes);
                if (b200_gguf_read_tensor(s->gguf, idx, data.data(), data.size()) == B200_OK) {
                    std::lock_guard<std::mutex> lock(s->backend_mutex);
                    if (s->live(q.tensor.buffer) &&
                        b200_buffer_set_tensor((b200_buffer *)(uintptr_t)q.tensor.buffer, &q.tensor, data.data(),
                                               (size_t)q.offset, data.size()) == B200_OK)
                        r = 1;
                }
            }
        }
        return send_rsp(fd, &r, 1); // 0: not in the local file (or no file) -> the client sends the bytes
    }
    case GRAPH_COMPUTE: {
        if (in.size() < 12) return false;
        uint32_t dev, n_nodes, n_tensors;
        memcpy(&dev, in.data(), 4);
        memcpy(&n_nodes, in.data() + 4, 4);
        const uint64_t after_nodes = 8 + (uint64_t)n_nodes * 8;
        if (in.size() < after_nodes + 4) return false;
        memcpy(&n_tensors, in.data() + after_nodes, 4);
        if (in.size() != after_nodes + 4 + (uint64_t)n_tensors * TSZ || (int)dev >= s->n_devices) return false;
        std::lock_guard<std::mutex> lock(s->backend_mutex);
        b200_rpc_server::StoredGraph &g = s->graphs[dev];
        g.nodes.resize(n_nodes);
        g.tensors.resize(n_tensors);
        memcpy(g.nodes.data(), in.data() + 8, (size_t)n_nodes * 8);
        memcpy(g.tensors.data(), in.data() + after_nodes + 4, (size_t)n_tensors * TSZ);
        g.valid = false;
        for (const b200_tensor &t : g.tensors)
            if (!s->tensor_ok(t)) return false;
        b200_backend *be = s->backend(dev);
        if (!be) return false;
        if (b200_backend_graph_compute(be, g.nodes.data(), n_nodes, g.tensors.data(), n_tensors) != B200_OK) return false;
        if (b200_backend_synchronize(be) != B200_OK) return false;
        g.valid = true;
        return true; // no response
    }
    case GRAPH_RECOMPUTE: {
        if (!need(4)) return false;
        uint32_t dev;
        memcpy(&dev, in.data(), 4);
        std::lock_guard<std::mutex> lock(s->backend_mutex);
        auto it = s->graphs.find(dev);
        if (it == s->graphs.end() || !it->second.valid) return false;
        b200_backend *be = s->backend(dev);
        if (!be) return false;
        if (b200_backend_graph_compute(be, it->second.nodes.data(), (uint32_t)it->second.nodes.size(),
                                       it->second.tensors.data(), (uint32_t)it->second.tensors.size()) != B200_OK)
            return false;
        return b200_backend_synchronize(be) == B200_OK; // no response
    }
    case REGISTER_PEER: {
        if (!need(sizeof(RegisterPeerReq))) return false;
        RegisterPeerReq q;
        memcpy(&q, in.data(), sizeof(q));
        const std::string ep(q.endpoint, strnlen(q.endpoint, sizeof(q.endpoint)));
        const size_t colon = ep.find(':');
        uint8_t r = 0;
        if (!ep.empty() && colon != std::string::npos && colon != 0 && colon != ep.size() - 1) {
            std::lock_guard<std::mutex> lock(s->peer_mutex);
            b200_rpc_server::Peer &p = s->peers[q.peer_id];
            if (p.fd >= 0) close(p.fd);
            p.fd = -1;
            p.endpoint = ep; // the connection is made on first use
            r = 1;
        }
        return send_rsp(fd, &r, 1);
    }
    case PUSH_TENSOR_TO_PEER: {
        if (!need(sizeof(PushReq))) return false;
        PushReq q;
        memcpy(&q, in.data(), sizeof(q));
        uint8_t r = 0;
        std::string ep;
        {
            std::lock_guard<std::mutex> lock(s->peer_mutex);
            auto it = s->peers.find(q.peer_id);
            if (it != s->peers.end()) ep = it->second.endpoint;
        }
        if (ep.empty() || q.size > MAX_PAYLOAD) return send_rsp(fd, &r, 1); // unknown peer: result 0, caller relays
        if (ep == s->self_endpoint) {
            // both tensors live in this process: one device-to-device (NVLink) copy
            std::lock_guard<std::mutex> lock(s->backend_mutex);
            if (s->live(q.src.buffer) && s->live(q.dst.buffer))
                r = b200_buffer_cpy_tensor(&q.src, &q.dst, (size_t)q.offset, (size_t)q.size) == 1 ? 1 : 0;
            return send_rsp(fd, &r, 1);
        }
        std::vector<uint8_t> payload(TSZ + 8 + (size_t)q.size);
        {
            std::lock_guard<std::mutex> lock(s->backend_mutex); // phase A: read from the local device
            if (!s->live(q.src.buffer) ||
                b200_buffer_get_tensor((b200_buffer *)(uintptr_t)q.src.buffer, &q.src, payload.data() + TSZ + 8,
                                       (size_t)q.offset, (size_t)q.size) != B200_OK)
                return send_rsp(fd, &r, 1);
        }
        memcpy(payload.data(), &q.dst, TSZ);
        memcpy(payload.data() + TSZ, &q.offset, 8);
        {
            std::lock_guard<std::mutex> lock(s->peer_mutex); // phase B: send, backend unlocked
            b200_rpc_server::Peer &p = s->peers[q.peer_id];
            if (p.fd < 0) {
                p.fd = connect_endpoint(p.endpoint);
                if (p.fd >= 0) { // version handshake with the peer
                    const uint8_t c = HELLO;
                    const uint64_t n = CAPS;
                    uint8_t caps[CAPS] = {0};
                    uint64_t rn = 0;
                    HelloRsp hr;
                    if (!send_all(p.fd, &c, 1) || !send_all(p.fd, &n, 8) || !send_all(p.fd, caps, CAPS) ||
                        !recv_all(p.fd, &rn, 8) || rn != sizeof(hr) || !recv_all(p.fd, &hr, sizeof(hr)) ||
                        hr.major != PROTO_MAJOR || hr.minor < 1) {
                        close(p.fd);
                        p.fd = -1;
                    }
                }
            }
            if (p.fd >= 0) {
                const uint8_t c = PEER_TENSOR_DATA;
                const uint64_t n = payload.size();
                uint64_t rn = 0;
                uint8_t pr = 0;
                if (send_all(p.fd, &c, 1) && send_all(p.fd, &n, 8) && send_all(p.fd, payload.data(), payload.size()) &&
                    recv_all(p.fd, &rn, 8) && rn == 1 && recv_all(p.fd, &pr, 1)) {
                    r = pr == 1 ? 1 : 0;
                } else {
                    close(p.fd); // stale connection: the next push reconnects
                    p.fd = -1;
                }
            }
        }
        return send_rsp(fd, &r, 1);
    }
    default: return false;
    }
}

void serve(b200_rpc_server *s, int fd) {
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    std::vector<uint8_t> in;
    bool first = true;
    while (!s->stopping.load()) {
        uint8_t cmd;
        uint64_t n;
        if (!recv_all(fd, &cmd, 1)) break;
        if (cmd >= CMD_COUNT || (first && cmd != HELLO)) break; // the handshake comes first
        first = false;
        if (!recv_all(fd, &n, 8) || n > MAX_PAYLOAD) break;
        try {
            in.resize((size_t)n);
        } catch (...) {
            break;
        }
        if (n > 0 && !recv_all(fd, in.data(), (size_t)n)) break;
        if (!handle(s, fd, cmd, in)) break;
    }
    {
        std::lock_guard<std::mutex> lock(s->conn_mutex);
        s->conn_fds.erase(fd);
    }
    close(fd);
    s->live_threads.fetch_sub(1);
}

void accept_loop(b200_rpc_server *s) {
    while (!s->stopping.load()) {
        const int fd = accept(s->listen_fd, nullptr, nullptr);
        if (fd < 0) {
            if (s->stopping.load()) break;
            continue;
        }
        {
            std::lock_guard<std::mutex> lock(s->conn_mutex);
            s->conn_fds.insert(fd);
        }
        s->live_threads.fetch_add(1);
        std::thread(serve, s, fd).detach();
    }
}

} // namespace

b200_status b200_rpc_server_start(const char *host, int32_t port, const char *gguf_path, b200_rpc_server **out) {
    KQ_REQUIRE(out, "rpc_server_start: null argument");
    *out = nullptr;
    std::unique_ptr<b200_rpc_server> s(new b200_rpc_server());
    s->host = host && host[0] ? host : "127.0.0.1";
    s->n_devices = b200_reg_device_count();
    if (gguf_path && gguf_path[0]) {
        const b200_status rc = b200_gguf_open(gguf_path, &s->gguf);
        if (rc != B200_OK) return rc;
    }
    s->listen_fd = socket(AF_INET, SOCK_STREAM, 0);
    KQ_REQUIRE(s->listen_fd >= 0, "rpc_server_start: socket: %s", strerror(errno));
    int one = 1;
    setsockopt(s->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    struct sockaddr_in addr = {};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, s->host.c_str(), &addr.sin_addr) != 1) {
        close(s->listen_fd);
        if (s->gguf) b200_gguf_close(s->gguf);
        kq_set_error("rpc_server_start: %s is not an IPv4 address", s->host.c_str());
        return B200_ERR_INVALID;
    }
    if (bind(s->listen_fd, (struct sockaddr *)&addr, sizeof(addr)) != 0 || listen(s->listen_fd, 64) != 0) {
        kq_set_error("rpc_server_start: cannot listen on %s:%d: %s", s->host.c_str(), port, strerror(errno));
        close(s->listen_fd);
        if (s->gguf) b200_gguf_close(s->gguf);
        return B200_ERR_INVALID;
    }
    socklen_t len = sizeof(addr);
    getsockname(s->listen_fd, (struct sockaddr *)&addr, &len);
    s->port = ntohs(addr.sin_port);
    s->self_endpoint = s->host + ":" + std::to_string(s->port);
    s->acceptor = std::thread(accept_loop, s.get());
    *out = s.release();
    return B200_OK;
}

int32_t b200_rpc_server_port(const b200_rpc_server *s) { return s ? s->port : -1; }

void b200_rpc_server_stop(b200_rpc_server *s) {
    if (!s) return;
    s->stopping.store(true);
    shutdown(s->listen_fd, SHUT_RDWR);
    close(s->listen_fd);
    if (s->acceptor.joinable()) s->acceptor.join();
    {
        std::lock_guard<std::mutex> lock(s->conn_mutex);
        for (int fd : s->conn_fds) shutdown(fd, SHUT_RDWR); // wakes the connection threads
    }
    for (int i = 0; i < 2000 && s->live_threads.load() > 0; i++) usleep(1000);
    {
        std::lock_guard<std::mutex> lock(s->peer_mutex);
        for (auto &p : s->peers)
            if (p.second.fd >= 0) close(p.second.fd);
    }
    {
        std::lock_guard<std::mutex> lock(s->backend_mutex);
        for (b200_buffer *b : s->buffers) b200_buffer_free(b);
        for (auto &be : s->backends) b200_backend_free(be.second);
    }
    if (s->gguf) b200_gguf_close(s->gguf);
    if (s->live_threads.load() == 0) delete s; // a connection thread that did not wake keeps the object alive
}
