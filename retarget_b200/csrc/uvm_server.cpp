// UVM control server: allocation registry, protocol handler, migration worker.
//
// Lock order: life -> state.  `life` serialises allocation lifetime events
// (alloc / free / context teardown) against one in-flight batch of prefetches;
// `state` guards the registry and the counters and is never held across a CUDA
// call.  `status` and `list` take `state` only, so they never wait for a
// migration.
#include <errno.h>
#include <poll.h>
#include <pthread.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "driver_api.h"
#include "rt_internal.h"
#include "uvm_plan.h"

namespace rt {
namespace {

struct Allocation {
    uint64_t id;
    CUdeviceptr ptr;
    uint64_t bytes;
    CUcontext ctx;
    int device;
    int concurrent;
};

struct Server {
    std::mutex control;                  // start / stop, held for the whole call; no thread of the
                                         // server ever takes it, so joining under it cannot deadlock
    std::mutex life;
    std::mutex state;
    std::condition_variable wake;        // worker: a job arrived / stop
    std::condition_variable done;        // waiters: a job completed
    std::vector<Allocation> allocations; // insertion order == id order
    uint64_t next_id = 0, managed_bytes = 0, generation = 0;
    uint64_t job_id = 0, completed_job = 0, job_bytes = 0, cpu_bytes = 0, gpu_bytes = 0;
    int last_error = 0;
    bool busy = false, stop = false, running = false;
    std::vector<rt_id_range> job;
    uint64_t chunk = 16ull << 20, batch = 256ull << 20, page = 4096;
    uint32_t n_streams = 4;
    bool overlap_phases = false;   // run a plan's CPU-bound and GPU-bound stretch at the same time
    std::thread worker, listener;
    int listen_fd = -1, client_fd = -1;
    int stop_fd = -1;                    // eventfd: wakes the listener for a stop
    std::string socket_path;
    dev_t socket_dev = 0;
    ino_t socket_ino = 0;
    pid_t owner = 0;
    // side streams, per context (with the device the context belongs to), used by
    // the worker thread under `life`
    struct SideStreams {
        int device = -1;
        std::vector<CUstream> list;
    };
    std::map<CUcontext, SideStreams> streams;
};

Server g;

uint64_t saturating_add(uint64_t a, uint64_t b) { return b > UINT64_MAX - a ? UINT64_MAX : a + b; }

std::vector<rt_alloc_info> snapshot_locked() {
    std::vector<rt_alloc_info> out;
    out.reserve(g.allocations.size());
    for (const Allocation &a : g.allocations) out.push_back({a.id, a.bytes, a.device, a.concurrent});
    return out;
}

// ---------------------------------------------------------------------------
// executor: one job = ranges in queue order; CPU-bound ranges come first in
// every plan and must have landed before the first GPU-bound one is issued.
// ---------------------------------------------------------------------------
struct Pending {
    uint64_t bytes;
    int dst;
};

CUresult streams_for(const DriverApi &api, CUcontext ctx, int device, std::vector<CUstream> **out) {
    auto it = g.streams.find(ctx);
    if (it == g.streams.end()) {
        Server::SideStreams made_for;
        made_for.device = device;
        std::vector<CUstream> &made = made_for.list;
        for (uint32_t i = 0; i < g.n_streams; ++i) {
            CUstream s = nullptr;
            CUresult r = api.stream_create(&s, CU_STREAM_NON_BLOCKING);
            if (r != CUDA_SUCCESS) {
                for (CUstream m : made) api.stream_destroy(m);
                return r;
            }
            made.push_back(s);
        }
        it = g.streams.emplace(ctx, std::move(made_for)).first;
    }
    *out = &it->second.list;
    return CUDA_SUCCESS;
}

// Forgets the side streams of the contexts of `device` (any device when < 0).
// `alive`: the contexts still exist, so the streams are destroyed properly;
// otherwise they went away with their context and only the handles are dropped.
// Caller holds `life`.
void drop_streams_locked(int device, bool alive) {
    const DriverApi *api = alive ? driver_api() : nullptr;
    for (auto it = g.streams.begin(); it != g.streams.end();) {
        if (device >= 0 && it->second.device != device) {
            ++it;
            continue;
        }
        if (api && api->ctx_set_current && api->stream_destroy && api->ctx_set_current(it->first) == CUDA_SUCCESS) {
            for (CUstream s : it->second.list) api->stream_destroy(s);
            api->ctx_set_current(nullptr);
        }
        it = g.streams.erase(it);
    }
}

// A stretch of the job that moves in one direction: ranges [range, end), `done`
// bytes of the first one already issued.
struct Lane {
    size_t range, end;
    uint64_t done;
    bool finished() const { return range >= end; }
};

// Issues up to `batch` bytes, taking chunks from the lanes in turn, and waits for
// them.  One lane: the job's queue order.  Two lanes (overlapped phases): the
// CPU-bound and the GPU-bound stretch advance together, each on its own share of
// the side streams, so that both directions of the host link are busy at once.
// Holds `life` for the whole batch so that no allocation can be freed under a
// queued prefetch.
CUresult run_batch(const DriverApi &api, const std::vector<rt_id_range> &job, Lane *lanes, uint32_t n_lanes) {
    std::lock_guard<std::mutex> life(g.life);
    std::vector<Pending> pending;
    std::vector<CUstream> used;
    CUcontext current = nullptr;
    bool have_ctx = false;
    CUresult result = CUDA_SUCCESS;
    uint64_t issued = 0;
    uint32_t rr[2] = {0, 0};
    bool progressed = true;
    while (progressed && issued < g.batch && result == CUDA_SUCCESS) {
        progressed = false;
        for (uint32_t k = 0; k < n_lanes && issued < g.batch && result == CUDA_SUCCESS; ++k) {
            Lane &lane = lanes[k];
            if (lane.finished()) continue;
            const rt_id_range &r = job[lane.range];
            CUdeviceptr ptr = 0;
            CUcontext ctx = nullptr;
            int device = -1;
            bool found = false, stopping;
            {
                std::lock_guard<std::mutex> st(g.state);
                for (const Allocation &a : g.allocations)
                    if (a.id == r.id) { ptr = a.ptr + r.offset + lane.done; ctx = a.ctx; device = a.device; found = true; break; }
                stopping = g.stop;
            }
            if (stopping) { result = CUDA_ERROR_DEINITIALIZED; break; }
            if (!found) { result = CUDA_ERROR_INVALID_VALUE; break; }
            if (have_ctx && ctx != current) continue;         // one context per batch: this lane waits for the next
            if (!have_ctx) {
                result = api.ctx_set_current(ctx);
                if (result != CUDA_SUCCESS) break;
                current = ctx;
                have_ctx = true;
            }
            std::vector<CUstream> *streams = nullptr;
            result = streams_for(api, ctx, device, &streams);
            if (result != CUDA_SUCCESS) break;
            uint64_t bytes = r.bytes - lane.done;
            if (bytes > g.chunk) bytes = g.chunk;
            // lane k of n takes every n-th side stream (all of them when it is alone)
            const size_t share = streams->size() >= n_lanes ? streams->size() / n_lanes : 1;
            CUstream s = (*streams)[(k * share + rr[k]++ % share) % streams->size()];
            result = api.prefetch(ptr, bytes, r.dst, s);
            if (result != CUDA_SUCCESS) break;
            bool seen = false;
            for (CUstream u : used) seen |= u == s;
            if (!seen) used.push_back(s);
            pending.push_back({bytes, r.dst});
            issued += bytes;
            lane.done += bytes;
            if (lane.done == r.bytes) { ++lane.range; lane.done = 0; }
            progressed = true;
        }
    }
    for (CUstream s : used) {
        CUresult r = api.stream_synchronize(s);
        if (result == CUDA_SUCCESS) result = r;
    }
    if (have_ctx) {
        // the worker owns its thread's context binding; never leave one behind
        CUresult r = api.ctx_set_current(nullptr);
        if (result == CUDA_SUCCESS) result = r;
    }
    if (result == CUDA_SUCCESS) {
        std::lock_guard<std::mutex> st(g.state);
        for (const Pending &p : pending) {
            g.job_bytes = saturating_add(g.job_bytes, p.bytes);
            uint64_t &side = p.dst < 0 ? g.cpu_bytes : g.gpu_bytes;
            side = saturating_add(side, p.bytes);
        }
    }
    return result;
}

// Runs one job.  The ranges are cut into stretches of one direction; a stretch
// has completed before the next one starts, which is the reference's order
// (every CPU-bound range has landed before the first GPU-bound one is issued,
// select.cpp:24231-24240 builds the list that way and 23990-24024 runs it in
// order).  With `overlap_phases` a job of exactly one CPU-bound stretch followed
// by one GPU-bound stretch -- every plan the protocol can express -- runs both
// at once.
CUresult run_job(const DriverApi &api, const std::vector<rt_id_range> &job, bool overlap) {
    std::vector<Lane> stretches;
    for (size_t i = 0; i < job.size(); ++i) {
        if (stretches.empty() || (job[i].dst < 0) != (job[stretches.back().range].dst < 0))
            stretches.push_back({i, i + 1, 0});
        else
            stretches.back().end = i + 1;
    }
    CUresult result = CUDA_SUCCESS;
    if (overlap && stretches.size() == 2 && job[stretches[0].range].dst < 0) {
        Lane both[2] = {stretches[0], stretches[1]};
        while (result == CUDA_SUCCESS && !(both[0].finished() && both[1].finished()))
            result = run_batch(api, job, both, 2);
        return result;
    }
    for (Lane &lane : stretches)
        while (result == CUDA_SUCCESS && !lane.finished()) result = run_batch(api, job, &lane, 1);
    return result;
}

void worker_main() {
    const DriverApi *api = driver_api();
    std::unique_lock<std::mutex> st(g.state);
    for (;;) {
        g.wake.wait(st, [] { return g.busy || g.stop; });
        if (g.stop && !g.busy) break;
        std::vector<rt_id_range> job;
        job.swap(g.job);
        const bool overlap = g.overlap_phases;
        st.unlock();
        CUresult result = api ? run_job(*api, job, overlap) : CUDA_ERROR_NOT_INITIALIZED;
        st.lock();
        g.last_error = (int)result;
        g.completed_job = g.job_id;
        g.busy = false;
        g.done.notify_all();
        if (g.stop) break;
    }
}

}  // namespace

namespace {

// ---------------------------------------------------------------------------
// protocol: one line in, one JSON line out (select.cpp:24045-24327)
// ---------------------------------------------------------------------------
std::string error_reply(const char *error) {
    return std::string("{\"ok\":false,\"error\":\"") + error + "\"}";
}

std::string status_reply_locked() {
    char buf[640];
    snprintf(buf, sizeof(buf),
             "{\"ok\":true,\"pid\":%ld,\"managed_bytes\":%llu,\"allocation_count\":%llu,"
             "\"allocation_generation\":%llu,\"busy\":%s,\"job_id\":%llu,"
             "\"completed_job\":%llu,\"last_error\":%d,"
             "\"completed_cpu_bytes\":%llu,\"completed_gpu_bytes\":%llu,\"job_completed_bytes\":%llu}",
             (long)g.owner, (unsigned long long)g.managed_bytes,
             (unsigned long long)g.allocations.size(), (unsigned long long)g.generation,
             g.busy ? "true" : "false", (unsigned long long)g.job_id,
             (unsigned long long)g.completed_job, g.last_error, (unsigned long long)g.cpu_bytes,
             (unsigned long long)g.gpu_bytes, (unsigned long long)g.job_bytes);
    return buf;
}

std::string list_reply_locked() {
    std::string out = "{\"ok\":true,\"allocation_generation\":" + std::to_string(g.generation) +
                      ",\"allocations\":[";
    bool first = true;
    for (const Allocation &a : g.allocations) {
        char item[128];
        snprintf(item, sizeof(item), "%s{\"id\":%llu,\"bytes\":%llu,\"device\":%d}", first ? "" : ",",
                 (unsigned long long)a.id, (unsigned long long)a.bytes, a.device);
        out += item;
        first = false;
    }
    return out + "]}";
}

bool single_word(const char *line, const char *word) {
    while (*line == ' ' || *line == '\t' || *line == '\r') ++line;
    size_t n = strlen(word);
    if (strncmp(line, word, n)) return false;
    line += n;
    while (*line == ' ' || *line == '\t' || *line == '\r') ++line;
    return !*line;
}

// Accepts the job under `state` (caller holds it): the admission checks of
// select.cpp:24131-24135 in their order.
const char *admit_locked(std::vector<rt_id_range> &ranges, uint64_t *accepted) {
    const DriverApi *api = driver_api();
    if (g.busy) return "busy";
    if (g.stop) return "stopping";
    if (!g.running || !api || !api->can_prefetch()) return "not_supported";
    if (g.job_id == UINT64_MAX) return "job_id_exhausted";
    (void)ranges;
    (void)accepted;
    return nullptr;
}

void publish_locked(std::vector<rt_id_range> &ranges, uint64_t *accepted) {
    g.job.swap(ranges);
    g.busy = true;
    g.job_bytes = 0;
    g.last_error = 0;
    *accepted = ++g.job_id;
    g.wake.notify_one();
}

std::string handle_line(const char *line) {
    if (single_word(line, "status")) {
        std::lock_guard<std::mutex> st(g.state);
        return status_reply_locked();
    }
    if (single_word(line, "list")) {
        std::lock_guard<std::mutex> st(g.state);
        return list_reply_locked();
    }
    // Syntax errors are reported before the admission checks, plan errors after
    // them, exactly as the reference orders them: parse once against an empty
    // registry to classify.
    std::vector<rt_id_range> ranges;
    {
        std::vector<rt_id_range> scratch;
        const char *syntax = expand_plan_line(nullptr, 0, 0, line, g.page, scratch);
        if (syntax && !strcmp(syntax, "invalid_command")) return error_reply("invalid_command");
    }
    uint64_t accepted = 0;
    {
        std::lock_guard<std::mutex> st(g.state);
        if (const char *why = admit_locked(ranges, &accepted)) return error_reply(why);
        std::vector<rt_alloc_info> reg = snapshot_locked();
        if (const char *why = expand_plan_line(reg.data(), reg.size(), g.generation, line, g.page, ranges))
            return error_reply(why);
        publish_locked(ranges, &accepted);
    }
    return "{\"ok\":true,\"job_id\":" + std::to_string(accepted) + "}";
}

// ---------------------------------------------------------------------------
// control socket (the protocol of select.cpp:24330-24445): one command per
// connection, one JSON line back
// ---------------------------------------------------------------------------
// The listener thread sleeps in poll() on the listening socket and on an
// eventfd that rt_uvm_stop() writes to, so it neither wakes up periodically nor
// needs a connection shut down under it to notice a stop.  A connection is
// served against ONE deadline (a second, as the protocol allows a client) that
// covers reading the line and writing the reply; the line is collected from
// whatever recv() returns, not byte by byte.

double monotonic_now() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

enum class Ready { yes, stop, timeout, error };

// Sleeps until `fd` is ready for `events`, the stop event fires or the deadline
// passes (deadline < 0: no deadline).
Ready wait_fd(int fd, short events, int stop_fd, double deadline) {
    for (;;) {
        int ms = -1;
        if (deadline >= 0) {
            const double left = deadline - monotonic_now();
            if (left <= 0) return Ready::timeout;
            ms = (int)(left * 1e3) + 1;
        }
        pollfd fds[2] = {{fd, events, 0}, {stop_fd, POLLIN, 0}};
        const int n = poll(fds, 2, ms);
        if (n < 0) {
            if (errno == EINTR) continue;
            return Ready::error;
        }
        if (fds[1].revents) return Ready::stop;
        if (fds[0].revents) return Ready::yes;
    }
}

constexpr size_t kLineBytes = 512;              // a command is shorter than this, terminator included

enum class Line { ok, invalid };

// One '\n'-terminated command without NUL bytes, shorter than kLineBytes.
// Anything else -- end of stream, a stalled or over-long line, a NUL -- is
// `invalid` (the protocol's invalid_line).
Line read_line(int fd, int stop_fd, double deadline, std::string *line) {
    char buf[kLineBytes];
    size_t used = 0;
    while (used + 1 < sizeof(buf)) {
        const ssize_t n = recv(fd, buf + used, sizeof(buf) - 1 - used, MSG_DONTWAIT);
        if (n > 0) {
            const char *chunk = buf + used;
            const char *nl = static_cast<const char *>(memchr(chunk, '\n', (size_t)n));
            const size_t fresh = nl ? (size_t)(nl - chunk) : (size_t)n;
            if (memchr(chunk, 0, fresh)) return Line::invalid;
            used += fresh;
            if (nl) {
                line->assign(buf, used);
                return Line::ok;
            }
        } else if (n == 0) {
            return Line::invalid;
        } else if (errno == EAGAIN || errno == EWOULDBLOCK) {
            if (wait_fd(fd, POLLIN, stop_fd, deadline) != Ready::yes) return Line::invalid;
        } else if (errno != EINTR) {
            return Line::invalid;
        }
    }
    return Line::invalid;
}

void write_reply(int fd, int stop_fd, double deadline, const std::string &text) {
    size_t sent = 0;
    while (sent < text.size()) {
        const ssize_t n = send(fd, text.data() + sent, text.size() - sent, MSG_NOSIGNAL | MSG_DONTWAIT);
        if (n > 0) sent += (size_t)n;
        else if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) {
            if (wait_fd(fd, POLLOUT, stop_fd, deadline) != Ready::yes) return;
        } else if (n < 0 && errno == EINTR) continue;
        else return;
    }
}

bool peer_is_us(int fd) {
    ucred peer;
    socklen_t size = sizeof(peer);
    return getsockopt(fd, SOL_SOCKET, SO_PEERCRED, &peer, &size) == 0 && size == sizeof(peer) &&
           peer.uid == getuid();
}

void serve_connection(int fd, int stop_fd) {
    if (!peer_is_us(fd)) return;                // another user's process gets no answer at all
    const double deadline = monotonic_now() + 1.0;
    std::string line;
    const std::string reply = read_line(fd, stop_fd, deadline, &line) == Line::ok ? handle_line(line.c_str())
                                                                                   : error_reply("invalid_line");
    write_reply(fd, stop_fd, deadline, reply + "\n");
}

void listener_main(int listen_fd, int stop_fd) {
    while (wait_fd(listen_fd, POLLIN, stop_fd, -1) == Ready::yes) {
        const int fd = accept4(listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd < 0) continue;
        {
            std::lock_guard<std::mutex> st(g.state);
            g.client_fd = fd;                   // the fork handler closes it in a child
        }
        serve_connection(fd, stop_fd);
        std::lock_guard<std::mutex> st(g.state);
        g.client_fd = -1;
        close(fd);
    }
}

// The socket file belongs to us only if WE created it: bind() fails on a path
// that exists, and nothing here ever removes a path first (a socket left behind
// by a dead process with the same PID is somebody else's to clean up).  What
// was created is remembered by device and inode and removed only while the
// path still names that very file.
void unlink_owned_socket() {
    std::string path;
    dev_t dev;
    ino_t ino;
    {
        std::lock_guard<std::mutex> lock(g.state);
        path = g.socket_path;
        dev = g.socket_dev;
        ino = g.socket_ino;
        g.socket_ino = 0;
    }
    struct stat now;
    if (!ino || lstat(path.c_str(), &now) != 0) return;
    if (S_ISSOCK(now.st_mode) && now.st_uid == getuid() && now.st_dev == dev && now.st_ino == ino)
        unlink(path.c_str());
}

int open_socket(const char *requested) {
    std::string path = requested ? requested
                                 : "/tmp/select-uvm-" + std::to_string((unsigned long)getuid()) + "-" +
                                       std::to_string((long)getpid()) + ".sock";
    sockaddr_un address = {};
    address.sun_family = AF_UNIX;
    if (path.size() >= sizeof(address.sun_path)) return RT_ERR_INVALID_ARGUMENT;
    memcpy(address.sun_path, path.c_str(), path.size() + 1);
    const int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
    if (fd < 0) return RT_ERR_IO;
    struct stat made;
    if (bind(fd, reinterpret_cast<sockaddr *>(&address), sizeof(address)) != 0 || lstat(path.c_str(), &made) != 0) {
        close(fd);
        return RT_ERR_IO;
    }
    {
        std::lock_guard<std::mutex> lock(g.state);    // status readers look at these under `state`
        g.socket_path = path;
        g.socket_dev = made.st_dev;
        g.socket_ino = made.st_ino;
    }
    const int stop_fd = eventfd(0, EFD_CLOEXEC | EFD_NONBLOCK);
    if (stop_fd < 0 || chmod(path.c_str(), 0600) != 0 || listen(fd, 16) != 0) {
        if (stop_fd >= 0) close(stop_fd);
        close(fd);
        unlink_owned_socket();
        return RT_ERR_IO;
    }
    std::lock_guard<std::mutex> lock(g.state);
    g.listen_fd = fd;
    g.stop_fd = stop_fd;
    return RT_OK;
}

}  // namespace
}  // namespace rt

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
using rt::g;

extern "C" {

int rt_uvm_start(const rt_uvm_config *config) {
    std::lock_guard<std::mutex> control(g.control);
    {
        std::lock_guard<std::mutex> st(g.state);
        if (g.running) return RT_ERR_BUSY;
    }
    rt_uvm_config cfg = {};
    if (config) cfg = *config;
    uint64_t chunk = cfg.chunk_bytes;
    if (!chunk) {
        // SELECT_UVM_CHUNK_MB: 1..256, default 16 MiB (select.cpp:23794,23853-23856)
        chunk = 16ull << 20;
        uint64_t mb = 0;
        const char *s = getenv("SELECT_UVM_CHUNK_MB");
        if (s && rt::parse_u64(s, strlen(s), &mb) && mb >= 1 && mb <= 256) chunk = mb << 20;
    }
    long page = sysconf(_SC_PAGESIZE);
    {
        // callers of the other entry points may be running while the server
        // restarts: everything they read changes under the locks they hold
        std::lock_guard<std::mutex> life(g.life);
        std::lock_guard<std::mutex> st(g.state);
        g.page = page > 0 ? (uint64_t)page : 4096;
        g.chunk = chunk;
        g.batch = cfg.batch_bytes ? cfg.batch_bytes : (256ull << 20);
        if (g.batch < g.chunk) g.batch = g.chunk;
        g.n_streams = cfg.streams ? cfg.streams : 4;
        g.overlap_phases = cfg.overlap_phases != 0;
        g.owner = getpid();
        g.stop = false;
        g.listen_fd = -1;
        g.stop_fd = -1;
        g.socket_path.clear();
    }
    if (cfg.listen) {
        int st = rt::open_socket(cfg.socket_path);
        if (st != RT_OK) return st;
    }
    g.worker = std::thread(rt::worker_main);
    int listen_fd, stop_fd;
    {
        std::lock_guard<std::mutex> st(g.state);
        listen_fd = g.listen_fd;
        stop_fd = g.stop_fd;
    }
    if (listen_fd >= 0) g.listener = std::thread(rt::listener_main, listen_fd, stop_fd);
    std::lock_guard<std::mutex> st(g.state);
    g.running = true;
    return RT_OK;
}

int rt_uvm_stop(void) {
    std::lock_guard<std::mutex> control(g.control);
    {
        std::lock_guard<std::mutex> st(g.state);
        if (!g.running) return RT_ERR_NOT_RUNNING;
        g.stop = true;
        if (g.stop_fd >= 0) {
            const uint64_t one = 1;                    // wakes the listener wherever it sleeps
            if (write(g.stop_fd, &one, sizeof(one)) < 0) { /* the counter is saturated: it is awake */ }
        }
        g.wake.notify_all();
    }
    if (g.listener.joinable()) g.listener.join();
    if (g.worker.joinable()) g.worker.join();
    rt::unlink_owned_socket();
    std::lock_guard<std::mutex> life(g.life);
    std::lock_guard<std::mutex> st(g.state);
    if (g.listen_fd >= 0) close(g.listen_fd);
    if (g.stop_fd >= 0) close(g.stop_fd);
    g.listen_fd = g.stop_fd = -1;
    g.running = false;
    g.busy = false;
    g.job.clear();
    rt::drop_streams_locked(-1, true);       // the contexts live on: give their streams back
    g.done.notify_all();
    return RT_OK;
}

int rt_uvm_register(uint64_t ptr, uint64_t bytes, void *ctx, int device, int concurrent, uint64_t *id) {
    if (!bytes) return RT_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> life(g.life);
    std::lock_guard<std::mutex> st(g.state);
    rt::Allocation a = {++g.next_id, (CUdeviceptr)ptr, bytes, (CUcontext)ctx, device, concurrent};
    g.allocations.push_back(a);
    g.managed_bytes += bytes;
    ++g.generation;
    if (id) *id = a.id;
    return RT_OK;
}

static int remove_where(bool (*match)(const rt::Allocation &, const void *), const void *key) {
    std::lock_guard<std::mutex> life(g.life);
    std::lock_guard<std::mutex> st(g.state);
    size_t kept = 0, removed = 0;
    for (size_t i = 0; i < g.allocations.size(); ++i) {
        if (match(g.allocations[i], key)) {
            g.managed_bytes -= g.allocations[i].bytes;
            ++removed;
        } else {
            g.allocations[kept++] = g.allocations[i];
        }
    }
    g.allocations.resize(kept);
    if (removed) ++g.generation;
    return (int)removed;
}

int rt_uvm_unregister_ptr(uint64_t ptr) {
    return remove_where([](const rt::Allocation &a, const void *k) { return a.ptr == *(const CUdeviceptr *)k; },
                        &ptr);
}

int rt_uvm_unregister_ctx(void *ctx) {
    int n = remove_where([](const rt::Allocation &a, const void *k) { return (const void *)a.ctx == k; }, ctx);
    std::lock_guard<std::mutex> life(g.life);
    g.streams.erase((CUcontext)ctx);
    return n;
}

int rt_uvm_unregister_device(int device) {
    // conservative, like the reference (select.cpp:23894-23913): everything on
    // the device goes, explicit-context records included
    int n = remove_where([](const rt::Allocation &a, const void *k) { return a.device == *(const int *)k; },
                         &device);
    // (the caller says the device's contexts are gone: nothing left to destroy)
    std::lock_guard<std::mutex> life(g.life);
    rt::drop_streams_locked(device, false);
    return n;
}

int rt_uvm_command(const char *line, char *reply, size_t cap) {
    if (!line || !reply || !cap) return RT_ERR_INVALID_ARGUMENT;
    std::string text;
    if (strlen(line) >= 512 || strchr(line, '\n')) text = rt::error_reply("invalid_line");
    else text = rt::handle_line(line);
    if (text.size() + 1 > cap) return RT_ERR_CAPACITY;
    memcpy(reply, text.c_str(), text.size() + 1);
    return (int)text.size();
}

int rt_uvm_submit_ranges(const rt_range *ranges, size_t n, const uint64_t *buffer_ids, size_t n_ids,
                         uint64_t *job_id) {
    if ((!ranges && n) || (!buffer_ids && n_ids) || !job_id) return RT_ERR_INVALID_ARGUMENT;
    std::vector<rt_id_range> job;
    job.reserve(n);
    for (size_t i = 0; i < n; ++i) {
        if (ranges[i].buffer >= n_ids) return RT_ERR_INVALID_ARGUMENT;
        if (!ranges[i].bytes) continue;
        job.push_back({buffer_ids[ranges[i].buffer], ranges[i].offset, ranges[i].bytes, ranges[i].dst, 0});
    }
    std::lock_guard<std::mutex> st(g.state);
    uint64_t accepted = 0;
    if (const char *why = rt::admit_locked(job, &accepted))
        return !strcmp(why, "busy") ? RT_ERR_BUSY : RT_ERR_NOT_RUNNING;
    // the same bounds the text commands enforce, against the live registry
    for (const rt_id_range &r : job) {
        const rt::Allocation *a = nullptr;
        for (const rt::Allocation &x : g.allocations)
            if (x.id == r.id) { a = &x; break; }
        if (!a || r.offset >= a->bytes || r.bytes > a->bytes - r.offset || r.offset % g.page ||
            (r.bytes % g.page && r.bytes != a->bytes - r.offset) || !a->concurrent)
            return RT_ERR_INVALID_ARGUMENT;
    }
    rt::publish_locked(job, &accepted);
    *job_id = accepted;
    return RT_OK;
}

int rt_uvm_wait(uint64_t job_id, double timeout_s, int *cuda_error) {
    std::unique_lock<std::mutex> st(g.state);
    auto ready = [&] { return !g.running || (!g.busy && g.completed_job >= job_id); };
    if (timeout_s < 0) {
        g.done.wait(st, ready);
    } else if (!g.done.wait_for(st, std::chrono::duration<double>(timeout_s), ready)) {
        return RT_ERR_BUSY;
    }
    if (!g.running) return RT_ERR_NOT_RUNNING;
    if (cuda_error) *cuda_error = g.last_error;
    return g.last_error ? RT_ERR_CUDA : RT_OK;
}

int rt_uvm_socket_path(char *out, size_t cap) {
    if (!out || !cap) return RT_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> st(g.state);
    if (g.socket_path.size() + 1 > cap) return RT_ERR_CAPACITY;
    memcpy(out, g.socket_path.c_str(), g.socket_path.size() + 1);
    return (int)g.socket_path.size();
}

}  // extern "C"

// ---------------------------------------------------------------------------
// driver-call wrappers for the preload hooks
// ---------------------------------------------------------------------------
#include "uvm_server.h"

namespace rt {

CUresult uvm_tracked_alloc(CUdeviceptr *dptr, size_t bytes, unsigned int flags) {
    const DriverApi *api = driver_api();
    if (!api || !api->mem_alloc_managed) return CUDA_ERROR_NOT_SUPPORTED;
    if (!dptr || !bytes) return CUDA_ERROR_INVALID_VALUE;
    Allocation a = {};
    std::lock_guard<std::mutex> life(g.life);
    CUresult result = api->ctx_get_current ? api->ctx_get_current(&a.ctx) : CUDA_ERROR_NOT_SUPPORTED;
    if (result == CUDA_SUCCESS && !a.ctx) result = CUDA_ERROR_INVALID_CONTEXT;
    if (result == CUDA_SUCCESS)
        result = api->ctx_get_device ? api->ctx_get_device(&a.device) : CUDA_ERROR_NOT_SUPPORTED;
    if (result == CUDA_SUCCESS)
        result = api->device_get_attribute
                     ? api->device_get_attribute(&a.concurrent, CU_DEVICE_ATTRIBUTE_CONCURRENT_MANAGED_ACCESS,
                                                 a.device)
                     : CUDA_ERROR_NOT_SUPPORTED;
    {
        std::lock_guard<std::mutex> st(g.state);
        if (result == CUDA_SUCCESS && (g.next_id == UINT64_MAX || bytes > UINT64_MAX - g.managed_bytes))
            result = CUDA_ERROR_OUT_OF_MEMORY;
    }
    if (result == CUDA_SUCCESS) result = api->mem_alloc_managed(dptr, bytes, flags);
    if (result != CUDA_SUCCESS) return result;
    a.ptr = *dptr;
    a.bytes = bytes;
    std::lock_guard<std::mutex> st(g.state);
    a.id = ++g.next_id;
    g.allocations.push_back(a);
    g.managed_bytes += bytes;
    ++g.generation;
    return CUDA_SUCCESS;
}

static uint64_t forget_locked(bool (*match)(const Allocation &, const void *), const void *key) {
    std::lock_guard<std::mutex> st(g.state);
    size_t kept = 0;
    uint64_t removed = 0;
    for (size_t i = 0; i < g.allocations.size(); ++i) {
        if (match(g.allocations[i], key)) {
            g.managed_bytes -= g.allocations[i].bytes;
            ++removed;
        } else {
            g.allocations[kept++] = g.allocations[i];
        }
    }
    g.allocations.resize(kept);
    if (removed) ++g.generation;
    return removed;
}

CUresult uvm_tracked_free(CUdeviceptr dptr) {
    const DriverApi *api = driver_api();
    if (!api || !api->mem_free) return CUDA_ERROR_NOT_SUPPORTED;
    std::lock_guard<std::mutex> life(g.life);
    CUresult result = api->mem_free(dptr);
    if (result == CUDA_SUCCESS)
        forget_locked([](const Allocation &a, const void *k) { return a.ptr == *(const CUdeviceptr *)k; }, &dptr);
    return result;
}

CUresult uvm_tracked_ctx_destroy(CUcontext ctx) {
    const DriverApi *api = driver_api();
    if (!api || !api->ctx_destroy) return CUDA_ERROR_NOT_SUPPORTED;
    std::lock_guard<std::mutex> life(g.life);
    CUresult result = api->ctx_destroy(ctx);
    if (result == CUDA_SUCCESS && ctx) {
        forget_locked([](const Allocation &a, const void *k) { return (const void *)a.ctx == k; }, ctx);
        g.streams.erase(ctx);                // they went away with the context
    }
    return result;
}

CUresult uvm_tracked_primary(CUdevice device, CUresult (*real)(CUdevice), const char *name) {
    if (!real) return CUDA_ERROR_NOT_SUPPORTED;
    const bool is_reset = strstr(name, "Reset") != nullptr;
    uint64_t removed = 0;
    CUresult result;
    {
        std::lock_guard<std::mutex> life(g.life);
        result = real(device);
        if (result == CUDA_SUCCESS) {
            removed = forget_locked([](const Allocation &a, const void *k) { return a.device == *(const int *)k; },
                                    &device);
            // Side streams of THIS device only.  A reset destroys the context and
            // its streams with it; a release usually leaves the context alive (other
            // holders), and then its streams are destroyed properly instead of
            // being leaked and made anew by the next job.
            const DriverApi *api = driver_api();
            unsigned int flags = 0;
            int active = 0;
            const bool alive = !is_reset && api && api->primary_get_state &&
                               api->primary_get_state(device, &flags, &active) == CUDA_SUCCESS && active;
            drop_streams_locked((int)device, alive);
        }
    }
    if (removed)
        fprintf(stderr,
                "retarget_b200 UVM: %s succeeded on device %d; conservatively dropped %llu allocation "
                "records (a release may leave the context alive).\n",
                name, device, (unsigned long long)removed);
    return result;
}

void uvm_fork_child() {
    // no mutex and no CUDA call is safe here; the path still belongs to the parent
    if (g.listen_fd >= 0) close(g.listen_fd);
    if (g.client_fd >= 0) close(g.client_fd);
    if (g.stop_fd >= 0) close(g.stop_fd);
    g.listen_fd = g.client_fd = g.stop_fd = -1;
}

}  // namespace rt
