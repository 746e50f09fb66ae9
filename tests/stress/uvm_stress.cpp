// Concurrency stress for the UVM control server and the prefetch executor,
// meant to run under ThreadSanitizer or AddressSanitizer on a CPU-only host.
//
//   uvm_stress <path of the stub libcuda> <socket path> [seconds]
//
// Threads hammer every entry into the server at once, the way a serving process
// does: an "application" thread registers and frees managed allocations, two
// socket clients send status / list / plan lines, an in-process caller submits
// planner ranges and waits for jobs, and the main thread stops and restarts the
// server in between.  The lock order under test is the reference's:
// life -> state, CUDA calls under life only, status/list never take life
// (select.cpp:23750-23754).  Replies are checked for shape only; any reply the
// protocol allows (busy, stale_allocations, ...) is fine.  Exit code 0 = no
// crash and no malformed reply; the sanitizer adds its own verdict.
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "retarget_b200.h"

// The host sources are linked without the CUDA half of the library.
namespace rt {
int last_cuda_error_get() { return 0; }
}  // namespace rt

namespace {

std::atomic<bool> g_stop{false};
std::atomic<int> g_bad{0};
std::atomic<long> g_commands{0}, g_jobs{0}, g_allocs{0};
const char *g_socket = nullptr;
constexpr uint64_t kMiB = 1ull << 20;

void bad(const char *what, const std::string &detail) {
    fprintf(stderr, "uvm_stress: %s: %s\n", what, detail.c_str());
    g_bad.fetch_add(1);
}

bool well_formed(const std::string &reply) {
    return reply.size() >= 2 && reply.front() == '{' && reply.back() == '}' &&
           reply.find("\"ok\":") != std::string::npos;
}

unsigned long long field(const std::string &reply, const char *name) {
    std::string key = std::string("\"") + name + "\":";
    size_t at = reply.find(key);
    return at == std::string::npos ? 0ull : strtoull(reply.c_str() + at + key.size(), nullptr, 10);
}

// One command per connection, as the reference's client does (control.py:427-460).
bool socket_command(const std::string &line, std::string *reply) {
    int fd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (fd < 0) return false;
    sockaddr_un addr{};
    addr.sun_family = AF_UNIX;
    snprintf(addr.sun_path, sizeof(addr.sun_path), "%s", g_socket);
    if (connect(fd, reinterpret_cast<sockaddr *>(&addr), sizeof(addr)) != 0) {
        close(fd);
        return false;                       // server between stop and start
    }
    std::string out = line + "\n";
    // the server may stop between connect and write: no SIGPIPE, just a failed command
    bool ok = send(fd, out.data(), out.size(), MSG_NOSIGNAL) == (ssize_t)out.size();
    reply->clear();
    char buf[4096];
    while (ok) {
        ssize_t n = read(fd, buf, sizeof(buf));
        if (n <= 0) break;
        reply->append(buf, (size_t)n);
    }
    close(fd);
    while (!reply->empty() && (reply->back() == '\n' || reply->back() == '\r')) reply->pop_back();
    return ok && !reply->empty();
}

std::string local_command(const std::string &line) {
    std::vector<char> buf(1 << 20);
    int n = rt_uvm_command(line.c_str(), buf.data(), buf.size());
    return n > 0 ? std::string(buf.data(), (size_t)n) : std::string();
}

// Registers and frees allocations of a few sizes; keeps at most 24 alive.
void app_thread() {
    std::vector<uint64_t> live;
    uint64_t next = 0x7f1000000000ull;
    unsigned seed = 1;
    while (!g_stop.load()) {
        seed = seed * 1103515245u + 12345u;
        if (live.size() < 24 && (live.size() < 4 || (seed >> 16) % 3)) {
            uint64_t bytes = ((seed >> 8) % 4 == 0 ? 6 : 32) * kMiB;
            uint64_t id = 0;
            int st = rt_uvm_register(next, bytes, nullptr, 0, 1, &id);
            if (st == RT_OK) {
                live.push_back(next);
                g_allocs.fetch_add(1);
            } else if (st != RT_ERR_NOT_RUNNING) {
                bad("register", std::to_string(st));
            }
            next += 64 * kMiB;
        } else if (!live.empty()) {
            size_t k = (seed >> 4) % live.size();
            int st = rt_uvm_unregister_ptr(live[k]);          // number of records removed, or an error
            if (st < 0 && st != RT_ERR_NOT_RUNNING) bad("unregister", std::to_string(st));
            live.erase(live.begin() + (long)k);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    for (uint64_t p : live) rt_uvm_unregister_ptr(p);
}

// status / list / plan lines through the socket.
void client_thread(int which) {
    unsigned seed = 77u + (unsigned)which;
    std::string reply;
    while (!g_stop.load()) {
        seed = seed * 1103515245u + 12345u;
        std::string line;
        switch ((seed >> 12) % 6) {
            case 0: line = "status"; break;
            case 1: line = "list"; break;
            case 2: {
                if (!socket_command("status", &reply)) continue;
                line = "targetv " + std::to_string(field(reply, "allocation_generation")) + " " +
                       std::to_string(field(reply, "managed_bytes") / (4 * kMiB) * (2 * kMiB));
                break;
            }
            case 3: {
                if (!socket_command("status", &reply)) continue;
                line = "blocksv " + std::to_string(field(reply, "allocation_generation")) + " " +
                       std::to_string(32 * kMiB) + " 1 " + std::to_string(2 * kMiB) + " a5f";
                break;
            }
            case 4: line = "windowv 0 1 2 3"; break;                 // malformed on purpose
            default: line = "prefetch 1 0 4096 gpu"; break;
        }
        if (!socket_command(line, &reply)) continue;
        g_commands.fetch_add(1);
        if (!well_formed(reply)) bad("socket reply", line + " -> " + reply);
    }
}

// The device planner's hand-off: ranges by buffer index, then a wait.
void submit_thread() {
    unsigned seed = 5;
    while (!g_stop.load()) {
        seed = seed * 1103515245u + 12345u;
        std::string list = local_command("list");
        if (!well_formed(list)) {
            if (!list.empty()) bad("list reply", list);
            continue;
        }
        // first allocation id and size in the list, if any
        size_t at = list.find("\"id\":");
        if (at == std::string::npos) continue;
        uint64_t id = strtoull(list.c_str() + at + 5, nullptr, 10);
        uint64_t bytes = field(list.substr(at), "bytes");
        if (!bytes) continue;
        rt_range r[2] = {{0, -1, 0, bytes / 2 / 4096 * 4096}, {0, 0, 0, bytes / 4 / 4096 * 4096}};
        uint64_t job = 0;
        int st = rt_uvm_submit_ranges(r, 2, &id, 1, &job);
        if (st == RT_OK) {
            int cuda_error = 0;
            st = rt_uvm_wait(job, 5.0, &cuda_error);
            // RT_ERR_CUDA: the allocation was freed while its job ran, which the
            // worker reports as an invalid value, like select.cpp:23960-23963
            if (st != RT_OK && st != RT_ERR_NOT_RUNNING && st != RT_ERR_CUDA) bad("wait", std::to_string(st));
            g_jobs.fetch_add(1);
        } else if (st != RT_ERR_BUSY && st != RT_ERR_NOT_RUNNING && st != RT_ERR_PLAN &&
                   st != RT_ERR_INVALID_ARGUMENT) {
            bad("submit", std::to_string(st));
        }
        if ((seed >> 9) % 8 == 0) std::this_thread::sleep_for(std::chrono::microseconds(300));
    }
}

}  // namespace

int main(int argc, char **argv) {
    if (argc < 3) {
        fprintf(stderr, "usage: uvm_stress <stub libcuda> <socket path> [seconds]\n");
        return 2;
    }
    setenv("RETARGET_B200_LIBCUDA", argv[1], 1);
    g_socket = argv[2];
    const double seconds = argc > 3 ? atof(argv[3]) : 2.0;
    rt_uvm_config cfg{};
    cfg.socket_path = g_socket;
    cfg.chunk_bytes = 4 * kMiB;
    cfg.batch_bytes = 16 * kMiB;
    cfg.streams = 3;
    cfg.listen = 1;
    if (rt_uvm_start(&cfg) != RT_OK) {
        fprintf(stderr, "uvm_stress: rt_uvm_start failed\n");
        return 1;
    }
    std::vector<std::thread> threads;
    threads.emplace_back(app_thread);
    threads.emplace_back(client_thread, 0);
    threads.emplace_back(client_thread, 1);
    threads.emplace_back(submit_thread);
    const auto t0 = std::chrono::steady_clock::now();
    int restarts = 0;
    while (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() < seconds) {
        std::this_thread::sleep_for(std::chrono::milliseconds(250));
        // stop and start under load: callers see "not running" or a refused connection
        if (rt_uvm_stop() != RT_OK) bad("stop", "");
        if (rt_uvm_start(&cfg) != RT_OK) bad("restart", "");
        ++restarts;
    }
    g_stop.store(true);
    for (auto &t : threads) t.join();
    if (rt_uvm_stop() != RT_OK) bad("final stop", "");
    printf("uvm_stress: commands=%ld jobs=%ld allocations=%ld restarts=%d bad=%d\n", g_commands.load(),
           g_jobs.load(), g_allocs.load(), restarts, g_bad.load());
    return g_bad.load() ? 1 : 0;
}
