// Client side of the UVM control socket, and the identity checks a client makes
// before it trusts a PID.
//
// The protocol (select.cpp:24330-24376 is the server's half): connect to the
// AF_UNIX stream socket of the controlled process, send ONE line of at most 511
// bytes, read ONE line of JSON back, close.  The reference's client does this in
// Python (experiments/control.py:427-460); here the transport is native and
// deadline-driven: one deadline covers connect, send and receive, every wait is
// a poll() against what is left of it, and the reply is collected in the
// caller's buffer until the first newline.
#include <fcntl.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <unistd.h>

#include <cerrno>
#include <cinttypes>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>

#include "rt_internal.h"

namespace {

constexpr size_t kMaxLine = 512;            // including the newline, select.cpp:24047-24054
constexpr size_t kMaxReply = 1u << 20;

double monotonic_s() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

struct Fd {
    int fd = -1;
    ~Fd() {
        if (fd >= 0) close(fd);
    }
};

// Waits until `fd` is ready for `events` or the deadline passes.  0 ok, else errno.
int wait_ready(int fd, short events, double deadline) {
    for (;;) {
        const double left = deadline - monotonic_s();
        if (left <= 0) return ETIMEDOUT;
        pollfd p = {fd, events, 0};
        int ms = left > 3600 ? 3600000 : (int)(left * 1e3) + 1;
        int r = poll(&p, 1, ms);
        if (r > 0) return 0;                 // readable / writable, or an error the next call reports
        if (r < 0 && errno != EINTR) return errno;
    }
}

// Value of `"key":` in a flat JSON object, as text up to the next , or }.
bool flat_value(const char *text, const char *key, const char **begin, const char **end) {
    char pattern[64];
    int n = snprintf(pattern, sizeof(pattern), "\"%s\":", key);
    if (n <= 0 || (size_t)n >= sizeof(pattern)) return false;
    const char *at = strstr(text, pattern);
    if (!at) return false;
    at += n;
    while (*at == ' ') ++at;
    const char *stop = at;
    while (*stop && *stop != ',' && *stop != '}') ++stop;
    *begin = at;
    *end = stop;
    return stop > at;
}

bool flat_u64(const char *text, const char *key, uint64_t *out) {
    const char *b, *e;
    if (!flat_value(text, key, &b, &e)) return false;
    char *stop = nullptr;
    errno = 0;
    unsigned long long v = strtoull(b, &stop, 10);
    if (errno || stop == b) return false;
    *out = v;
    return true;
}

bool flat_i64(const char *text, const char *key, int64_t *out) {
    const char *b, *e;
    if (!flat_value(text, key, &b, &e)) return false;
    char *stop = nullptr;
    errno = 0;
    long long v = strtoll(b, &stop, 10);
    if (errno || stop == b) return false;
    *out = v;
    return true;
}

bool flat_bool(const char *text, const char *key, int *out) {
    const char *b, *e;
    if (!flat_value(text, key, &b, &e)) return false;
    if (!strncmp(b, "true", 4)) *out = 1;
    else if (!strncmp(b, "false", 5)) *out = 0;
    else {
        uint64_t v;
        if (!flat_u64(text, key, &v)) return false;
        *out = v != 0;
    }
    return true;
}

}  // namespace

extern "C" {

int rt_uvm_client_command(const char *socket_path, const char *line, double timeout_s, char *reply, size_t cap,
                          int *os_error) {
    if (os_error) *os_error = 0;
    if (!socket_path || !line || !reply || cap < 2 || !(timeout_s > 0)) return RT_ERR_INVALID_ARGUMENT;
    const size_t len = strlen(line);
    if (len + 1 >= kMaxLine || strpbrk(line, "\r\n")) return RT_ERR_INVALID_ARGUMENT;
    sockaddr_un addr = {};
    addr.sun_family = AF_UNIX;
    if (strlen(socket_path) >= sizeof(addr.sun_path)) return RT_ERR_INVALID_ARGUMENT;
    strcpy(addr.sun_path, socket_path);
    auto fail = [&](int err) {
        if (os_error) *os_error = err;
        return RT_ERR_IO;
    };
    const double deadline = monotonic_s() + timeout_s;
    Fd s;
    s.fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
    if (s.fd < 0) return fail(errno);
    if (connect(s.fd, reinterpret_cast<sockaddr *>(&addr), sizeof(addr)) != 0) {
        if (errno != EINPROGRESS && errno != EAGAIN) return fail(errno);
        if (int err = wait_ready(s.fd, POLLOUT, deadline)) return fail(err);
        int so_error = 0;
        socklen_t sl = sizeof(so_error);
        if (getsockopt(s.fd, SOL_SOCKET, SO_ERROR, &so_error, &sl) != 0) return fail(errno);
        if (so_error) return fail(so_error);
    }
    // the line and its terminator go out as one buffer
    char wire[kMaxLine];
    memcpy(wire, line, len);
    wire[len] = '\n';
    for (size_t sent = 0; sent < len + 1;) {
        ssize_t n = send(s.fd, wire + sent, len + 1 - sent, MSG_NOSIGNAL);
        if (n > 0) {
            sent += (size_t)n;
        } else if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) {
            if (int err = wait_ready(s.fd, POLLOUT, deadline)) return fail(err);
        } else if (n < 0 && errno != EINTR) {
            return fail(errno);
        }
    }
    // the reply: everything up to the first newline (or to end of stream)
    size_t got = 0;
    for (;;) {
        if (got + 1 >= cap || got >= kMaxReply) return RT_ERR_CAPACITY;
        ssize_t n = recv(s.fd, reply + got, cap - 1 - got, 0);
        if (n > 0) {
            char *nl = static_cast<char *>(memchr(reply + got, '\n', (size_t)n));
            got += (size_t)n;
            if (nl) {
                got = (size_t)(nl - reply);
                break;
            }
        } else if (n == 0) {
            break;
        } else if (errno == EAGAIN || errno == EWOULDBLOCK) {
            if (int err = wait_ready(s.fd, POLLIN, deadline)) return fail(err);
        } else if (errno != EINTR) {
            return fail(errno);
        }
    }
    reply[got] = 0;
    return (int)got;
}

// select.cpp:24058-24068: the status reply.  RT_ERR_PLAN when it says ok:false,
// RT_ERR_INVALID_ARGUMENT when a field is missing.
int rt_uvm_parse_status(const char *reply, rt_uvm_status *out) {
    if (!reply || !out) return RT_ERR_INVALID_ARGUMENT;
    int ok = 0;
    if (!flat_bool(reply, "ok", &ok)) return RT_ERR_INVALID_ARGUMENT;
    if (!ok) return RT_ERR_PLAN;
    memset(out, 0, sizeof(*out));
    int64_t last_error = 0;
    int busy = 0;
    bool all = flat_u64(reply, "pid", &out->pid) && flat_u64(reply, "managed_bytes", &out->managed_bytes) &&
               flat_u64(reply, "allocation_count", &out->allocation_count) && flat_bool(reply, "busy", &busy) &&
               flat_u64(reply, "job_id", &out->job_id) && flat_u64(reply, "completed_job", &out->completed_job) &&
               flat_i64(reply, "last_error", &last_error) &&
               flat_u64(reply, "completed_cpu_bytes", &out->completed_cpu_bytes) &&
               flat_u64(reply, "completed_gpu_bytes", &out->completed_gpu_bytes) &&
               flat_u64(reply, "job_completed_bytes", &out->job_completed_bytes);
    if (!all) return RT_ERR_INVALID_ARGUMENT;
    flat_u64(reply, "allocation_generation", &out->allocation_generation);   // older servers omit it: 0
    out->busy = busy;
    out->last_error = (int32_t)last_error;
    return RT_OK;
}

// Start time of a process in clock ticks since boot (field 22 of
// /proc/<pid>/stat): a PID that comes back with another start time is another
// process.  The command name (field 2) may contain spaces and parentheses, so
// the fields are counted from the LAST closing parenthesis.
int rt_process_start_time(uint64_t pid, uint64_t *ticks, int *os_error) {
    if (os_error) *os_error = 0;
    if (!ticks) return RT_ERR_INVALID_ARGUMENT;
    char path[64], text[1024];
    snprintf(path, sizeof(path), "/proc/%" PRIu64 "/stat", pid);
    Fd f;
    f.fd = open(path, O_RDONLY | O_CLOEXEC);
    if (f.fd < 0) {
        if (os_error) *os_error = errno;
        return RT_ERR_IO;
    }
    ssize_t n = read(f.fd, text, sizeof(text) - 1);
    if (n < 0) {
        if (os_error) *os_error = errno;
        return RT_ERR_IO;
    }
    text[n] = 0;
    const char *p = strrchr(text, ')');
    if (!p) return RT_ERR_INVALID_ARGUMENT;
    // after ") " comes field 3 (state); the start time is field 22
    int field = 2;
    for (++p; *p; ++p) {
        if (*p != ' ') continue;
        if (++field == 22) {
            char *stop = nullptr;
            errno = 0;
            unsigned long long v = strtoull(p + 1, &stop, 10);
            if (errno || stop == p + 1) return RT_ERR_INVALID_ARGUMENT;
            *ticks = v;
            return RT_OK;
        }
    }
    return RT_ERR_INVALID_ARGUMENT;
}

// Owner of a process (the uid of /proc/<pid>).
int rt_process_owner(uint64_t pid, uint32_t *uid, int *os_error) {
    if (os_error) *os_error = 0;
    if (!uid) return RT_ERR_INVALID_ARGUMENT;
    char path[64];
    snprintf(path, sizeof(path), "/proc/%" PRIu64, pid);
    struct stat st;
    if (stat(path, &st) != 0) {
        if (os_error) *os_error = errno;
        return RT_ERR_IO;
    }
    *uid = st.st_uid;
    return RT_OK;
}

}  // extern "C"
