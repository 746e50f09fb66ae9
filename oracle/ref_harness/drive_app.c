/*
 * Drives a preload library (the reference's, or this repository's) through its
 * own control socket under the stub driver, and prints everything observable:
 * the socket replies and the driver calls each plan caused.
 *
 *   LD_PRELOAD=<lib> LD_LIBRARY_PATH=<stubs> drive_app <libcuda path> <size> [<size> ...] < commands
 *
 * Each <size> is one cuMemAlloc_v2 (converted to a managed allocation by the
 * library).  A size prefixed with '-' frees the allocation with that 1-based
 * index instead.  stdin: one socket command per line; after a reply with a
 * job_id the program polls `status` until the job is done and prints the
 * prefetch calls the driver saw.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

typedef int (*init_fn)(unsigned);
typedef int (*alloc_fn)(unsigned long long *, size_t);
typedef int (*free_fn)(unsigned long long);
typedef int (*setctx_fn)(void *);
typedef size_t (*log_fn)(char *, size_t);
typedef void (*reset_fn)(void);

static int ask(const char *line, char *reply, size_t cap)
{
    char path[108];
    snprintf(path, sizeof(path), "/tmp/select-uvm-%lu-%ld.sock", (unsigned long)getuid(), (long)getpid());
    struct sockaddr_un addr = {0};
    addr.sun_family = AF_UNIX;
    strcpy(addr.sun_path, path);
    int fd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (connect(fd, (struct sockaddr *)&addr, sizeof(addr)) != 0) { close(fd); return -1; }
    dprintf(fd, "%s\n", line);
    size_t used = 0;
    ssize_t n;
    while ((n = read(fd, reply + used, cap - 1 - used)) > 0) used += (size_t)n;
    reply[used] = 0;
    if (used && reply[used - 1] == '\n') reply[used - 1] = 0;
    close(fd);
    return 0;
}

int main(int argc, char **argv)
{
    void *drv = dlopen(argv[1], RTLD_NOW | RTLD_GLOBAL);
    if (!drv) { printf("no driver: %s\n", dlerror()); return 2; }
    init_fn init = (init_fn)dlsym(drv, "cuInit");
    setctx_fn setctx = (setctx_fn)dlsym(drv, "cuCtxSetCurrent");
    alloc_fn alloc = (alloc_fn)dlsym(drv, "cuMemAlloc_v2");
    free_fn release = (free_fn)dlsym(drv, "cuMemFree_v2");
    log_fn fake_log = (log_fn)dlsym(drv, "fake_cuda_log");
    reset_fn fake_reset = (reset_fn)dlsym(drv, "fake_cuda_reset");
    if (init(0) != 0) { printf("cuInit failed\n"); return 3; }
    setctx((void *)0xC000);
    static unsigned long long ptrs[1024];
    int n_alloc = 0;
    for (int i = 2; i < argc; ++i) {
        if (argv[i][0] == '-') {
            int idx = atoi(argv[i] + 1);
            printf("FREE %d -> %d\n", idx, release(ptrs[idx - 1]));
        } else {
            int rc = alloc(&ptrs[n_alloc], (size_t)strtoull(argv[i], NULL, 10));
            printf("ALLOC %d %s -> %d %llx\n", n_alloc + 1, argv[i], rc, ptrs[n_alloc]);
            ++n_alloc;
        }
    }
    static char line[1024], reply[1 << 20], log[1 << 20];
    while (fgets(line, sizeof(line), stdin)) {
        line[strcspn(line, "\n")] = 0;
        fake_reset();
        if (ask(line, reply, sizeof(reply)) != 0) { printf("REPLY %s -> connect failed\n", line); continue; }
        printf("REPLY %s -> %s\n", line, reply);
        if (strstr(reply, "\"job_id\"") && strstr(reply, "\"ok\":true") && !strstr(reply, "\"busy\"")) {
            for (int spin = 0; spin < 2000; ++spin) {
                ask("status", reply, sizeof(reply));
                if (strstr(reply, "\"busy\":false")) break;
                usleep(2000);
            }
            printf("STATUS %s\n", reply);
            fake_log(log, sizeof(log));
            for (char *p = strtok(log, "\n"); p; p = strtok(NULL, "\n"))
                if (!strncmp(p, "prefetch ", 9)) printf("CALL %s\n", p);
        }
        printf("END\n");
    }
    fflush(stdout);
    return 0;
}
