/*
 * Stand-in for a CUDA application under LD_PRELOAD: it finds the driver the way
 * a CUDA runtime does (dlopen + dlsym, and cuGetProcAddress), allocates
 * "device" memory, then talks to the control socket of its own process.
 * Prints what it sees; the test checks the text.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <sys/wait.h>
#include <unistd.h>

typedef int (*init_fn)(unsigned);
typedef int (*alloc_fn)(unsigned long long *, size_t);
typedef int (*free_fn)(unsigned long long);
typedef int (*setctx_fn)(void *);
typedef int (*gpa_fn)(const char *, void **, int, unsigned long long);
typedef size_t (*log_fn)(char *, size_t);

static void ask(const char *line)
{
    char path[108], reply[65536];
    snprintf(path, sizeof(path), "/tmp/select-uvm-%lu-%ld.sock", (unsigned long)getuid(), (long)getpid());
    struct sockaddr_un addr = {0};
    addr.sun_family = AF_UNIX;
    strcpy(addr.sun_path, path);
    int fd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (connect(fd, (struct sockaddr *)&addr, sizeof(addr)) != 0) { printf("REPLY %s -> connect failed\n", line); close(fd); return; }
    dprintf(fd, "%s\n", line);
    size_t used = 0;
    ssize_t n;
    while ((n = read(fd, reply + used, sizeof(reply) - 1 - used)) > 0) used += (size_t)n;
    reply[used] = 0;
    if (used && reply[used - 1] == '\n') reply[used - 1] = 0;
    printf("REPLY %s -> %s\n", line, reply);
    close(fd);
}

int main(int argc, char **argv)
{
    void *drv = dlopen(argv[1], RTLD_NOW | RTLD_GLOBAL);
    if (!drv) { printf("no driver: %s\n", dlerror()); return 2; }
    init_fn init = (init_fn)dlsym(drv, "cuInit");
    setctx_fn setctx = (setctx_fn)dlsym(drv, "cuCtxSetCurrent");
    alloc_fn alloc = (alloc_fn)dlsym(drv, "cuMemAlloc_v2");
    gpa_fn gpa = (gpa_fn)dlsym(drv, "cuGetProcAddress");
    free_fn release = NULL;
    printf("cuInit=%d\n", init(0));
    setctx((void *)0xC000);
    gpa("cuMemFree", (void **)&release, 12000, 0);
    unsigned long long p[5];
    for (int i = 0; i < 4; ++i) printf("alloc%d=%d\n", i, alloc(&p[i], 32u << 20));
    printf("alloc4=%d\n", alloc(&p[4], 4096));
    ask("status");
    ask("list");
    char line[256];
    snprintf(line, sizeof(line), "windowv 5 %u 4 18446744073709551615 18446744073709551615 0 %u", 32u << 20, 8u << 20);
    ask(line);
    usleep(200000);
    ask("status");
    printf("free=%d\n", release(p[1]));
    ask("list");
    if (argc > 2 && !strcmp(argv[2], "fork")) {
        fflush(stdout);
        pid_t child = fork();
        if (child == 0) {
            unsigned long long q;
            printf("child alloc=%d\n", alloc(&q, 4096));   /* must be refused */
            fflush(stdout);
            _exit(0);
        }
        int st; waitpid(child, &st, 0);
    }
    log_fn fake_log = (log_fn)dlsym(drv, "fake_cuda_log");
    static char buf[1 << 20];
    fake_log(buf, sizeof(buf));
    printf("DRIVER LOG\n%s", buf);
    return 0;
}
