// Stress for the host-side id narrowing pool: several threads call it at once
// with lists of different lengths and chunk sizes; every result is compared
// with the single-thread form and every chunk must be reported once, in order,
// and only after its ids are in place.
#include <atomic>
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#include "host_pack.h"

namespace {

std::atomic<int> g_bad{0};

struct Seen {
    const int64_t *src;
    const int32_t *dst;
    size_t next = 0, calls = 0;
};

void on_chunk(void *ctx, size_t first, size_t count) {
    Seen *s = static_cast<Seen *>(ctx);
    if (first != s->next || count == 0) g_bad.fetch_add(1);
    // the chunk is complete when it is reported
    int32_t want[4];
    for (size_t k = 0; k < 4 && k < count; ++k) {
        const size_t i = first + (count - 1) * k / 3;
        rt::narrow_ids(s->src + i, want, 1);
        if (s->dst[i] != want[0]) g_bad.fetch_add(1);
    }
    s->next = first + count;
    ++s->calls;
}

void caller(unsigned seed, int rounds, unsigned threads) {
    std::mt19937_64 rng(seed);
    for (int r = 0; r < rounds; ++r) {
        const size_t n = 1 + rng() % 700000;
        std::vector<int64_t> src(n);
        for (auto &v : src) v = (int64_t)(rng() % 300000);
        for (int k = 0; k < 8; ++k) src[rng() % n] = (int64_t)rng();          // any 64-bit pattern
        std::vector<int32_t> got(n, 0x5a5a5a5a), want(n);
        rt::narrow_ids(src.data(), want.data(), n);
        Seen seen{src.data(), got.data()};
        const size_t chunk = (size_t)65536 << (rng() % 4);
        rt::narrow_ids_streamed(src.data(), got.data(), n, threads, chunk, on_chunk, &seen);
        if (seen.next != n || got != want) g_bad.fetch_add(1);
    }
}

}  // namespace

int main(int argc, char **argv) {
    const int rounds = argc > 1 ? atoi(argv[1]) : 20;
    std::vector<std::thread> callers;
    for (unsigned t = 0; t < 3; ++t) callers.emplace_back(caller, 100 + t, rounds, 4u);
    for (auto &t : callers) t.join();
    printf("pack_stress: bad=%d\n", g_bad.load());
    return g_bad.load() ? 1 : 0;
}
