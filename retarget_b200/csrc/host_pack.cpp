#include "host_pack.h"

#include <sched.h>
#if defined(__x86_64__)
#include <immintrin.h>
#endif

#include <atomic>
#include <climits>
#include <condition_variable>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace rt {

namespace {

inline int32_t narrow_one(int64_t s) {
    const int32_t lo = (int32_t)s, hi = (int32_t)(s >> 32);
    // hi == 0 and lo >= 0: the id itself; otherwise the sign of the id decides
    return (hi == 0 && lo >= 0) ? lo : (hi < 0 ? -1 : INT32_MAX);
}

void narrow_scalar(const int64_t *src, int32_t *dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = narrow_one(src[i]);
}

#if defined(__x86_64__)
// Eight ids per step: when none of them has a bit at or above 2^31 (the rule in
// a slot table) their low halves are gathered with three shuffles and written
// with a streaming store, which keeps the staging buffer out of the caches the
// DMA engine does not read from anyway; any other group of eight goes id by id.
__attribute__((target("avx2"))) void narrow_avx2(const int64_t *src, int32_t *dst, size_t n) {
    size_t i = 0;
    while (i < n && (reinterpret_cast<uintptr_t>(dst + i) & 31u)) {
        dst[i] = narrow_one(src[i]);
        ++i;
    }
    const __m256i high = _mm256_set1_epi64x((long long)0xffffffff80000000ull);
    const __m256i evens = _mm256_setr_epi32(0, 2, 4, 6, 0, 2, 4, 6);
    for (; i + 8 <= n; i += 8) {
        const __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(src + i));
        const __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(src + i + 4));
        if (_mm256_testz_si256(_mm256_or_si256(a, b), high)) {
            const __m256i pa = _mm256_permutevar8x32_epi32(a, evens), pb = _mm256_permutevar8x32_epi32(b, evens);
            _mm256_stream_si256(reinterpret_cast<__m256i *>(dst + i), _mm256_permute2x128_si256(pa, pb, 0x20));
        } else {
            for (size_t k = i; k < i + 8; ++k) dst[k] = narrow_one(src[k]);
        }
    }
    for (; i < n; ++i) dst[i] = narrow_one(src[i]);
    _mm_sfence();                              // streaming stores are visible before the copy is issued
}
#endif

}  // namespace

void narrow_ids(const int64_t *src, int32_t *dst, size_t n) {
#if defined(__x86_64__)
    static const bool avx2 = __builtin_cpu_supports("avx2");
    if (avx2) return narrow_avx2(src, dst, n);
#endif
    narrow_scalar(src, dst, n);
}

unsigned narrow_threads(unsigned sharers) {
    if (const char *text = std::getenv("RETARGET_B200_PACK_THREADS")) {
        char *end = nullptr;
        long v = std::strtol(text, &end, 10);
        if (end != text && v >= 0) return (unsigned)(v > 64 ? 64 : v);
    }
    cpu_set_t set;
    unsigned cpus = std::thread::hardware_concurrency();
    if (sched_getaffinity(0, sizeof(set), &set) == 0) cpus = (unsigned)CPU_COUNT(&set);
    // Narrowing trades host memory traffic for link traffic: it reads 8 and writes 4
    // bytes per id to save 4 on the link, and the copy engine reads those 4 again.  It
    // pays when the link is what is short and the host's memory is not: one planner on
    // a host.  Two planners narrowing side by side on one host measured slower than two
    // wide copies (3.98 against 3.60 ms per step), and with fewer than 8 threads the
    // narrowing is slower than the copy it shortens.
    if (sharers > 1) return 0;
    // three quarters of the CPUs: the rest stays free for the caller's other threads
    // and the driver's
    unsigned t = cpus * 3 / 4;
    if (t > 16) t = 16;
    return t >= 8 ? t : 0;
}

namespace {

constexpr size_t kPartIds = 1 << 16;          // 512 KiB in, 256 KiB out per part

// One call's work: parts are claimed in ascending order by whoever is free, the
// caller included; `left[c]` counts the parts of chunk c that are not done yet.
struct Job {
    const int64_t *src;
    int32_t *dst;
    size_t n, parts, chunk_parts;
    std::atomic<size_t> next{0};
    std::unique_ptr<std::atomic<uint32_t>[]> left;

    Job(const int64_t *s, int32_t *d, size_t count, size_t chunk_ids)
        : src(s), dst(d), n(count), parts((count + kPartIds - 1) / kPartIds),
          chunk_parts((chunk_ids + kPartIds - 1) / kPartIds) {
        const size_t chunks = (parts + chunk_parts - 1) / chunk_parts;
        left.reset(new std::atomic<uint32_t>[chunks]);
        for (size_t c = 0; c < chunks; ++c) {
            const size_t first = c * chunk_parts;
            left[c].store((uint32_t)(parts - first < chunk_parts ? parts - first : chunk_parts),
                          std::memory_order_relaxed);
        }
    }

    bool work_one() {
        const size_t p = next.fetch_add(1, std::memory_order_relaxed);
        if (p >= parts) return false;
        const size_t lo = p * kPartIds, hi = lo + kPartIds < n ? lo + kPartIds : n;
        narrow_ids(src + lo, dst + lo, hi - lo);
        left[p / chunk_parts].fetch_sub(1, std::memory_order_release);
        return true;
    }
};

class Pool {
  public:
    explicit Pool(unsigned workers) {
        for (unsigned i = 0; i < workers; ++i) std::thread([this] { loop(); }).detach();
    }

    // Publishes the job, then hands every chunk to `ready` as soon as its last
    // part is done, working on parts itself while it waits.
    void run(const std::shared_ptr<Job> &job, ChunkReady ready, void *ctx) {
        std::lock_guard<std::mutex> turn(callers_);
        {
            std::lock_guard<std::mutex> lock(m_);
            job_ = job;
            seq_.fetch_add(1, std::memory_order_release);
        }
        wake_.notify_all();
        const size_t chunk_ids = job->chunk_parts * kPartIds;
        for (size_t c = 0, first = 0; first < job->n; ++c, first += chunk_ids) {
            while (job->left[c].load(std::memory_order_acquire) != 0)
                if (!job->work_one()) std::this_thread::yield();
            if (ready) ready(ctx, first, job->n - first < chunk_ids ? job->n - first : chunk_ids);
        }
    }

  private:
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            // calls tend to come in quick succession: look for the next one for a
            // while before going to sleep
            for (int spin = 0; spin < 20000 && seq_.load(std::memory_order_acquire) == seen; ++spin)
                std::this_thread::yield();
            std::shared_ptr<Job> job;
            {
                std::unique_lock<std::mutex> lock(m_);
                wake_.wait(lock, [&] { return seq_.load(std::memory_order_acquire) != seen; });
                seen = seq_.load(std::memory_order_acquire);
                job = job_;
            }
            if (job)                         // a job that is already finished has no part left to claim
                while (job->work_one()) {
                }
        }
    }

    std::mutex callers_, m_;
    std::condition_variable wake_;
    std::atomic<uint64_t> seq_{0};
    std::shared_ptr<Job> job_;
};

}  // namespace

void narrow_ids_streamed(const int64_t *src, int32_t *dst, size_t n, unsigned threads, size_t chunk_ids,
                         ChunkReady ready, void *ctx) {
    if (!n) return;
    if (chunk_ids < kPartIds) chunk_ids = kPartIds;
    if (threads <= 1 || n <= kPartIds) {
        for (size_t first = 0; first < n; first += chunk_ids) {
            const size_t m = n - first < chunk_ids ? n - first : chunk_ids;
            narrow_ids(src + first, dst + first, m);
            if (ready) ready(ctx, first, m);
        }
        return;
    }
    // never destroyed: its threads are detached and may outlive static destructors
    static Pool *pool = new Pool(threads - 1);
    pool->run(std::make_shared<Job>(src, dst, n, chunk_ids), ready, ctx);
}

void narrow_ids_parallel(const int64_t *src, int32_t *dst, size_t n, unsigned threads) {
    narrow_ids_streamed(src, dst, n, threads, n, nullptr, nullptr);
}

}  // namespace rt
