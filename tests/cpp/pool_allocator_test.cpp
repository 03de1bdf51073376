// CPU test of glasssix::memory::pool_allocator (excalibur_b200/csrc/host/primitives.hpp) against the behaviour of
// the reference's allocator (include/Primitives/pool_allocator.hpp:72-146): the 75 %..100 % reuse rule,
// the adjustable ratio, a pointer the pool never handed out, and two threads allocating and freeing at once
// (the two lists have a mutex each; a call that held both in opposite orders would deadlock here).
// Heap memory only (device_id = -1): no GPU is touched.  Prints "ok" and exits 0 on success.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <thread>
#include <vector>

#include "primitives.hpp"

using glasssix::memory::pool_allocator;

#define EXPECT(c)                                                        \
    do {                                                                 \
        if (!(c)) {                                                      \
            std::fprintf(stderr, "%s:%d: EXPECT(%s) failed\n", __FILE__, __LINE__, #c); \
            return 1;                                                    \
        }                                                                \
    } while (0)

int main() {
    glasssix::set_log_quiet(true);
    {
        pool_allocator<float> pool;
        void* a = pool.fastMalloc(1000);
        EXPECT(a != nullptr && pool.payout_count() == 1 && pool.budget_count() == 0);
        pool.fastFree(a);
        EXPECT(pool.payout_count() == 0 && pool.budget_count() == 1);
        void* b = pool.fastMalloc(800);      // 80 % of the free 1000-byte buffer: reused
        EXPECT(b == a && pool.budget_count() == 0);
        pool.fastFree(b);
        void* c = pool.fastMalloc(700);      // 70 %: below the 75 % rule, a new buffer
        EXPECT(c != a && pool.budget_count() == 1);
        void* d = pool.fastMalloc(1001);     // larger than the free buffer: a new one
        EXPECT(d != a && pool.budget_count() == 1);
        void* e = pool.fastMalloc(1000);     // exact fit
        EXPECT(e == a);
        pool.fastFree(c);
        pool.fastFree(d);
        pool.fastFree(e);
        EXPECT(pool.payout_count() == 0 && pool.budget_count() == 3);
        pool.set_size_compare_ratio(0.5f);
        void* f = pool.fastMalloc(500);      // 50 % of 1000 (or 71 % of 700) is acceptable now
        EXPECT(f == c || f == a || f == d);
        pool.fastFree(f);
        pool.clear();
        EXPECT(pool.budget_count() == 0);
        // a pointer the pool did not hand out is released after an error line, as the reference does
        void* wild = nullptr;
        EXPECT(posix_memalign(&wild, 64, 256) == 0);
        pool.fastFree(wild);
        EXPECT(pool.budget_count() == 0 && pool.payout_count() == 0);
    }
    {
        pool_allocator<float> pool;
        std::atomic<bool> stop{false};
        std::atomic<long> rounds{0};
        auto worker = [&](unsigned seed) {
            std::vector<void*> mine;
            unsigned s = seed;
            while (!stop.load()) {
                s = s * 1664525u + 1013904223u;
                if (mine.size() < 8 && (s >> 16) % 3 != 0) {
                    void* p = pool.fastMalloc(256 + (s >> 8) % 4096);
                    static_cast<char*>(p)[0] = (char)s;     // the buffer is ours alone
                    mine.push_back(p);
                } else if (!mine.empty()) {
                    pool.fastFree(mine.back());
                    mine.pop_back();
                }
                rounds.fetch_add(1);
            }
            for (void* p : mine) pool.fastFree(p);
        };
        std::thread t1(worker, 1u), t2(worker, 2u), t3(worker, 3u);
        std::this_thread::sleep_for(std::chrono::milliseconds(1000));
        stop.store(true);
        t1.join();
        t2.join();
        t3.join();
        EXPECT(pool.payout_count() == 0);
        EXPECT(rounds.load() > 1000);
        std::printf("threads: %ld allocate/free rounds, %zu buffers on the free list\n", rounds.load(), pool.budget_count());
    }
    std::printf("ok\n");
    return 0;
}
