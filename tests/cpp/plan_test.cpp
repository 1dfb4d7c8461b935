// The chunk arithmetic of the pipelined broadcast and the staged reduces, checked on the host:
// for awkward lengths, rank counts, grid sizes and chunk sizes, the (slice, CTA, chunk) ranges
// that the kernels derive from bcast_plan / reduce_plan must cover every byte / element of the
// message exactly once, never reach past it, and never exceed a chunk (a staging slot).
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "kernels/collectives.cuh"
#include "mini_test.h"

using namespace mgk::coll;

namespace {

// what direct_family_kernel computes for broadcast (bytes relative to slice v)
void bcast_range(const BcastPlan& pl, uint64_t S, uint32_t chunk, int cta, int v, uint32_t k, uint64_t* lo, uint64_t* hi) {
    const uint64_t sb = pl.per_cta * static_cast<uint64_t>(cta);
    const uint64_t s0 = static_cast<uint64_t>(v) * pl.slice;
    const uint64_t L = s0 >= S ? 0 : std::min(pl.slice, S - s0);
    *lo = std::min(L, sb + static_cast<uint64_t>(k) * chunk);
    *hi = std::min(L, std::min(sb + pl.per_cta, sb + static_cast<uint64_t>(k + 1) * chunk));
}

// ... and for the staged reduces (elements relative to slice v)
void reduce_range(const ReducePlan& pl, uint64_t len, int cta, int v, uint32_t k, uint64_t* lo, uint64_t* hi) {
    const uint64_t sb = pl.per_cta * static_cast<uint64_t>(cta);
    const uint64_t s0 = static_cast<uint64_t>(v) * pl.slice;
    const uint64_t L = s0 >= len ? 0 : std::min(pl.slice, len - s0);
    *lo = std::min(L, sb + static_cast<uint64_t>(k) * pl.chunk_el);
    *hi = std::min(L, std::min(sb + pl.per_cta, sb + static_cast<uint64_t>(k + 1) * pl.chunk_el));
}

}  // namespace

TEST(Plan_BroadcastChunksCoverTheMessageExactlyOnce) {
    const uint64_t sizes[] = {1, 15, 16, 17, 4096, 65537, 280004, 1200028};
    const uint32_t chunks[] = {4096, 16384, 65536, 1u << 20};
    for (int n = 2; n <= 8; ++n)
        for (uint64_t S : sizes)
            for (int ctas : {1, 3, 4, 36, 85, 128})
                for (uint32_t chunk : chunks) {
                    const BcastPlan pl = bcast_plan(S, n, ctas, chunk);
                    EXPECT_TRUE(pl.slice % 16 == 0 && pl.per_cta % 16 == 0 && pl.chunks >= 1);
                    std::vector<uint8_t> seen(S, 0);
                    bool fine = true;
                    for (int v = 0; v < n - 1; ++v)
                        for (int b = 0; b < ctas; ++b)
                            for (uint32_t k = 0; k < pl.chunks; ++k) {
                                uint64_t lo, hi;
                                bcast_range(pl, S, chunk, b, v, k, &lo, &hi);
                                if (hi < lo || hi - lo > chunk)
                                    fine = false;
                                for (uint64_t i = lo; i < hi; ++i) {
                                    const uint64_t at = static_cast<uint64_t>(v) * pl.slice + i;
                                    if (at >= S || seen[at]++)
                                        fine = false;
                                }
                            }
                    for (uint64_t i = 0; i < S && fine; ++i)
                        fine = seen[i] == 1;
                    EXPECT_TRUE(fine);
                }
}

TEST(Plan_StagedReduceChunksCoverTheMessageExactlyOnceAndFitTheirSlots) {
    const uint64_t lens[] = {1, 5, 1000, 70001, 300007};
    const uint32_t chunk_bytes[] = {4096, 16384, 65536, 262144};
    for (int n = 3; n <= 8; ++n)
        for (uint64_t len : lens)
            for (uint32_t elem : {1u, 2u, 4u, 8u})
                for (int ctas : {1, 4, 16, 128})
                    for (uint32_t cb : chunk_bytes) {
                        const ReducePlan pl = reduce_plan(len, n, ctas, cb, elem);
                        const uint64_t v16 = 16 / elem;
                        EXPECT_TRUE(pl.slice % v16 == 0 && pl.per_cta % v16 == 0 && pl.chunk_el * elem == cb);
                        std::vector<uint8_t> seen(len, 0);
                        bool fine = true;
                        for (int v = 0; v < n - 1; ++v)
                            for (int b = 0; b < ctas; ++b) {
                                bool ended = false;
                                for (uint32_t k = 0; k < pl.chunks; ++k) {
                                    uint64_t lo, hi;
                                    reduce_range(pl, len, b, v, k, &lo, &hi);
                                    if (hi < lo || (hi - lo) * elem > cb)
                                        fine = false;
                                    // once a chunk is empty, every later one is (the consumed-chunk
                                    // counters rely on it)
                                    if (hi == lo)
                                        ended = true;
                                    else if (ended)
                                        fine = false;
                                    // 16-byte alignment of every chunk start inside the message
                                    if (hi > lo && ((static_cast<uint64_t>(v) * pl.slice + lo) * elem) % 16 != 0)
                                        fine = false;
                                    for (uint64_t i = lo; i < hi; ++i) {
                                        const uint64_t at = static_cast<uint64_t>(v) * pl.slice + i;
                                        if (at >= len || seen[at]++)
                                            fine = false;
                                    }
                                }
                            }
                        for (uint64_t i = 0; i < len && fine; ++i)
                            fine = seen[i] == 1;
                        EXPECT_TRUE(fine);
                    }
}
