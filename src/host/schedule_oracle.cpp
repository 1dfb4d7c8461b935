#include "host/schedule_oracle.h"

#include <cstring>
#include <vector>

#include "host/cpu_reduce.h"
#include "megray/common.h"

namespace MegRay {
namespace host {

namespace {
inline int wrap(int v, int n) { return ((v % n) + n) % n; }
}  // namespace

Status ring_all_reduce_schedule(const void* const* in, void* const* out, int nranks, size_t len,
                                DType dtype, ReduceOp op) {
    if (nranks <= 0 || in == nullptr || out == nullptr || dtype == MEGRAY_CHAR)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t esz = get_dtype_size(dtype);
    // chunk c has len / n elements, the first len % n chunks one more
    std::vector<size_t> count(nranks, len / nranks), first(nranks, 0);
    for (size_t c = 0; c < len % nranks; ++c)
        ++count[c];
    for (int c = 1; c < nranks; ++c)
        first[c] = first[c - 1] + count[c - 1];
    // every rank starts from a copy of its own input
    std::vector<std::vector<char>> buf(nranks, std::vector<char>(len * esz));
    for (int r = 0; r < nranks; ++r)
        if (len)
            std::memcpy(buf[r].data(), in[r], len * esz);
    std::vector<std::vector<char>> wire(nranks);
    // reduce-scatter ring: in step i rank r passes chunk r-i to its right neighbour, which
    // combines it into its own copy of that chunk (own value first, received value second)
    for (int i = 0; i + 1 < nranks; ++i) {
        for (int r = 0; r < nranks; ++r) {
            const int c = wrap(r - i, nranks);
            wire[r].assign(buf[r].begin() + first[c] * esz, buf[r].begin() + (first[c] + count[c]) * esz);
        }
        for (int r = 0; r < nranks; ++r) {
            const int left = wrap(r - 1, nranks);
            const int c = wrap(r - i - 1, nranks);  // the chunk the left neighbour sent
            char* mine = buf[r].data() + first[c] * esz;
            Status s = cpu_reduce(mine, wire[left].data(), mine, count[c], dtype, op);
            if (s != MEGRAY_OK)
                return s;
        }
    }
    // all-gather ring: rank r owns the finished chunk r+1 and passes finished chunks on
    for (int i = 0; i + 1 < nranks; ++i) {
        for (int r = 0; r < nranks; ++r) {
            const int c = wrap(r + 1 - i, nranks);
            wire[r].assign(buf[r].begin() + first[c] * esz, buf[r].begin() + (first[c] + count[c]) * esz);
        }
        for (int r = 0; r < nranks; ++r) {
            const int left = wrap(r - 1, nranks);
            const int c = wrap(r - i, nranks);
            if (count[c])
                std::memcpy(buf[r].data() + first[c] * esz, wire[left].data(), count[c] * esz);
        }
    }
    for (int r = 0; r < nranks; ++r)
        if (len && out[r] != nullptr)
            std::memcpy(out[r], buf[r].data(), len * esz);
    return MEGRAY_OK;
}

Status tree_reduce_schedule(const void* const* in, void* out, int nranks, int root, size_t len,
                            DType dtype, ReduceOp op) {
    if (nranks <= 0 || root < 0 || root >= nranks || in == nullptr || out == nullptr ||
        dtype == MEGRAY_CHAR)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t esz = get_dtype_size(dtype);
    // positions are counted from the root (virtual rank 0 = root)
    std::vector<std::vector<char>> acc(nranks, std::vector<char>(len * esz));
    for (int v = 0; v < nranks; ++v)
        if (len)
            std::memcpy(acc[v].data(), in[wrap(v + root, nranks)], len * esz);
    // round with bit b: every position whose lower bits are zero and whose bit b is set hands
    // its partial result to the position with that bit cleared (received value first)
    for (int bit = 1; bit < nranks; bit <<= 1) {
        for (int v = 0; v < nranks; ++v) {
            if ((v & (bit - 1)) != 0 || (v & bit) != 0)
                continue;
            const int src = v | bit;
            if (src >= nranks)
                continue;
            Status s = cpu_reduce(acc[src].data(), acc[v].data(), acc[v].data(), len, dtype, op);
            if (s != MEGRAY_OK)
                return s;
        }
    }
    if (len)
        std::memcpy(out, acc[0].data(), len * esz);
    return MEGRAY_OK;
}

}  // namespace host
}  // namespace MegRay
