// The KV pool's page allocator, native: a min-heap of the free page ids (the lowest free page is always the next one
// taken, the order the reference's pool keeps: inference/attention-state/code/pages.py:721-741), a reference count per
// page (forks share pages until one of them writes), and the floor (one past the highest page in use).  Host code only:
// no stream, no device memory; a pool's Python side keeps the page tables and asks here for pages, one at a time or for
// a whole step's rows at once.
#include <algorithm>
#include <cstdint>
#include <functional>
#include <new>
#include <queue>
#include <vector>

#include "../../include/crit_b200.h"

namespace {

struct Pager {
    std::priority_queue<int32_t, std::vector<int32_t>, std::greater<int32_t>> free;
    std::vector<int32_t> refs;
    int32_t floor = 0;
    int32_t shared = 0;              // pages held more than once

    explicit Pager(int32_t pages) : refs((size_t)pages, 0) {
        std::vector<int32_t> all((size_t)pages);
        for (int32_t i = 0; i < pages; ++i) all[(size_t)i] = i;
        free = decltype(free)(std::greater<int32_t>(), std::move(all));
    }
    int32_t take() {
        if (free.empty()) return -1;
        const int32_t page = free.top();
        free.pop();
        floor = std::max(floor, page + 1);
        refs[(size_t)page] = 1;
        return page;
    }
    int32_t drop(int32_t page) {
        int32_t& n = refs[(size_t)page];
        if (n <= 0) return -1;
        if (n == 2) --shared;
        if (--n == 0) {
            free.push(page);
            while (floor > 0 && refs[(size_t)floor - 1] == 0) --floor;
        }
        return n;
    }
};

inline Pager* pager(void* handle) { return static_cast<Pager*>(handle); }
inline bool held(const Pager* p, int32_t page) { return p && page >= 0 && (size_t)page < p->refs.size(); }

}  // namespace

#define CRIT_EXPORT extern "C" __attribute__((visibility("default")))

CRIT_EXPORT void* crit_b200_pager_create(int32_t pages) {
    if (pages < 1) return nullptr;
    return new (std::nothrow) Pager(pages);
}
CRIT_EXPORT void crit_b200_pager_destroy(void* handle) { delete pager(handle); }
CRIT_EXPORT int32_t crit_b200_pager_take(void* handle) { return handle ? pager(handle)->take() : -1; }
CRIT_EXPORT int32_t crit_b200_pager_drop(void* handle, int32_t page) { return held(pager(handle), page) ? pager(handle)->drop(page) : -1; }
CRIT_EXPORT int32_t crit_b200_pager_share(void* handle, int32_t page) {
    if (!held(pager(handle), page) || pager(handle)->refs[(size_t)page] <= 0) return -1;
    if (pager(handle)->refs[(size_t)page] == 1) ++pager(handle)->shared;
    return ++pager(handle)->refs[(size_t)page];
}
CRIT_EXPORT int32_t crit_b200_pager_shared(void* handle) { return handle ? pager(handle)->shared : -1; }
CRIT_EXPORT int32_t crit_b200_pager_refs(void* handle, int32_t page) { return held(pager(handle), page) ? pager(handle)->refs[(size_t)page] : -1; }
CRIT_EXPORT int32_t crit_b200_pager_free(void* handle) { return handle ? (int32_t)pager(handle)->free.size() : -1; }
CRIT_EXPORT int32_t crit_b200_pager_floor(void* handle) { return handle ? pager(handle)->floor : -1; }

// A step's rows grown at once: row i holds have[i] pages and needs need[i]; the pages it gains are taken in row order,
// lowest free page first, and written to `out` one row after another.  Returns how many were taken; when the pool runs
// out, -(taken + 1): the pages taken so far stay taken and are in `out` (the caller's tables hold them, as a loop of
// single takes would have left them).
CRIT_EXPORT int64_t crit_b200_pager_grow(void* handle, int32_t rows, const int32_t* have, const int32_t* need, int32_t* out,
                                         int64_t capacity) {
    if (!handle || rows < 0 || (rows > 0 && (!have || !need || !out))) return INT64_MIN;
    Pager* p = pager(handle);
    int64_t taken = 0;
    for (int32_t i = 0; i < rows; ++i)
        for (int32_t n = have[i]; n < need[i]; ++n) {
            if (taken >= capacity) return INT64_MIN;
            const int32_t page = p->take();
            if (page < 0) return -(taken + 1);
            out[taken++] = page;
        }
    return taken;
}
