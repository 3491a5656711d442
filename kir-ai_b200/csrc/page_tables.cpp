// Host bookkeeping of the paged cache, native: page pools with free-list stacks, state slots,
// and per-request block tables for every group of cache layers.  Same rules as the Python
// classes in cache/pages.py (which remain as the readable model and are checked against this
// in the tests): a request's logical page p holds positions [p * page_size, (p + 1) * page_size);
// reserve() takes pages for the next tokens in every group or nothing; commit() records written
// tokens and gives back the pages of windowed groups that no later token can see; close() gives
// back everything.  The reference's allocator of this kind is BlockPool
// (crates/llm-kv-cache/src/block_pool.rs:158-171,630-670,740-760).
//
// C interface (every function returns >= 0 on success, a negative code on misuse):
//   -1 no slot / not enough pages (not an error: the caller decides), -2 unknown or closed request,
//   -3 request already live, -4 double free or bad page id, -5 tokens do not fit the reserved pages,
//   -6 bad argument.
#include <cstdint>
#include <unordered_map>
#include <vector>

namespace {

constexpr int NO_PAGE = -1;

struct Pool {
    int num_pages = 0;
    std::vector<int> free_list;  // stack: the page freed last is given out first
    std::vector<char> held;
    int high_water = 0;
    long handed_out = 0;  // pages given out since creation; more than num_pages means that pages were used again
    int used() const { return num_pages - (int)free_list.size(); }
};

struct Request {
    int slot = -1;
    long length = 0;
    long version = 0;
    std::vector<std::vector<int>> tables;  // per group
};

struct Tables {
    int page_size = 0;
    std::vector<long> windows;  // per group, -1: keeps everything
    std::vector<Pool> pools;
    std::vector<int> free_slots;
    std::vector<char> slot_held;
    std::unordered_map<long, Request> live;
};

long pages_for(const Tables& t, long tokens) { return (tokens + t.page_size - 1) / t.page_size; }

}  // namespace

#define KIRAI_HOST_EXPORT extern "C" __attribute__((visibility("default")))

KIRAI_HOST_EXPORT void* kirai_pages_create(int num_groups, const long* windows, int page_size, const int* num_pages, int num_slots) {
    if (num_groups < 0 || page_size <= 0 || num_slots <= 0) return nullptr;
    Tables* t = new Tables();
    t->page_size = page_size;
    for (int g = 0; g < num_groups; ++g) {
        if (num_pages[g] <= 0) { delete t; return nullptr; }
        t->windows.push_back(windows[g]);
        Pool pool;
        pool.num_pages = num_pages[g];
        pool.held.assign(num_pages[g], 0);
        for (int p = num_pages[g] - 1; p >= 0; --p) pool.free_list.push_back(p);
        t->pools.push_back(pool);
    }
    t->slot_held.assign(num_slots, 0);
    for (int s = num_slots - 1; s >= 0; --s) t->free_slots.push_back(s);
    return t;
}

KIRAI_HOST_EXPORT void kirai_pages_destroy(void* handle) { delete static_cast<Tables*>(handle); }

// Admits a request: returns its slot, -1 when no slot is free, -3 when the key is live already.
KIRAI_HOST_EXPORT int kirai_pages_open(void* handle, long key) {
    Tables& t = *static_cast<Tables*>(handle);
    if (t.live.count(key)) return -3;
    if (t.free_slots.empty()) return -1;
    Request request;
    request.slot = t.free_slots.back();
    t.free_slots.pop_back();
    t.slot_held[request.slot] = 1;
    request.tables.resize(t.pools.size());
    t.live.emplace(key, std::move(request));
    return t.live[key].slot;
}

// Pages each group must add for `new_tokens` more tokens; writes them to need[groups]. Returns 0 or -2.
KIRAI_HOST_EXPORT int kirai_pages_needed(void* handle, long key, long new_tokens, int* need) {
    Tables& t = *static_cast<Tables*>(handle);
    auto it = t.live.find(key);
    if (it == t.live.end()) return -2;
    const long total = pages_for(t, it->second.length + new_tokens);
    for (size_t g = 0; g < t.pools.size(); ++g) {
        const long extra = total - (long)it->second.tables[g].size();
        need[g] = extra > 0 ? (int)extra : 0;
    }
    return 0;
}

// 1 if reserve() would succeed, 0 if not.
KIRAI_HOST_EXPORT int kirai_pages_can_reserve(void* handle, long key, long new_tokens) {
    Tables& t = *static_cast<Tables*>(handle);
    auto it = t.live.find(key);
    if (it == t.live.end()) return -2;
    const long total = pages_for(t, it->second.length + new_tokens);
    for (size_t g = 0; g < t.pools.size(); ++g) {
        const long extra = total - (long)it->second.tables[g].size();
        if (extra > (long)t.pools[g].free_list.size()) return 0;
    }
    return 1;
}

// Takes the pages for the next `new_tokens` tokens in every group, or none: 1 taken, 0 not enough pages.
KIRAI_HOST_EXPORT int kirai_pages_reserve(void* handle, long key, long new_tokens) {
    if (new_tokens < 0) return -6;
    const int can = kirai_pages_can_reserve(handle, key, new_tokens);
    if (can != 1) return can;
    Tables& t = *static_cast<Tables*>(handle);
    Request& request = t.live[key];
    const long total = pages_for(t, request.length + new_tokens);
    for (size_t g = 0; g < t.pools.size(); ++g) {
        Pool& pool = t.pools[g];
        bool changed = false;
        while ((long)request.tables[g].size() < total) {
            const int page = pool.free_list.back();
            pool.free_list.pop_back();
            if (pool.held[page]) return -4;
            pool.held[page] = 1;
            ++pool.handed_out;
            request.tables[g].push_back(page);
            changed = true;
        }
        if (changed) ++request.version;
        if (pool.used() > pool.high_water) pool.high_water = pool.used();
    }
    return 1;
}

// Records `new_tokens` written tokens; windowed groups give back pages wholly before length - window + 1.
KIRAI_HOST_EXPORT int kirai_pages_commit(void* handle, long key, long new_tokens) {
    Tables& t = *static_cast<Tables*>(handle);
    auto it = t.live.find(key);
    if (it == t.live.end()) return -2;
    Request& request = it->second;
    const long new_length = request.length + new_tokens;
    for (size_t g = 0; g < t.pools.size(); ++g)
        if (new_length > (long)request.tables[g].size() * t.page_size) return -5;
    request.length = new_length;
    for (size_t g = 0; g < t.pools.size(); ++g) {
        if (t.windows[g] < 0) continue;
        const long first_visible = request.length - t.windows[g] + 1;
        if (first_visible <= 0) continue;
        long dead = first_visible / t.page_size;
        if (dead > (long)request.tables[g].size()) dead = (long)request.tables[g].size();
        bool changed = false;
        for (long p = 0; p < dead; ++p) {
            const int page = request.tables[g][p];
            if (page == NO_PAGE) continue;
            Pool& pool = t.pools[g];
            if (page < 0 || page >= pool.num_pages || !pool.held[page]) return -4;
            pool.held[page] = 0;
            pool.free_list.push_back(page);
            request.tables[g][p] = NO_PAGE;
            changed = true;
        }
        if (changed) ++request.version;
    }
    return 0;
}

KIRAI_HOST_EXPORT int kirai_pages_close(void* handle, long key) {
    Tables& t = *static_cast<Tables*>(handle);
    auto it = t.live.find(key);
    if (it == t.live.end()) return -2;
    Request& request = it->second;
    for (size_t g = 0; g < t.pools.size(); ++g) {
        Pool& pool = t.pools[g];
        for (int page : request.tables[g]) {
            if (page == NO_PAGE) continue;
            if (page < 0 || page >= pool.num_pages || !pool.held[page]) return -4;
            pool.held[page] = 0;
            pool.free_list.push_back(page);
        }
    }
    if (!t.slot_held[request.slot]) return -4;
    t.slot_held[request.slot] = 0;
    t.free_slots.push_back(request.slot);
    t.live.erase(it);
    return 0;
}

KIRAI_HOST_EXPORT long kirai_pages_length(void* handle, long key) {
    Tables& t = *static_cast<Tables*>(handle);
    auto it = t.live.find(key);
    return it == t.live.end() ? -2 : it->second.length;
}
KIRAI_HOST_EXPORT long kirai_pages_version(void* handle, long key) {
    Tables& t = *static_cast<Tables*>(handle);
    auto it = t.live.find(key);
    return it == t.live.end() ? -2 : it->second.version;
}
// Copies a request's block table of one group (NO_PAGE where given back); returns its length.
KIRAI_HOST_EXPORT int kirai_pages_table(void* handle, long key, int group, int* out, int capacity) {
    Tables& t = *static_cast<Tables*>(handle);
    auto it = t.live.find(key);
    if (it == t.live.end()) return -2;
    if (group < 0 || group >= (int)t.pools.size()) return -6;
    const std::vector<int>& table = it->second.tables[group];
    for (int i = 0; i < (int)table.size() && i < capacity; ++i) out[i] = table[i];
    return (int)table.size();
}
// Fills out[count][width] (row-major, NO_PAGE padded) with the block tables of `count` requests.
KIRAI_HOST_EXPORT int kirai_pages_fill_tables(void* handle, const long* keys, int count, int group, int* out, int width) {
    Tables& t = *static_cast<Tables*>(handle);
    if (group < 0 || group >= (int)t.pools.size()) return -6;
    for (int r = 0; r < count; ++r) {
        auto it = t.live.find(keys[r]);
        if (it == t.live.end()) return -2;
        const std::vector<int>& table = it->second.tables[group];
        if ((int)table.size() > width) return -6;
        int* row = out + (long)r * width;
        int i = 0;
        for (; i < (int)table.size(); ++i) row[i] = table[i];
        for (; i < width; ++i) row[i] = NO_PAGE;
    }
    return 0;
}
// what: 0 pages of the pool, 1 free, 2 used, 3 high water, 4 pages handed out since creation (saturating).  group < 0: slots (0 total, 1 free), live requests (2).
KIRAI_HOST_EXPORT int kirai_pages_stat(void* handle, int group, int what) {
    Tables& t = *static_cast<Tables*>(handle);
    if (group < 0) {
        if (what == 0) return (int)t.slot_held.size();
        if (what == 1) return (int)t.free_slots.size();
        if (what == 2) return (int)t.live.size();
        return -6;
    }
    if (group >= (int)t.pools.size()) return -6;
    const Pool& pool = t.pools[group];
    switch (what) {
        case 0: return pool.num_pages;
        case 1: return (int)pool.free_list.size();
        case 2: return pool.used();
        case 3: return pool.high_water;
        case 4: return pool.handed_out > 0x7fffffffL ? 0x7fffffff : (int)pool.handed_out;
    }
    return -6;
}
// 0 when every page is either free or held by exactly one live request, else the number of the check that failed.
KIRAI_HOST_EXPORT int kirai_pages_check(void* handle) {
    Tables& t = *static_cast<Tables*>(handle);
    for (size_t g = 0; g < t.pools.size(); ++g) {
        const Pool& pool = t.pools[g];
        std::vector<char> seen(pool.num_pages, 0);
        int held = 0;
        for (const auto& entry : t.live) {
            for (int page : entry.second.tables[g]) {
                if (page == NO_PAGE) continue;
                if (page < 0 || page >= pool.num_pages) return 1;
                if (seen[page]) return 2;  // held twice
                seen[page] = 1;
                ++held;
            }
        }
        if (held != pool.used()) return 3;  // a page lost
        for (int page : pool.free_list)
            if (seen[page] || pool.held[page]) return 4;  // a held page on the free list
    }
    return 0;
}
