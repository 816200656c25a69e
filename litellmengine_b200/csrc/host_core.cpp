// The host side's bookkeeping, native: page pools, block tables and request slots of the cache
// manager.  Plain C++ behind a C interface (called through ctypes like the kernels); it touches no
// device and runs on a machine without one.  The Python classes of `cache/pages.py` own the device
// tensors and present these records under their documented names; the rules are the ones stated
// there and are pinned by the CPU tests.
//
// What is kept from the reference's block table manager (src/engine/block_table_manager.cpp:17-275):
// a last-in first-out free list that hands out 0, 1, 2, ... first (213-253), all-or-nothing `ensure`
// (60-89), errors on double free and bad ids (226-235, 270-274).  Not kept: one pool for everything
// and host tables that are packed and uploaded per layer per step; here a group of stages has its
// own pool and table, and only changed entries travel (`drain`).
//
// Every function returns 0, or 1 (out of pages or slots: nothing was taken) or 2 (a misuse); the
// message of the last failure of the calling thread is `hc_last_error()`.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

namespace {

enum { HC_OK = 0, HC_OUT_OF_PAGES = 1, HC_MISUSE = 2 };

thread_local std::string g_error;

int fail(int code, const std::string& message) {
    g_error = message;
    return code;
}

std::string str(long long v) { return std::to_string(v); }

struct Pool {
    int num_pages = 0;
    std::vector<int32_t> free_list;      // the back is handed out next
    std::vector<uint8_t> used;

    explicit Pool(int n) : num_pages(n), free_list(n), used(n, 0) {
        for (int i = 0; i < n; ++i) free_list[i] = n - 1 - i;
    }
    int free_count() const { return static_cast<int>(free_list.size()); }
    int take(int n, int32_t* out) {
        if (n < 0) return fail(HC_MISUSE, "cannot take a negative number of pages");
        if (n > free_count())
            return fail(HC_OUT_OF_PAGES, "not enough free pages: want " + str(n) + ", have " + str(free_count()) + " of " + str(num_pages));
        for (int i = 0; i < n; ++i) {
            out[i] = free_list.back();
            free_list.pop_back();
            used[out[i]] = 1;
        }
        return HC_OK;
    }
    int give(const int32_t* pages, int n) {              // checks everything first, then gives
        for (int i = 0; i < n; ++i) {
            if (pages[i] < 0 || pages[i] >= num_pages) return fail(HC_MISUSE, "page id " + str(pages[i]) + " is outside the pool");
            if (!used[pages[i]]) return fail(HC_MISUSE, "page " + str(pages[i]) + " freed twice");
        }
        for (int i = 0; i < n; ++i) {
            if (!used[pages[i]]) {                        // the same id earlier in this call
                for (int j = 0; j < i; ++j) {             // undo, so that a refused call changes nothing
                    used[pages[j]] = 1;
                    free_list.pop_back();
                }
                return fail(HC_MISUSE, "the same page given back twice in one call");
            }
            used[pages[i]] = 0;
            free_list.push_back(pages[i]);
        }
        return HC_OK;
    }
};

struct Group {
    int page_size, window, max_pages;                    // window < 0: every earlier position stays
    Pool pool;
    std::vector<int32_t> table;                          // [slots][max_pages], -1 where nothing is held
    std::vector<int32_t> first_held, num_logical;        // per slot: lowest logical page still held; pages ever appended
    std::vector<int32_t> pending_index, pending_value;   // table entries changed since the last drain

    Group(int page_size_, int window_, int num_pages, int slots, int max_pages_)
        : page_size(page_size_), window(window_), max_pages(max_pages_), pool(num_pages),
          table(static_cast<size_t>(slots) * max_pages_, -1), first_held(slots, 0), num_logical(slots, 0) {}

    int pages_for(long long length) const { return static_cast<int>((length + page_size - 1) / page_size); }
    int missing(int slot, long long new_len) const { return std::max(0, pages_for(new_len) - num_logical[slot]); }
    int append(int slot, long long new_len) {
        const int want = pages_for(new_len), have = num_logical[slot];
        if (want > max_pages)
            return fail(HC_MISUSE, "a request of " + str(new_len) + " tokens needs " + str(want) + " pages; the table holds " + str(max_pages));
        if (want <= have) return HC_OK;
        int32_t* row = table.data() + static_cast<size_t>(slot) * max_pages;
        const int rc = pool.take(want - have, row + have);
        if (rc != HC_OK) return rc;
        for (int i = have; i < want; ++i) {
            pending_index.push_back(slot * max_pages + i);
            pending_value.push_back(row[i]);
        }
        num_logical[slot] = want;
        return HC_OK;
    }
    // Pages every position of which lies before the window of the next query (position `length`,
    // which sees keys > length - window) go back.  Returns how many through `given`.
    int trim_window(int slot, long long length, int* given) {
        *given = 0;
        if (window < 0) return HC_OK;
        const long long first_needed = std::max(0LL, length - window + 1);
        const int keep_from = static_cast<int>(std::min<long long>(first_needed / page_size, num_logical[slot]));
        const int lo = first_held[slot];
        if (keep_from <= lo) return HC_OK;
        const int rc = pool.give(table.data() + static_cast<size_t>(slot) * max_pages + lo, keep_from - lo);
        if (rc != HC_OK) return rc;
        first_held[slot] = keep_from;
        *given = keep_from - lo;
        return HC_OK;
    }
    int release(int slot) {
        const int lo = first_held[slot], hi = num_logical[slot];
        const int rc = pool.give(table.data() + static_cast<size_t>(slot) * max_pages + lo, hi - lo);
        if (rc != HC_OK) return rc;
        first_held[slot] = num_logical[slot] = 0;
        return HC_OK;
    }
};

struct Cache {
    int max_slots, max_request_tokens;
    std::vector<Group> groups;
    std::vector<int32_t> free_slots;                     // the back is handed out next: 0, 1, 2, ... first
    std::vector<uint8_t> live;
    std::vector<long long> length;

    bool held(int slot) const { return slot >= 0 && slot < max_slots && live[slot]; }
    int check_live(int slot) const {
        return held(slot) ? HC_OK : fail(HC_MISUSE, "slot " + str(slot) + " is not held by a request");
    }
};

Pool* pool_of(void* p) { return static_cast<Pool*>(p); }
Cache* cache_of(void* p) { return static_cast<Cache*>(p); }

}  // namespace

extern "C" {

const char* hc_last_error() { return g_error.c_str(); }

// ---- a pool on its own -------------------------------------------------------------------------------
void* hc_pool_new(int num_pages) {
    if (num_pages <= 0) {
        fail(HC_MISUSE, "a page pool needs at least one page");
        return nullptr;
    }
    return new Pool(num_pages);
}
void hc_pool_delete(void* p) { delete pool_of(p); }
int hc_pool_num_pages(void* p) { return pool_of(p)->num_pages; }
int hc_pool_free_count(void* p) { return pool_of(p)->free_count(); }
int hc_pool_take(void* p, int n, int32_t* out) { return pool_of(p)->take(n, out); }
int hc_pool_give(void* p, const int32_t* pages, int n) { return pool_of(p)->give(pages, n); }
int hc_pool_used(void* p, int32_t* out) {                // ascending page ids; returns how many
    int k = 0;
    for (int i = 0; i < pool_of(p)->num_pages; ++i)
        if (pool_of(p)->used[i]) out[k++] = i;
    return k;
}

// ---- the cache manager's records ----------------------------------------------------------------------
void* hc_cache_new(int num_groups, const int32_t* windows, int page_size, int num_pages, int max_slots,
                   int max_pages_per_request, int max_request_tokens) {
    if (page_size <= 0 || num_pages <= 0 || max_slots <= 0 || num_groups < 0) {
        fail(HC_MISUSE, "page size, pages and slots must be positive");
        return nullptr;
    }
    Cache* c = new Cache();
    c->max_slots = max_slots;
    c->max_request_tokens = max_request_tokens;
    c->groups.reserve(num_groups);
    for (int g = 0; g < num_groups; ++g) c->groups.emplace_back(page_size, windows[g], num_pages, max_slots, max_pages_per_request);
    c->free_slots.resize(max_slots);
    for (int i = 0; i < max_slots; ++i) c->free_slots[i] = max_slots - 1 - i;
    c->live.assign(max_slots, 0);
    c->length.assign(max_slots, 0);
    return c;
}
void hc_cache_delete(void* c) { delete cache_of(c); }
void* hc_cache_pool(void* c, int g) { return &cache_of(c)->groups[g].pool; }
int32_t* hc_cache_table(void* c, int g) { return cache_of(c)->groups[g].table.data(); }
int32_t* hc_cache_first_held(void* c, int g) { return cache_of(c)->groups[g].first_held.data(); }
int32_t* hc_cache_num_logical(void* c, int g) { return cache_of(c)->groups[g].num_logical.data(); }
int hc_cache_free_slots(void* c) { return static_cast<int>(cache_of(c)->free_slots.size()); }
int hc_cache_is_live(void* c, int slot) { return cache_of(c)->held(slot) ? 1 : 0; }

int hc_cache_admit(void* cp, int* slot) {
    Cache* c = cache_of(cp);
    if (c->free_slots.empty()) return fail(HC_OUT_OF_PAGES, "no free request slot");
    *slot = c->free_slots.back();
    c->free_slots.pop_back();
    c->live[*slot] = 1;
    c->length[*slot] = 0;
    return HC_OK;
}

int hc_cache_length(void* cp, int slot, long long* length) {
    Cache* c = cache_of(cp);
    if (int rc = c->check_live(slot)) return rc;
    *length = c->length[slot];
    return HC_OK;
}

// The request is over (finished or preempted): every page and the slot go back.
int hc_cache_release(void* cp, int slot) {
    Cache* c = cache_of(cp);
    if (int rc = c->check_live(slot)) return rc;
    for (Group& g : c->groups)
        if (int rc = g.release(slot)) return rc;
    c->live[slot] = 0;
    c->length[slot] = 0;
    c->free_slots.push_back(slot);
    return HC_OK;
}

int hc_cache_pages_missing(void* cp, int slot, long long new_len, int32_t* out) {
    Cache* c = cache_of(cp);
    if (int rc = c->check_live(slot)) return rc;
    for (size_t g = 0; g < c->groups.size(); ++g) out[g] = c->groups[g].missing(slot, new_len);
    return HC_OK;
}

// Would `ensure` succeed for all of (slot, or -1 for a request not yet admitted; new length) together?
int hc_cache_can_hold(void* cp, int n, const int32_t* slots, const long long* lens, int* yes) {
    Cache* c = cache_of(cp);
    std::vector<long long> need(c->groups.size(), 0);
    int new_slots = 0;
    *yes = 0;
    for (int i = 0; i < n; ++i) {
        if (lens[i] > c->max_request_tokens) return HC_OK;
        if (slots[i] < 0) {
            ++new_slots;
            for (size_t g = 0; g < c->groups.size(); ++g) need[g] += c->groups[g].pages_for(lens[i]);
        } else {
            if (int rc = c->check_live(slots[i])) return rc;
            for (size_t g = 0; g < c->groups.size(); ++g) need[g] += c->groups[g].missing(slots[i], lens[i]);
        }
    }
    if (new_slots > static_cast<int>(c->free_slots.size())) return HC_OK;
    for (size_t g = 0; g < c->groups.size(); ++g)
        if (need[g] > c->groups[g].pool.free_count()) return HC_OK;
    *yes = 1;
    return HC_OK;
}

// `need` (pages per group already promised in this step) plus what (slot or -1, new length) wants, into
// `total`; `fits` says whether that is within the free pages.
int hc_cache_reserve(void* cp, const int32_t* need, int slot, long long new_len, int32_t* total, int* fits) {
    Cache* c = cache_of(cp);
    *fits = 0;
    if (new_len > c->max_request_tokens) return HC_OK;
    if (slot >= 0)
        if (int rc = c->check_live(slot)) return rc;
    bool ok = true;
    for (size_t g = 0; g < c->groups.size(); ++g) {
        total[g] = need[g] + (slot < 0 ? c->groups[g].pages_for(new_len) : c->groups[g].missing(slot, new_len));
        ok = ok && total[g] <= c->groups[g].pool.free_count();
    }
    *fits = ok ? 1 : 0;
    return HC_OK;
}

// Make room for positions [0, new_len) of the request, in every group, or take nothing.
int hc_cache_ensure(void* cp, int slot, long long new_len) {
    Cache* c = cache_of(cp);
    if (int rc = c->check_live(slot)) return rc;
    if (new_len < c->length[slot]) return fail(HC_MISUSE, "a request's cache never shrinks");
    if (new_len > c->max_request_tokens)
        return fail(HC_OUT_OF_PAGES, "a request of " + str(new_len) + " tokens exceeds the limit of " + str(c->max_request_tokens));
    for (Group& g : c->groups) {
        const int m = g.missing(slot, new_len);
        if (m > g.pool.free_count())
            return fail(HC_OUT_OF_PAGES, "not enough free pages: want " + str(m) + ", have " + str(g.pool.free_count()) + " of " + str(g.pool.num_pages));
        if (g.pages_for(new_len) > g.max_pages)
            return fail(HC_MISUSE, "a request of " + str(new_len) + " tokens needs " + str(g.pages_for(new_len)) + " pages; the table holds " + str(g.max_pages));
    }
    for (Group& g : c->groups)
        if (int rc = g.append(slot, new_len)) return rc;
    return HC_OK;
}

// The step that filled positions up to new_len has been issued: record the length and give back pages
// that a window has passed (`given`: how many).
int hc_cache_commit(void* cp, int slot, long long new_len, int* given) {
    Cache* c = cache_of(cp);
    *given = 0;
    if (int rc = c->check_live(slot)) return rc;
    if (new_len < c->length[slot]) return fail(HC_MISUSE, "a request's cache never shrinks");
    c->length[slot] = new_len;
    for (Group& g : c->groups) {
        int n = 0;
        if (int rc = g.trim_window(slot, new_len, &n)) return rc;
        *given += n;
    }
    return HC_OK;
}

int hc_cache_pending(void* c, int g) { return static_cast<int>(cache_of(c)->groups[g].pending_index.size()); }
void hc_cache_drain(void* c, int g, int32_t* index, int32_t* value) {
    Group& gr = cache_of(c)->groups[g];
    std::copy(gr.pending_index.begin(), gr.pending_index.end(), index);
    std::copy(gr.pending_value.begin(), gr.pending_value.end(), value);
    gr.pending_index.clear();
    gr.pending_value.clear();
}

// No page lost, none held twice, none both free and held; slots accounted for.
int hc_cache_check(void* cp) {
    Cache* c = cache_of(cp);
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        Group& g = c->groups[gi];
        std::vector<int> count(g.pool.num_pages, 0);
        int held = 0;
        for (int slot = 0; slot < c->max_slots; ++slot) {
            if (!c->live[slot]) {
                if (g.num_logical[slot] || g.first_held[slot])
                    return fail(HC_MISUSE, "group " + str(gi) + ": released slot " + str(slot) + " still has pages");
                continue;
            }
            for (int i = g.first_held[slot]; i < g.num_logical[slot]; ++i) {
                const int p = g.table[static_cast<size_t>(slot) * g.max_pages + i];
                if (p < 0 || p >= g.pool.num_pages) return fail(HC_MISUSE, "group " + str(gi) + ": slot " + str(slot) + " holds page id " + str(p));
                if (++count[p] > 1) return fail(HC_MISUSE, "group " + str(gi) + ": a page is held twice");
                ++held;
            }
        }
        for (int p = 0; p < g.pool.num_pages; ++p)
            if ((count[p] != 0) != (g.pool.used[p] != 0))
                return fail(HC_MISUSE, "group " + str(gi) + ": the pool and the requests disagree about page " + str(p));
        if (g.pool.free_count() + held != g.pool.num_pages)
            return fail(HC_MISUSE, "group " + str(gi) + ": " + str(g.pool.free_count()) + " free + " + str(held) + " held != " + str(g.pool.num_pages));
    }
    int live = 0;
    for (int s = 0; s < c->max_slots; ++s) live += c->live[s];
    std::vector<int32_t> sorted(c->free_slots);
    std::sort(sorted.begin(), sorted.end());
    if (live + static_cast<int>(sorted.size()) != c->max_slots || std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end())
        return fail(HC_MISUSE, "slot accounting is off");
    return HC_OK;
}

}  // extern "C"
