// The host side's bookkeeping, native: page pools, block tables and request slots of the cache
// manager, the scheduler's records and decisions, and the packing of a step's arrays.  Plain C++
// behind a C interface (called through ctypes like the kernels); it touches no device and runs on a
// machine without one.  The Python classes of `cache/pages.py`, `engine/scheduler.py` and
// `engine/batch.py` own the device tensors and the token lists and present these records under their
// documented names; the rules are the ones stated there and are pinned by the CPU tests.
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
#include <deque>
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

// ---- the scheduler's records --------------------------------------------------------------------------
// A request as the scheduler knows it: lengths and states, no token (the token lists stay with the
// caller).  `pending` counts a token that a launched step has sampled on the device and the host has
// not read yet: part of the request's length, not of its known tokens.
enum { ST_WAITING = 0, ST_RUNNING = 1, ST_FINISHED = 2 };
enum { FIN_NONE = 0, FIN_EOS = 1, FIN_LENGTH = 2, FIN_RELEASED = 3 };

struct Req {
    int32_t status = ST_WAITING, slot = -1, pending = 0, feedback_index = -1, preemptions = 0, finish = FIN_NONE, eos = -1;
    long long input_len = 0, prompt_len = 0, max_new = 0, generated = 0, cached_len = 0;
    long long extend_len() const { return input_len + pending - cached_len; }
    long long remain_len() const { return max_new - generated - pending; }   // tokens still to be sampled by steps not yet launched
};

struct Portion {
    int32_t id;
    long long num_tokens;
    int32_t samples, admitted;
};

struct Sched {
    Cache* cache;
    long long max_tokens, chunk, num_preemptions = 0;
    std::vector<Req> reqs;                                // by request id
    std::deque<int32_t> waiting;                          // first come first served; a preempted request goes to the front
    std::vector<int32_t> running;                         // in admission order

    // `need` plus what (slot or -1, new length) wants, into `need`; false if that exceeds the free pages
    // (or the request's limit), and `need` is then left as it was.
    bool reserve(std::vector<int32_t>& need, int slot, long long new_len, bool keep_anyway = false) const {
        if (new_len > cache->max_request_tokens && !keep_anyway) return false;
        std::vector<int32_t> total(need.size());
        bool ok = true;
        for (size_t g = 0; g < need.size(); ++g) {
            const Group& gr = cache->groups[g];
            total[g] = need[g] + (slot < 0 ? gr.pages_for(new_len) : gr.missing(slot, new_len));
            ok = ok && total[g] <= gr.pool.free_count();
        }
        if (ok || keep_anyway) need = total;
        return ok;
    }
    int release_slot(Req& r) {
        for (Group& g : cache->groups)
            if (int rc = g.release(r.slot)) return rc;
        cache->live[r.slot] = 0;
        cache->length[r.slot] = 0;
        cache->free_slots.push_back(r.slot);
        r.slot = -1;
        return HC_OK;
    }
    // Pages ran out for an older request: the most recently admitted running request gives back its
    // pages and its slot, keeps its tokens and goes to the front of the waiting queue.
    int preempt_latest(int32_t* victim) {
        *victim = running.back();
        running.pop_back();
        Req& r = reqs[*victim];
        if (int rc = release_slot(r)) return rc;
        r.cached_len = 0;
        r.status = ST_WAITING;
        ++r.preemptions;
        ++num_preemptions;
        waiting.push_front(*victim);
        return HC_OK;
    }
    bool has_work() const { return !waiting.empty() || !running.empty(); }
};

Pool* pool_of(void* p) { return static_cast<Pool*>(p); }
Cache* cache_of(void* p) { return static_cast<Cache*>(p); }
Sched* sched_of(void* p) { return static_cast<Sched*>(p); }

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

// ---- a step's entries at once ------------------------------------------------------------------------------
int hc_cache_lengths(void* cp, int n, const int32_t* slots, long long* out) {
    Cache* c = cache_of(cp);
    for (int i = 0; i < n; ++i) {
        if (int rc = c->check_live(slots[i])) return rc;
        out[i] = c->length[slots[i]];
    }
    return HC_OK;
}

// Room for positions [0, lens[i]) of every listed request, or nothing is taken.
int hc_cache_ensure_all(void* cp, int n, const int32_t* slots, const long long* lens) {
    Cache* c = cache_of(cp);
    std::vector<long long> need(c->groups.size(), 0);
    for (int i = 0; i < n; ++i) {
        if (int rc = c->check_live(slots[i])) return rc;
        if (lens[i] < c->length[slots[i]]) return fail(HC_MISUSE, "a request's cache never shrinks");
        if (lens[i] > c->max_request_tokens)
            return fail(HC_OUT_OF_PAGES, "a request of " + str(lens[i]) + " tokens exceeds the limit of " + str(c->max_request_tokens));
        for (size_t g = 0; g < c->groups.size(); ++g) {
            const Group& gr = c->groups[g];
            if (gr.pages_for(lens[i]) > gr.max_pages)
                return fail(HC_MISUSE, "a request of " + str(lens[i]) + " tokens needs " + str(gr.pages_for(lens[i])) + " pages; the table holds " + str(gr.max_pages));
            need[g] += gr.missing(slots[i], lens[i]);
        }
    }
    for (size_t g = 0; g < c->groups.size(); ++g)
        if (need[g] > c->groups[g].pool.free_count()) return fail(HC_OUT_OF_PAGES, "the step's tokens do not fit the free pages");
    for (int i = 0; i < n; ++i)
        for (Group& g : c->groups)
            if (int rc = g.append(slots[i], lens[i])) return rc;
    return HC_OK;
}

int hc_cache_commit_all(void* cp, int n, const int32_t* slots, const long long* lens, int* given) {
    *given = 0;
    for (int i = 0; i < n; ++i) {
        int one = 0;
        if (int rc = hc_cache_commit(cp, slots[i], lens[i], &one)) return rc;
        *given += one;
    }
    return HC_OK;
}

// ---- the scheduler ----------------------------------------------------------------------------------------
// Rules, every step: (1) running requests that decode go first, oldest admission first; (2) running
// requests still reading their prompt get a portion of at most `chunk` tokens within what is left of
// `max_tokens`; (3) waiting requests are admitted first come first served while a slot is free, budget
// is left and the pages of their first portion are free, stopping at the first that does not fit.
// When pages run out for a running request the most recently admitted one is preempted, again and
// again until the older one fits; no admission in a step that preempted.
void* hc_sched_new(void* cache, long long max_tokens, long long chunk) {
    if (max_tokens <= 0 || chunk <= 0) {
        fail(HC_MISUSE, "max_tokens_per_step and chunk must be positive");
        return nullptr;
    }
    Sched* s = new Sched();
    s->cache = cache_of(cache);
    s->max_tokens = max_tokens;
    s->chunk = std::min(chunk, max_tokens);
    return s;
}
void hc_sched_delete(void* s) { delete sched_of(s); }

int hc_sched_add(void* sp, long long prompt_len, long long max_new, int eos, int* id) {
    Sched* s = sched_of(sp);
    if (prompt_len <= 0) return fail(HC_MISUSE, "a request needs at least one prompt token");
    if (max_new < 0) return fail(HC_MISUSE, "max_new_tokens must be >= 0");
    const long long longest = prompt_len + std::max(max_new - 1, 0LL);   // the last sampled token is never run
    if (longest > s->cache->max_request_tokens)
        return fail(HC_OUT_OF_PAGES, "request needs " + str(longest) + " cached tokens; the cache takes at most " +
                                         str(s->cache->max_request_tokens) + " per request");
    Req r;
    r.input_len = r.prompt_len = prompt_len;
    r.max_new = max_new;
    r.eos = eos;
    *id = static_cast<int>(s->reqs.size());
    if (max_new == 0) {
        r.status = ST_FINISHED;
        r.finish = FIN_LENGTH;
    } else {
        s->waiting.push_back(*id);
    }
    s->reqs.push_back(r);
    return HC_OK;
}

int hc_sched_has_work(void* s) { return sched_of(s)->has_work() ? 1 : 0; }
long long hc_sched_num_preemptions(void* s) { return sched_of(s)->num_preemptions; }
int hc_sched_queue(void* sp, int which, int32_t* out, int cap) {     // which: 0 waiting, 1 running; returns the length
    Sched* s = sched_of(sp);
    int n = 0;
    if (which == 0) {
        for (int32_t id : s->waiting) { if (n < cap) out[n] = id; ++n; }
    } else {
        for (int32_t id : s->running) { if (n < cap) out[n] = id; ++n; }
    }
    return n;
}

// field: 0 status, 1 slot, 2 pending, 3 feedback_index, 4 preemptions, 5 finish reason, 6 cached_len,
// 7 input_len, 8 generated
long long hc_sched_get(void* sp, int id, int field) {
    const Req& r = sched_of(sp)->reqs[id];
    switch (field) {
        case 0: return r.status;
        case 1: return r.slot;
        case 2: return r.pending;
        case 3: return r.feedback_index;
        case 4: return r.preemptions;
        case 5: return r.finish;
        case 6: return r.cached_len;
        case 7: return r.input_len;
        default: return r.generated;
    }
}

// The next step: up to `cap` portions (request id, tokens, whether a token is sampled at its end, whether
// the request was admitted just now: its slot's state is the caller's to clear).
// `facts`: per portion {slot, tokens already cached, tokens known to the host, feedback index}, what the
// caller needs to build the step's entry without asking for each.
int hc_sched_schedule(void* sp, int32_t* ids, long long* num_tokens, int32_t* samples, int32_t* admitted, long long* facts, int cap,
                      int* count) {
    Sched* s = sched_of(sp);
    Cache* c = s->cache;
    long long budget = s->max_tokens;
    std::vector<Portion> plan;
    std::vector<int32_t> need(c->groups.size(), 0);       // pages per group already promised in this step
    bool preempted = false;
    std::vector<int32_t> queue(s->running);               // decoders first, each kind oldest first
    std::stable_sort(queue.begin(), queue.end(), [&](int32_t a, int32_t b) {
        return (s->reqs[a].extend_len() > 1) < (s->reqs[b].extend_len() > 1);
    });
    for (size_t i = 0; i < queue.size(); ++i) {
        Req& r = s->reqs[queue[i]];
        if (r.status != ST_RUNNING || r.remain_len() <= 0) continue;    // preempted below, or only awaiting its last token
        if (budget <= 0) break;
        const long long n = std::min({r.extend_len(), s->chunk, budget});
        bool fits;
        while (!(fits = s->reserve(need, r.slot, r.cached_len + n))) {
            int32_t victim;
            if (int rc = s->preempt_latest(&victim)) return rc;
            preempted = true;
            plan.erase(std::remove_if(plan.begin(), plan.end(), [&](const Portion& p) { return p.id == victim; }), plan.end());
            budget = s->max_tokens;
            std::fill(need.begin(), need.end(), 0);
            for (const Portion& p : plan) {               // the pool changed: count the promises again
                budget -= p.num_tokens;
                const Req& q = s->reqs[p.id];
                s->reserve(need, q.slot, q.cached_len + p.num_tokens, true);
            }
            if (victim == queue[i]) break;
        }
        if (!fits || r.status != ST_RUNNING) continue;
        plan.push_back({queue[i], n, n == r.extend_len() ? 1 : 0, 0});
        budget -= n;
    }
    // no admission in a step that had to preempt: the victim would come straight back
    while (!preempted && !s->waiting.empty() && budget > 0 && !c->free_slots.empty()) {
        const int32_t id = s->waiting.front();
        Req& r = s->reqs[id];
        if (r.remain_len() <= 0) break;                   // preempted with its last token on its way
        const long long n = std::min({r.extend_len(), s->chunk, budget});
        if (!s->reserve(need, -1, n)) break;
        s->waiting.pop_front();
        int slot;
        if (int rc = hc_cache_admit(c, &slot)) return rc;
        r.slot = slot;
        r.status = ST_RUNNING;
        s->running.push_back(id);
        plan.push_back({id, n, n == r.extend_len() ? 1 : 0, 1});
        budget -= n;
    }
    if (plan.empty() && s->has_work()) {
        bool any_pending = false;
        for (int32_t id : s->running) any_pending = any_pending || s->reqs[id].pending;
        for (int32_t id : s->waiting) any_pending = any_pending || s->reqs[id].pending;
        if (!any_pending) return fail(HC_OUT_OF_PAGES, "nothing can be scheduled: the cache is too small for the oldest request");
    }
    if (static_cast<int>(plan.size()) > cap) return fail(HC_MISUSE, "a plan of " + str(plan.size()) + " portions where " + str(cap) + " fit");
    for (size_t k = 0; k < plan.size(); ++k) {
        ids[k] = plan[k].id;
        num_tokens[k] = plan[k].num_tokens;
        samples[k] = plan[k].samples;
        admitted[k] = plan[k].admitted;
        const Req& r = s->reqs[plan[k].id];
        facts[4 * k] = r.slot;
        facts[4 * k + 1] = r.cached_len;
        facts[4 * k + 2] = r.input_len;
        facts[4 * k + 3] = r.feedback_index;
    }
    *count = static_cast<int>(plan.size());
    return HC_OK;
}

// The step of the plan has been launched: its tokens count as cached, and each portion that samples
// leaves a pending token (`feedback_index`: its place among the step's sampled tokens, in plan order).
void hc_sched_advance(void* sp, const int32_t* ids, const long long* num_tokens, const int32_t* samples, int n) {
    Sched* s = sched_of(sp);
    int k = 0;
    for (int i = 0; i < n; ++i) {
        Req& r = s->reqs[ids[i]];
        r.cached_len += num_tokens[i];
        if (samples[i]) {
            ++r.pending;                                  // two for a moment: the step before is read after this
            r.feedback_index = k++;
        }
    }
}

// The host has read the tokens of the step of the plan (one per sampling portion, in plan order): count
// them, finish requests (a token equal to the request's end-of-sequence id, when that is >= 0, finishes it
// and is kept; so does reaching max_new), free finished requests' pages and slots.  `kept[i]` says
// whether token i counts: a token sampled for a request that had already finished is dropped.
int hc_sched_deliver(void* sp, const int32_t* ids, const int32_t* samples, int n, const int32_t* tokens, int n_tokens, int32_t* kept) {
    Sched* s = sched_of(sp);
    int k = 0;
    for (int i = 0; i < n; ++i) {
        if (!samples[i]) continue;
        if (k >= n_tokens) return fail(HC_MISUSE, "fewer tokens than portions that sample");
        Req& r = s->reqs[ids[i]];
        const int32_t token = tokens[k];
        kept[k++] = 0;
        --r.pending;
        if (r.status == ST_FINISHED) continue;
        kept[k - 1] = 1;
        ++r.input_len;
        ++r.generated;
        if (r.eos >= 0 && token == r.eos) {
            r.finish = FIN_EOS;
        } else if (r.generated >= r.max_new) {
            r.finish = FIN_LENGTH;
        } else {
            continue;
        }
        const int32_t before = r.status;
        r.status = ST_FINISHED;
        if (before == ST_RUNNING) {
            s->running.erase(std::find(s->running.begin(), s->running.end(), ids[i]));
            if (int rc = s->release_slot(r)) return rc;
        } else {                                          // preempted while its last token was on its way
            auto it = std::find(s->waiting.begin(), s->waiting.end(), ids[i]);
            if (it != s->waiting.end()) s->waiting.erase(it);
        }
    }
    return HC_OK;
}

// Forget an unfinished request: out of the queues, its pages and slot freed (a token of it that a
// launched step is still sampling is dropped when it arrives).
int hc_sched_release(void* sp, int id) {
    Sched* s = sched_of(sp);
    Req& r = s->reqs[id];
    if (r.status == ST_FINISHED) return HC_OK;
    if (r.status == ST_RUNNING) {
        s->running.erase(std::find(s->running.begin(), s->running.end(), id));
        if (int rc = s->release_slot(r)) return rc;
    } else {
        auto it = std::find(s->waiting.begin(), s->waiting.end(), id);
        if (it != s->waiting.end()) s->waiting.erase(it);
    }
    r.status = ST_FINISHED;
    r.finish = FIN_RELEASED;
    return HC_OK;
}

// ---- packing a step -----------------------------------------------------------------------------------------
// The arrays every kernel of a step reads, written into the step's pinned buffer (`base`, int32) at the
// offsets the buffer's layout gives: per token its id, its absolute position and its entry; per entry its
// slot, first row, number of rows and cached length after the step; the rows whose logits are wanted
// (padded with row 0 up to `want_cap`, for a graph that reads that many) and their slots; counts
// {tokens, entries, wanted}.  A token id that is still on the device is written as -1 - (its index among
// the previous step's sampled tokens).  offsets: token_ids, positions, token_entry, entry_slot,
// entry_q_start, entry_q_len, entry_kv_len, want_rows, want_slot, counts.
// facts (out): tokens, wanted rows, longest portion, longest cached length.
int hc_pack_step(int32_t* base, const long long* offsets, int num_entries, const int32_t* slot, const long long* past,
                 const long long* q_len, const int32_t* feedback, const long long* tokens, const long long* want,
                 const int32_t* want_count, int want_cap, long long* facts) {
    int32_t* token_ids = base + offsets[0];
    int32_t* positions = base + offsets[1];
    int32_t* token_entry = base + offsets[2];
    int32_t* entry_slot = base + offsets[3];
    int32_t* entry_q_start = base + offsets[4];
    int32_t* entry_q_len = base + offsets[5];
    int32_t* entry_kv_len = base + offsets[6];
    int32_t* want_rows = base + offsets[7];
    int32_t* want_slot = base + offsets[8];
    int32_t* counts = base + offsets[9];
    long long t = 0, w = 0, wi = 0, max_q = 0, max_kv = 0;
    for (int e = 0; e < num_entries; ++e) {
        const long long n = q_len[e];
        entry_slot[e] = slot[e];
        entry_q_start[e] = static_cast<int32_t>(t);
        entry_q_len[e] = static_cast<int32_t>(n);
        entry_kv_len[e] = static_cast<int32_t>(past[e] + n);
        max_q = std::max(max_q, n);
        max_kv = std::max(max_kv, past[e] + n);
        for (long long i = 0; i < n; ++i) {
            token_ids[t + i] = static_cast<int32_t>(tokens[t + i]);
            positions[t + i] = static_cast<int32_t>(past[e] + i);
            token_entry[t + i] = e;
        }
        if (feedback[e] >= 0) token_ids[t + n - 1] = -1 - feedback[e];
        for (int k = 0; k < want_count[e]; ++k) {
            const long long j = want[wi++];
            if (j < 0 || j >= n) return fail(HC_MISUSE, "want=" + str(j) + " is outside the entry's " + str(n) + " tokens");
            want_rows[w] = static_cast<int32_t>(t + j);
            want_slot[w++] = slot[e];
        }
        t += n;
    }
    for (long long k = w; k < want_cap; ++k) want_rows[k] = 0;
    counts[0] = static_cast<int32_t>(t);
    counts[1] = num_entries;
    counts[2] = static_cast<int32_t>(w);
    facts[0] = t;
    facts[1] = w;
    facts[2] = max_q;
    facts[3] = max_kv;
    return HC_OK;
}

}  // extern "C"
