// The host side of the cache manager and of a step's descriptor, in C++: page pools, per-request page lists and
// lengths, all-or-nothing reservation, release of pages a window has passed, and the packing of a step's
// descriptor (rows, sequences, block tables) into the pinned buffers that travel to the device.
//
// One page-id space per group of layers with the same cache needs; free pages are reused in the order they came
// back (first in, first out), like the reference's host allocator
// (crates/forward/src/core/scratch.rs:602-703); a request for several pages is all-or-nothing.  A page of a group
// with a window W is given back after the step that makes it dead: a page whose last position is below
// length - W + 1 can be seen by no future query.  The reference bounds windowed layers with ring slabs instead
// and rejects paged windowed attention (crates/forward/src/core/composites/standard_attn.rs:436-441); its
// descriptor upload happens inside every layer (standard_attn.rs:315-329, 1133-1175).
//
// Plain C ABI for ctypes; a handle is one cache.  Functions return 0 or a negative error code and leave a message
// for fbh_last_error().  Nothing here touches the device.
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <deque>
#include <vector>

#define FBH_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

constexpr int ERR_PAGES = -10;      // not enough free pages (nothing was taken)
constexpr int ERR_STATE = -11;      // a page or slot is used against the rules
constexpr int ERR_LIMIT = -12;      // a request would outgrow its limit
constexpr int ERR_BATCH = -13;      // a step's entries are inconsistent

struct Pool {
    int n_pages = 0;
    std::deque<int> free_ids;
    std::vector<uint8_t> held;

    explicit Pool(int n) : n_pages(n), held((size_t)n, 0) {
        for (int p = 0; p < n; ++p) free_ids.push_back(p);
    }
    int n_free() const { return (int)free_ids.size(); }
    int take() {
        const int p = free_ids.front();
        free_ids.pop_front();
        held[(size_t)p] = 1;
        return p;
    }
    int give_back(int p) {
        if (p < 0 || p >= n_pages) return fail(ERR_STATE, "page id %d is outside the pool of %d", p, n_pages);
        if (!held[(size_t)p]) return fail(ERR_STATE, "page %d is given back but is not held", p);
        held[(size_t)p] = 0;
        free_ids.push_back(p);
        return 0;
    }
};

struct PageList {
    int base = 0;                   // logical pages below this index have been given back
    std::vector<int> ids;           // the live pages: ids[i] is logical page base + i
    int end() const { return base + (int)ids.size(); }    // logical pages [0, end()) have been taken so far
};

struct Record {
    bool live = false;
    int length = 0;                 // tokens whose keys are in the cache
    int reserved_to = 0;            // positions [0, reserved_to) have pages (where still live)
    std::vector<PageList> pages;    // per group
};

struct Cache {
    int page_size = 16, max_requests = 0, max_pages_per_request = 0;
    std::vector<Pool> pools;
    std::vector<int> windows;
    std::vector<Record> records;    // by slot
    std::vector<int> free_slots;    // a stack; the lowest slot on top at the start
    int n_groups() const { return (int)pools.size(); }
};

Cache* as_cache(void* h) { return static_cast<Cache*>(h); }

int check_slot(const Cache& c, int slot) {
    if (slot < 0 || slot >= c.max_requests || !c.records[(size_t)slot].live)
        return fail(ERR_STATE, "slot %d holds no request", slot);
    return 0;
}

}  // namespace

FBH_API const char* fbh_last_error() { return g_error; }

// n_pages[g], windows[g] (0 = all earlier keys stay live) per group.
FBH_API void* fbh_cache_new(int n_groups, const int* n_pages, const int* windows, int page_size, int max_requests,
                            int max_pages_per_request) {
    if (n_groups < 0 || page_size <= 0 || max_requests <= 0 || max_pages_per_request <= 0) {
        fail(ERR_STATE, "cache: bad geometry");
        return nullptr;
    }
    Cache* c = new Cache();
    c->page_size = page_size;
    c->max_requests = max_requests;
    c->max_pages_per_request = max_pages_per_request;
    for (int g = 0; g < n_groups; ++g) {
        if (n_pages[g] <= 0) {
            delete c;
            fail(ERR_STATE, "a page pool needs at least one page");
            return nullptr;
        }
        c->pools.emplace_back(n_pages[g]);
        c->windows.push_back(windows[g]);
    }
    c->records.resize((size_t)max_requests);
    for (int s = max_requests - 1; s >= 0; --s) c->free_slots.push_back(s);
    return c;
}

FBH_API void fbh_cache_free(void* h) { delete as_cache(h); }

FBH_API int fbh_has_slot(void* h) { return as_cache(h)->free_slots.empty() ? 0 : 1; }

// A fresh request: returns its slot, or a negative code when all slots are taken.
FBH_API int fbh_admit(void* h) {
    Cache& c = *as_cache(h);
    if (c.free_slots.empty()) return fail(ERR_STATE, "all %d request slots are taken", c.max_requests);
    const int slot = c.free_slots.back();
    c.free_slots.pop_back();
    Record& r = c.records[(size_t)slot];
    r.live = true;
    r.length = r.reserved_to = 0;
    r.pages.assign((size_t)c.n_groups(), PageList());
    return slot;
}

// A request that comes back from a snapshot: `length` tokens whose keys are to be put back, the pages below
// first_pages[g] of each group already given back when the snapshot was taken.  Takes a slot and the pages for
// logical pages [first_pages[g], ceil(length / page_size)) of every group, or nothing at all; returns the slot.
FBH_API int fbh_admit_at(void* h, int length, const int* first_pages) {
    Cache& c = *as_cache(h);
    if (c.free_slots.empty()) return fail(ERR_STATE, "all %d request slots are taken", c.max_requests);
    const int limit = c.max_pages_per_request * c.page_size;
    if (length < 0 || length > limit)
        return fail(ERR_LIMIT, "a request of %d tokens; the cache holds at most %d per request", length, limit);
    const int pages_to = (length + c.page_size - 1) / c.page_size;
    for (int g = 0; g < c.n_groups(); ++g) {
        if (first_pages[g] < 0 || first_pages[g] > pages_to)
            return fail(ERR_STATE, "group %d: first live page %d of a request of %d pages", g, first_pages[g], pages_to);
        const int want = pages_to - first_pages[g];
        if (want > c.pools[(size_t)g].n_free())
            return fail(ERR_PAGES, "%d cache pages wanted, %d of %d free", want, c.pools[(size_t)g].n_free(),
                        c.pools[(size_t)g].n_pages);
    }
    const int slot = c.free_slots.back();
    c.free_slots.pop_back();
    Record& r = c.records[(size_t)slot];
    r.live = true;
    r.length = r.reserved_to = length;
    r.pages.assign((size_t)c.n_groups(), PageList());
    for (int g = 0; g < c.n_groups(); ++g) {
        PageList& pl = r.pages[(size_t)g];
        pl.base = first_pages[g];
        while (pl.end() < pages_to) pl.ids.push_back(c.pools[(size_t)g].take());
    }
    return slot;
}

FBH_API int fbh_release(void* h, int slot) {
    Cache& c = *as_cache(h);
    if (int rc = check_slot(c, slot)) return rc;
    Record& r = c.records[(size_t)slot];
    for (int g = 0; g < c.n_groups(); ++g) {
        PageList& pl = r.pages[(size_t)g];
        for (int id : pl.ids)
            if (int rc = c.pools[(size_t)g].give_back(id)) return rc;
        pl = PageList();
    }
    r.live = false;
    c.free_slots.push_back(slot);
    return 0;
}

FBH_API int fbh_length(void* h, int slot) {
    Cache& c = *as_cache(h);
    if (int rc = check_slot(c, slot)) return rc;
    return c.records[(size_t)slot].length;
}

FBH_API int fbh_reserved_to(void* h, int slot) {
    Cache& c = *as_cache(h);
    if (int rc = check_slot(c, slot)) return rc;
    return c.records[(size_t)slot].reserved_to;
}

FBH_API int fbh_free_pages(void* h, int* out) {
    Cache& c = *as_cache(h);
    for (int g = 0; g < c.n_groups(); ++g) out[g] = c.pools[(size_t)g].n_free();
    return 0;
}

FBH_API int fbh_pool_pages(void* h, int group) { return as_cache(h)->pools[(size_t)group].n_pages; }

FBH_API int fbh_is_held(void* h, int group, int page) {
    Cache& c = *as_cache(h);
    if (page < 0 || page >= c.pools[(size_t)group].n_pages) return 0;
    return c.pools[(size_t)group].held[(size_t)page];
}

// Pages each group would have to take so that n_new more tokens of the request fit.
FBH_API int fbh_pages_needed(void* h, int slot, int n_new, int* out) {
    Cache& c = *as_cache(h);
    if (int rc = check_slot(c, slot)) return rc;
    const Record& r = c.records[(size_t)slot];
    const int want = (r.length + n_new + c.page_size - 1) / c.page_size;
    for (int g = 0; g < c.n_groups(); ++g) {
        const int have = r.pages[(size_t)g].end();
        out[g] = want > have ? want - have : 0;
    }
    return 0;
}

// The pages for positions [length, length + n_new[i]) of every request i in every group, or none at all.
// dry_run != 0 only answers whether the pools have the pages (0) or not (ERR_PAGES).
FBH_API int fbh_reserve_all(void* h, int n, const int* slots, const int* n_new, int dry_run) {
    Cache& c = *as_cache(h);
    const int G = c.n_groups();
    const int limit = c.max_pages_per_request * c.page_size;
    std::vector<int> total((size_t)G, 0);
    for (int i = 0; i < n; ++i) {
        if (int rc = check_slot(c, slots[i])) return rc;
        const Record& r = c.records[(size_t)slots[i]];
        const int end = r.length + n_new[i];
        if (!dry_run && end > limit)
            return fail(ERR_LIMIT, "a request would reach %d tokens; the cache holds at most %d per request", end, limit);
        const int pages_to = (end + c.page_size - 1) / c.page_size;
        for (int g = 0; g < G; ++g) {
            const int have = r.pages[(size_t)g].end();
            if (pages_to > have) total[(size_t)g] += pages_to - have;
        }
    }
    for (int g = 0; g < G; ++g)
        if (total[(size_t)g] > c.pools[(size_t)g].n_free())
            return fail(ERR_PAGES, "%d cache pages wanted, %d of %d free", total[(size_t)g], c.pools[(size_t)g].n_free(),
                        c.pools[(size_t)g].n_pages);
    if (dry_run) return 0;
    for (int i = 0; i < n; ++i) {
        Record& r = c.records[(size_t)slots[i]];
        const int end = r.length + n_new[i];
        const int pages_to = (end + c.page_size - 1) / c.page_size;
        for (int g = 0; g < G; ++g) {
            PageList& pl = r.pages[(size_t)g];
            while (pl.end() < pages_to) pl.ids.push_back(c.pools[(size_t)g].take());
        }
        if (end > r.reserved_to) r.reserved_to = end;
    }
    return 0;
}

// The step that wrote n_new[i] tokens of request i is launched: lengths advance, and pages that no later query can
// see go back to their pools.
FBH_API int fbh_commit(void* h, int n, const int* slots, const int* n_new) {
    Cache& c = *as_cache(h);
    for (int i = 0; i < n; ++i) {
        if (int rc = check_slot(c, slots[i])) return rc;
        Record& r = c.records[(size_t)slots[i]];
        if (r.length + n_new[i] > r.reserved_to)
            return fail(ERR_STATE, "%d tokens committed, %d reserved", r.length + n_new[i], r.reserved_to);
        r.length += n_new[i];
        for (int g = 0; g < c.n_groups(); ++g) {
            const int w = c.windows[(size_t)g];
            if (w <= 0) continue;
            const int first_live = r.length - w + 1;          // lowest position a future query can see
            PageList& pl = r.pages[(size_t)g];
            int dead = (first_live > 0 ? first_live : 0) / c.page_size;       // logical pages [0, dead) are dead
            if (dead > pl.end()) dead = pl.end();
            const int n_dead = dead - pl.base;
            if (n_dead > 0) {
                for (int i = 0; i < n_dead; ++i)
                    if (int rc = c.pools[(size_t)g].give_back(pl.ids[(size_t)i])) return rc;
                pl.ids.erase(pl.ids.begin(), pl.ids.begin() + n_dead);
                pl.base = dead;
            }
        }
    }
    return 0;
}

// The page ids of a request in a group by logical page index (-1 = given back): returns how many there are and
// copies the first `cap` of them.
FBH_API int fbh_pages(void* h, int slot, int group, int* out, int cap) {
    Cache& c = *as_cache(h);
    if (int rc = check_slot(c, slot)) return rc;
    const PageList& pl = c.records[(size_t)slot].pages[(size_t)group];
    const int n = pl.end();
    for (int i = 0; out && i < n && i < cap; ++i) out[i] = i < pl.base ? -1 : pl.ids[(size_t)(i - pl.base)];
    return n;
}

// The logical page index of the request's first live page in a group (what its table row starts at).
FBH_API int fbh_first_live_page(void* h, int slot, int group) {
    Cache& c = *as_cache(h);
    if (int rc = check_slot(c, slot)) return rc;
    return c.records[(size_t)slot].pages[(size_t)group].base;
}

// No page lost, held twice or free while in a table; no slot held twice.
FBH_API int fbh_check_invariants(void* h) {
    Cache& c = *as_cache(h);
    for (int g = 0; g < c.n_groups(); ++g) {
        const Pool& pool = c.pools[(size_t)g];
        std::vector<uint8_t> seen((size_t)pool.n_pages, 0);
        int n_seen = 0;
        for (const Record& r : c.records) {
            if (!r.live) continue;
            for (int p : r.pages[(size_t)g].ids) {
                if (p < 0 || p >= pool.n_pages) return fail(ERR_STATE, "group %d: page %d is outside the pool", g, p);
                if (seen[(size_t)p]) return fail(ERR_STATE, "group %d: page %d is held twice", g, p);
                if (!pool.held[(size_t)p]) return fail(ERR_STATE, "group %d: page %d is in a table but free in the pool", g, p);
                seen[(size_t)p] = 1;
                ++n_seen;
            }
        }
        const int n_held = pool.n_pages - pool.n_free();
        if (n_seen != n_held)
            return fail(ERR_STATE, "group %d: %d pages held in the pool, %d in tables (lost pages)", g, n_held, n_seen);
    }
    std::vector<uint8_t> slot_free((size_t)c.max_requests, 0);
    for (int s : c.free_slots) {
        if (slot_free[(size_t)s] || c.records[(size_t)s].live) return fail(ERR_STATE, "a request slot is held twice");
        slot_free[(size_t)s] = 1;
    }
    return 0;
}

// Packs the descriptor of one step.  Entry i: request in slots[i], its next q_len[i] tokens (tokens, concatenated),
// wanted places among them (wants, concatenated, n_want[i] each).  Pages for the new tokens must be reserved.
//   rows   [4][max_tokens]: token id, position, sequence of the row, rows whose logits are wanted
//   seqs   [5 + groups][max_seqs]: first row, rows, first position, slot, then for each group the logical page
//          index that column 0 of the sequence's table row stands for (its first live page), then the list of the
//          sequences that bring more than one token (info[4] of them)
//   tables [groups][max_seqs][max_pages]: the ids of the live pages, from the first live page on, -1 behind them
//   fill   [groups][max_seqs]: how many entries of each table row were valid after the last call (kept by the caller)
//   info   [5]: rows, wanted rows, longest entry, longest context, sequences with more than one token
FBH_API int fbh_build_step(void* h, int n_entries, const int* slots, const int* q_len, const int* tokens,
                           const int* n_want, const int* wants, int vocab, int max_tokens, int max_seqs, int max_pages,
                           int* rows, int* seqs, int* tables, int* fill, int* info) {
    Cache& c = *as_cache(h);
    if (n_entries <= 0) return fail(ERR_BATCH, "a step needs at least one entry");
    if (n_entries > max_seqs) return fail(ERR_BATCH, "%d entries in one step; the engine was built for %d", n_entries, max_seqs);
    long n = 0;
    for (int i = 0; i < n_entries; ++i) {
        if (int rc = check_slot(c, slots[i])) return rc;
        if (q_len[i] <= 0) return fail(ERR_BATCH, "a request brings no tokens");
        for (int j = 0; j < i; ++j)
            if (slots[j] == slots[i]) return fail(ERR_BATCH, "a request appears twice in one step");
        n += q_len[i];
    }
    if (n > max_tokens) return fail(ERR_BATCH, "the step has %ld tokens; the engine was built for %d a step", n, max_tokens);
    int* tok = rows;
    int* pos = rows + max_tokens;
    int* row_seq = rows + 2 * (size_t)max_tokens;
    int* out_rows = rows + 3 * (size_t)max_tokens;
    int row = 0, n_out = 0, w = 0, max_q = 0, max_kv = 0, n_multi = 0;
    int* multi = seqs + (size_t)(4 + c.n_groups()) * max_seqs;
    for (int i = 0; i < n_entries; ++i) {
        const Record& r = c.records[(size_t)slots[i]];
        const int k = q_len[i];
        if (r.length + k > r.reserved_to)
            return fail(ERR_BATCH, "entry %d: pages for positions up to %d are not reserved", i, r.length + k);
        for (int j = 0; j < k; ++j) {
            const int t = tokens[row + j];
            if (t < 0 || t >= vocab) return fail(ERR_BATCH, "token id outside [0, %d)", vocab);
            tok[row + j] = t;
            pos[row + j] = r.length + j;
            row_seq[row + j] = i;
        }
        for (int j = 0; j < n_want[i]; ++j) {
            const int place = wants[w + j];
            if (place < 0 || place >= k) return fail(ERR_BATCH, "entry %d: wanted place %d is outside its %d tokens", i, place, k);
            if (n_out >= max_tokens) return fail(ERR_BATCH, "more wanted rows than the engine was built for");
            out_rows[n_out++] = row + place;
        }
        w += n_want[i];
        seqs[i] = row;
        seqs[max_seqs + i] = k;
        seqs[2 * max_seqs + i] = r.length;
        seqs[3 * max_seqs + i] = slots[i];
        if (k > max_q) max_q = k;
        if (r.length + k > max_kv) max_kv = r.length + k;
        if (k > 1) multi[n_multi++] = i;
        for (int g = 0; g < c.n_groups(); ++g) {
            const PageList& pl = r.pages[(size_t)g];
            const std::vector<int>& ids = pl.ids;
            const int have = (int)ids.size();
            if (have > max_pages) return fail(ERR_BATCH, "entry %d holds %d live pages; tables have %d columns", i, have, max_pages);
            seqs[(size_t)(4 + g) * max_seqs + i] = pl.base;
            int* trow = tables + ((size_t)g * max_seqs + (size_t)i) * max_pages;
            memcpy(trow, ids.data(), sizeof(int) * (size_t)have);
            int& f = fill[(size_t)g * max_seqs + i];
            for (int p = have; p < f; ++p) trow[p] = -1;       // what an earlier step's request left in this row
            f = have;
        }
        row += k;
    }
    info[0] = (int)n;
    info[1] = n_out;
    info[2] = max_q;
    info[3] = max_kv;
    info[4] = n_multi;
    return 0;
}
