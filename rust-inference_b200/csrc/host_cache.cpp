// Host-side bookkeeping of the cache: which slots are live, which pages each slot maps in each
// group of layers, how long each sequence is.  No device memory is touched here; the Python side
// copies the tables that changed to the device before a step's kernels run.
//
// The paged design is thanhauco/rust-inference's (src/kvcache.rs:12-61, 106-135): fixed pages of
// `page_size` tokens, a page table row per sequence with -1 for "unmapped", pages handed out from
// a free list as a sequence grows (lowest page first).  Added to it: a row is a *slot* that is
// given out and taken back per sequence, sequences grow by different amounts in one step (all of
// a step's growth happens or none of it), a slot's pages return to the free list when the slot is
// freed, groups of layers with a window give pages back as soon as no later query can see them.
//
// Plain C functions over opaque handles; a non-zero return code means that nothing was changed and
// `ri_last_error()` holds the message.  Not thread-safe: one cache, one thread.
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <vector>

static thread_local char ri_errbuf[512];
extern "C" const char* ri_last_error() { return ri_errbuf; }

static int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ri_errbuf, sizeof(ri_errbuf), fmt, ap);
    va_end(ap);
    return code;
}

// return codes (the Python side raises CacheError for 1, AssertionError for 2)
enum { RI_OK = 0, RI_CACHE_ERROR = 1, RI_BROKEN = 2 };

// ---- slots -----------------------------------------------------------------------------------
struct Slots {
    int n;
    std::vector<int> free_list;          // back() is given out next: slot 0 first
    std::vector<uint8_t> live;

    explicit Slots(int n_) : n(n_), live(n_, 0) {
        for (int s = n - 1; s >= 0; s--) free_list.push_back(s);
    }
    bool is_live(int s) const { return s >= 0 && s < n && live[s]; }
    int require_live(int s) const { return is_live(s) ? RI_OK : fail(RI_CACHE_ERROR, "slot %d is not live", s); }
    int alloc(int* out) {
        if (free_list.empty()) return fail(RI_CACHE_ERROR, "all %d cache slots are in use", n);
        *out = free_list.back();
        free_list.pop_back();
        live[*out] = 1;
        return RI_OK;
    }
    int release(int s) {
        if (int rc = require_live(s)) return rc;
        live[s] = 0;
        free_list.push_back(s);
        return RI_OK;
    }
    // every slot is either free or live, never both, never twice
    int check() const {
        std::vector<int> seen(n, 0);
        for (int s : free_list) {
            if (s < 0 || s >= n) return fail(RI_BROKEN, "the free list holds slot %d", s);
            if (seen[s]++) return fail(RI_BROKEN, "a slot is in the free list twice");
            if (live[s]) return fail(RI_BROKEN, "a slot is both free and live");
        }
        int n_live = 0;
        for (int s = 0; s < n; s++) n_live += live[s] ? 1 : 0;
        if ((int)free_list.size() + n_live != n) return fail(RI_BROKEN, "a slot was lost");
        return RI_OK;
    }
};

// ---- the pages of one group of layers ------------------------------------------------------------
struct Pages {
    int slots, pages, mpps, page_size, window;
    std::vector<int32_t> table;          // [slots, mpps], -1: unmapped
    std::vector<int> lens;               // tokens stored per slot
    std::vector<int> first_mapped;       // logical pages below it were released (window)
    std::vector<int> free_list;          // back() is given out next: page 0 first
    std::vector<uint8_t> dirty;          // slots whose row changed since the last clear

    Pages(int slots_, int pages_, int mpps_, int page_size_, int window_)
        : slots(slots_), pages(pages_), mpps(mpps_), page_size(page_size_), window(window_),
          table((size_t)slots_ * mpps_, -1), lens(slots_, 0), first_mapped(slots_, 0), dirty(slots_, 0) {
        for (int p = pages - 1; p >= 0; p--) free_list.push_back(p);
    }
    int32_t* row(int s) { return table.data() + (size_t)s * mpps; }
    const int32_t* row(int s) const { return table.data() + (size_t)s * mpps; }
    long long max_seq_len() const { return (long long)mpps * page_size; }

    // pages that extend(slot, n) would take from the free list
    int pages_needed(int s, int n) const {
        const long long start = lens[s], end = start + n;
        const long long last = std::min<long long>((end + page_size - 1) / page_size, mpps);
        int need = 0;
        for (long long p = start / page_size; p < last; p++) need += row(s)[p] < 0 ? 1 : 0;
        return need;
    }
    // maps pages for the next n positions of slot s and advances its length; nothing changes if it fails
    int extend(int s, int n, int* before) {
        if (s < 0 || s >= slots) return fail(RI_CACHE_ERROR, "slot %d is outside the cache's %d slots", s, slots);
        if (n < 0) return fail(RI_CACHE_ERROR, "a sequence cannot shrink");
        const long long start = lens[s], end = start + n;
        if (end > max_seq_len())
            return fail(RI_CACHE_ERROR, "slot %d would reach %lld tokens, the cache holds %lld per sequence", s, end, max_seq_len());
        const int need = pages_needed(s, n);
        if (need > (int)free_list.size())
            return fail(RI_CACHE_ERROR, "cache out of pages: %d needed, %d of %d free", need, (int)free_list.size(), pages);
        int32_t* r = row(s);
        for (long long p = start / page_size; p < (end + page_size - 1) / page_size; p++) {
            if (r[p] < 0) {
                r[p] = free_list.back();
                free_list.pop_back();
                dirty[s] = 1;
            }
        }
        lens[s] = (int)end;
        if (before) *before = (int)start;
        return RI_OK;
    }
    // gives back the pages that no later query of slot s can see (groups with a window)
    int release_behind_window(int s) {
        if (window <= 0) return 0;
        const long long first_needed = (long long)lens[s] - window + 1;      // oldest key the next query reads
        int32_t* r = row(s);
        int n = 0, p = first_mapped[s];
        while ((long long)(p + 1) * page_size <= first_needed) {
            if (r[p] >= 0) {
                free_list.push_back(r[p]);
                r[p] = -1;
                n++;
            }
            p++;
        }
        first_mapped[s] = p;
        if (n) dirty[s] = 1;
        return n;
    }
    // gives back every page of slot s and resets its length
    void release(int s) {
        int32_t* r = row(s);
        bool any = false;
        for (int p = mpps - 1; p >= 0; p--) {       // the highest page first, so that the lowest is handed out first again
            if (r[p] >= 0) {
                free_list.push_back(r[p]);
                r[p] = -1;
                any = true;
            }
        }
        if (any) dirty[s] = 1;
        lens[s] = 0;
        first_mapped[s] = 0;
    }
    // every page is free or mapped exactly once
    int check() const {
        std::vector<int> seen(pages, 0);
        size_t mapped = 0;
        for (int32_t p : table) {
            if (p < 0) continue;
            if (p >= pages) return fail(RI_BROKEN, "the table maps page %d of %d", (int)p, pages);
            if (seen[p]++) return fail(RI_BROKEN, "a page is mapped twice");
            mapped++;
        }
        std::vector<int> in_free(pages, 0);
        for (int p : free_list) {
            if (p < 0 || p >= pages) return fail(RI_BROKEN, "the free list holds page %d", p);
            if (in_free[p]++) return fail(RI_BROKEN, "a page is in the free list twice");
            if (seen[p]) return fail(RI_BROKEN, "a page is both free and mapped");
        }
        if (mapped + free_list.size() != (size_t)pages) return fail(RI_BROKEN, "a page was lost");
        return RI_OK;
    }
};

// ---- the whole cache: slots, one Pages per group of layers, the sequences' lengths ----------------
struct HostCache {
    Slots slots;
    std::vector<Pages> groups;
    std::vector<int> lens;
    int mpps, page_size;
    std::vector<int> stamp;              // per slot: the step that named it last (a slot twice in one step)
    int step = 0;

    HostCache(int num_slots, int num_pages, int mpps_, int page_size_, int n_groups, const int* windows)
        : slots(num_slots), lens(num_slots, 0), mpps(mpps_), page_size(page_size_), stamp(num_slots, 0) {
        for (int g = 0; g < n_groups; g++) groups.emplace_back(num_slots, num_pages, mpps_, page_size_, windows[g]);
    }
    long long max_seq_len() const { return (long long)mpps * page_size; }

    // (slot, new tokens) for every sequence of a step: maps the pages in every group and gives each
    // sequence's length before.  Either all of it happens or none.
    int extend(int n, const int* slot, const int* news, int* before) {
        step++;
        for (int i = 0; i < n; i++) {
            if (int rc = slots.require_live(slot[i])) return rc;
            if (stamp[slot[i]] == step) return fail(RI_CACHE_ERROR, "slot %d appears twice in one step", slot[i]);
            stamp[slot[i]] = step;
            if (news[i] <= 0) return fail(RI_CACHE_ERROR, "every sequence of a step brings at least one token");
            if ((long long)lens[slot[i]] + news[i] > max_seq_len())
                return fail(RI_CACHE_ERROR, "slot %d would reach %lld tokens, the cache holds %lld per sequence", slot[i],
                            (long long)lens[slot[i]] + news[i], max_seq_len());
        }
        for (const Pages& g : groups) {
            long long need = 0;
            for (int i = 0; i < n; i++) need += g.pages_needed(slot[i], news[i]);
            if (need > (long long)g.free_list.size())
                return fail(RI_CACHE_ERROR, "cache out of pages: this step needs %lld, %d of %d are free", need,
                            (int)g.free_list.size(), g.pages);
        }
        for (int i = 0; i < n; i++) {
            for (Pages& g : groups)
                if (g.extend(slot[i], news[i], nullptr) != RI_OK) return RI_BROKEN;      // cannot happen after the checks above
            before[i] = lens[slot[i]];
            lens[slot[i]] += news[i];
        }
        return RI_OK;
    }
};

template <typename T>
static T* as(void* h) { return static_cast<T*>(h); }

extern "C" {

// ---- slots alone (used by the tests of the allocator) ---------------------------------------------
void* ri_slots_create(int n) {
    if (n <= 0) {
        fail(RI_CACHE_ERROR, "the cache needs at least one slot");
        return nullptr;
    }
    return new Slots(n);
}
void ri_slots_destroy(void* h) { delete as<Slots>(h); }
int ri_slots_alloc(void* h, int* out) { return as<Slots>(h)->alloc(out); }
int ri_slots_free(void* h, int s) { return as<Slots>(h)->release(s); }
int ri_slots_is_live(void* h, int s) { return as<Slots>(h)->is_live(s) ? 1 : 0; }
int ri_slots_require_live(void* h, int s) { return as<Slots>(h)->require_live(s); }
int ri_slots_live_count(void* h) { return as<Slots>(h)->n - (int)as<Slots>(h)->free_list.size(); }
int ri_slots_check(void* h) { return as<Slots>(h)->check(); }

// ---- one group's pages alone ----------------------------------------------------------------------
void* ri_pages_create(int slots, int pages, int mpps, int page_size, int window) {
    if (slots <= 0 || pages <= 0 || mpps <= 0 || page_size <= 0) {
        fail(RI_CACHE_ERROR, "page counts and the page size must be positive");
        return nullptr;
    }
    return new Pages(slots, pages, mpps, page_size, window);
}
void ri_pages_destroy(void* h) { delete as<Pages>(h); }
int32_t* ri_pages_table(void* h) { return as<Pages>(h)->table.data(); }
int ri_pages_free(void* h) { return (int)as<Pages>(h)->free_list.size(); }
int ri_pages_len(void* h, int s) { return as<Pages>(h)->lens[s]; }
int ri_pages_needed(void* h, int s, int n) { return as<Pages>(h)->pages_needed(s, n); }
int ri_pages_extend(void* h, int s, int n, int* before) { return as<Pages>(h)->extend(s, n, before); }
int ri_pages_release_behind_window(void* h, int s) { return as<Pages>(h)->release_behind_window(s); }
void ri_pages_release(void* h, int s) { as<Pages>(h)->release(s); }
int ri_pages_check(void* h) { return as<Pages>(h)->check(); }
// the slots whose rows changed since the last call, at most `cap` of them written to `out`; the marks are cleared
int ri_pages_take_dirty(void* h, int* out, int cap) {
    Pages* p = as<Pages>(h);
    int n = 0;
    for (int s = 0; s < p->slots; s++) {
        if (!p->dirty[s]) continue;
        if (n < cap) out[n] = s;
        n++;
        p->dirty[s] = 0;
    }
    return n;
}

// ---- the whole cache ------------------------------------------------------------------------------
void* ri_cache_create(int num_slots, int num_pages, int mpps, int page_size, int n_groups, const int* windows) {
    if (num_slots <= 0) {
        fail(RI_CACHE_ERROR, "the cache needs at least one slot");
        return nullptr;
    }
    if (num_pages <= 0 || mpps <= 0 || page_size <= 0 || n_groups < 0) {
        fail(RI_CACHE_ERROR, "page counts and the page size must be positive");
        return nullptr;
    }
    return new HostCache(num_slots, num_pages, mpps, page_size, n_groups, windows);
}
void ri_cache_destroy(void* h) { delete as<HostCache>(h); }
void* ri_cache_slots(void* h) { return &as<HostCache>(h)->slots; }
void* ri_cache_group(void* h, int g) { return &as<HostCache>(h)->groups[g]; }
int ri_cache_alloc_slot(void* h, int* out) {
    HostCache* c = as<HostCache>(h);
    if (int rc = c->slots.alloc(out)) return rc;
    c->lens[*out] = 0;
    return RI_OK;
}
int ri_cache_free_slot(void* h, int s) {
    HostCache* c = as<HostCache>(h);
    if (int rc = c->slots.release(s)) return rc;
    for (Pages& g : c->groups) g.release(s);
    c->lens[s] = 0;
    return RI_OK;
}
int ri_cache_length(void* h, int s, int* out) {
    HostCache* c = as<HostCache>(h);
    if (int rc = c->slots.require_live(s)) return rc;
    *out = c->lens[s];
    return RI_OK;
}
int ri_cache_extend(void* h, int n, const int* slot, const int* news, int* before) {
    return as<HostCache>(h)->extend(n, slot, news, before);
}
// after a step: releases what no later step can read (pages behind a window)
void ri_cache_after_step(void* h, int n, const int* slot) {
    for (Pages& g : as<HostCache>(h)->groups)
        if (g.window > 0)
            for (int i = 0; i < n; i++) g.release_behind_window(slot[i]);
}
int ri_cache_free_pages(void* h, int if_no_group) {
    HostCache* c = as<HostCache>(h);
    int least = if_no_group;
    bool first = true;
    for (const Pages& g : c->groups) {
        if (first || (int)g.free_list.size() < least) least = (int)g.free_list.size();
        first = false;
    }
    return least;
}
int ri_cache_check(void* h) {
    HostCache* c = as<HostCache>(h);
    if (int rc = c->slots.check()) return rc;
    for (const Pages& g : c->groups) {
        if (int rc = g.check()) return rc;
        for (int s = 0; s < c->slots.n; s++) {
            if (c->slots.is_live(s)) continue;
            for (int p = 0; p < g.mpps; p++)
                if (g.row(s)[p] >= 0) return fail(RI_BROKEN, "free slot %d still maps pages", s);
        }
    }
    return RI_OK;
}

}  // extern "C"
