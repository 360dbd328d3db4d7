// Host-side runtime of the cache manager and the step's batch, in C++: page pools with free lists
// per cache group, a block table per request and group, slots for per-request state, and the
// packing of one step (reserve pages for all its tokens, all or nothing; then write tokens,
// positions, lengths and block tables into one int32 buffer that goes to the device in one copy).
// No tensor lives here and nothing touches a GPU; the Python classes of cache/manager.py and
// engine/engine.py call these functions through ctypes.
//
// The bookkeeping follows the reference's PagedKVCache and PageAllocator
// (src/core/paging/paged_kv_cache.h:47-71, 96-107, 196-208: LIFO free list, one block table per
// sequence, rewind gives the tail pages back), without reference counts (pages are never shared),
// with one pool per group of layers and with the release of pages that a window has passed.
#include <cstdint>
#include <cstring>
#include <vector>

#define BWH_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

enum : int {
    BWH_OK = 0, BWH_NO_SLOT = -1, BWH_OUT_OF_PAGES = -2, BWH_BAD_ARG = -3, BWH_WINDOW_RELEASED = -4,
    BWH_BAD_TOKEN = -5, BWH_BAD_WANT = -6, BWH_TOO_SMALL = -7, BWH_TOO_MANY_TOKENS = -8, BWH_TWICE = -9,
    BWH_PAGE_HELD_TWICE = -20, BWH_PAGE_LOST = -21, BWH_HELD_PAGE_FREE = -22, BWH_FREED_TWICE = -23
};

struct Group {
    int window = 0;                 // 0: every key is kept
    int num_pages = 0;
    std::vector<int> free;          // LIFO: back() is handed out next
    std::vector<uint8_t> is_free;
};

struct Request {
    bool live = false;
    int slot = -1;
    long long length = 0;
    std::vector<std::vector<int>> blocks;   // per group: page id, or -1 once given back
    std::vector<int> first_live;            // per group: first block still held
};

struct Cache {
    int page_size = 0, max_requests = 0;
    std::vector<Group> groups;
    std::vector<int> free_slots;
    std::vector<uint8_t> slot_free;
    std::vector<Request> requests;          // index = handle
    std::vector<int> free_handles;
    std::vector<int> mark;                  // scratch for pack_step's duplicate check
};

inline long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

inline Request* get(Cache* c, int h) {
    if (h < 0 || h >= (int)c->requests.size() || !c->requests[h].live) return nullptr;
    return &c->requests[h];
}

int first_needed_block(const Cache* c, const Group& g, long long q_start) {
    if (g.window <= 0) return 0;
    const long long first_key = q_start - g.window + 1;
    return first_key > 0 ? (int)(first_key / c->page_size) : 0;
}

// pages a group must still hand out for the request to reach `new_length`
inline int pages_short(const Cache* c, const Request& r, int gi, long long new_length) {
    const long long total = ceil_div(new_length, c->page_size);
    const long long have = (long long)r.blocks[gi].size();
    return total > have ? (int)(total - have) : 0;
}

int free_pages_of(Group& g, const int* pages, int n) {
    for (int i = 0; i < n; ++i) {
        const int p = pages[i];
        if (p < 0 || p >= g.num_pages) return BWH_BAD_ARG;
        if (g.is_free[p]) return BWH_FREED_TWICE;
    }
    for (int i = 0; i < n; ++i) { g.is_free[pages[i]] = 1; g.free.push_back(pages[i]); }
    return BWH_OK;
}

int add_request(Cache* c) {
    if (c->free_slots.empty()) return BWH_NO_SLOT;
    int h;
    if (!c->free_handles.empty()) { h = c->free_handles.back(); c->free_handles.pop_back(); }
    else { h = (int)c->requests.size(); c->requests.emplace_back(); }
    Request& r = c->requests[h];
    r.live = true;
    r.slot = c->free_slots.back(); c->free_slots.pop_back();
    c->slot_free[r.slot] = 0;
    r.length = 0;
    r.blocks.assign(c->groups.size(), {});
    r.first_live.assign(c->groups.size(), 0);
    return h;
}

// grows the request; the caller has checked that every group has the pages
void grow(Cache* c, Request& r, long long n_new) {
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        Group& g = c->groups[gi];
        for (int k = pages_short(c, r, (int)gi, r.length + n_new); k > 0; --k) {
            const int p = g.free.back(); g.free.pop_back();
            g.is_free[p] = 0;
            r.blocks[gi].push_back(p);
        }
    }
    r.length += n_new;
}

}  // namespace

// windows[g] <= 0: no window.  Returns the cache, or null on bad sizes.
BWH_EXPORT void* bwh_create(int n_groups, const int* windows, const int* num_pages, int page_size, int max_requests) {
    if (n_groups < 0 || page_size <= 0 || max_requests <= 0) return nullptr;
    for (int g = 0; g < n_groups; ++g) if (num_pages[g] <= 0) return nullptr;
    Cache* c = new Cache();
    c->page_size = page_size; c->max_requests = max_requests;
    c->groups.resize(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        Group& G = c->groups[g];
        G.window = windows[g] > 0 ? windows[g] : 0;
        G.num_pages = num_pages[g];
        G.free.resize(num_pages[g]);
        for (int p = 0; p < num_pages[g]; ++p) G.free[p] = num_pages[g] - 1 - p;   // page 0 goes out first
        G.is_free.assign(num_pages[g], 1);
    }
    c->free_slots.resize(max_requests);
    for (int s = 0; s < max_requests; ++s) c->free_slots[s] = max_requests - 1 - s;
    c->slot_free.assign(max_requests, 1);
    return c;
}

BWH_EXPORT void bwh_destroy(void* cache) { delete (Cache*)cache; }

// A new request: a handle (>= 0) with a state slot, or BWH_NO_SLOT.
BWH_EXPORT int bwh_add_request(void* cache) { return add_request((Cache*)cache); }

BWH_EXPORT int bwh_slot(void* cache, int h) { Request* r = get((Cache*)cache, h); return r ? r->slot : BWH_BAD_ARG; }
BWH_EXPORT long long bwh_length(void* cache, int h) { Request* r = get((Cache*)cache, h); return r ? r->length : BWH_BAD_ARG; }
BWH_EXPORT int bwh_free_slots(void* cache) { return (int)((Cache*)cache)->free_slots.size(); }

BWH_EXPORT int bwh_free_pages(void* cache, int* out) {
    Cache* c = (Cache*)cache;
    for (size_t g = 0; g < c->groups.size(); ++g) out[g] = (int)c->groups[g].free.size();
    return BWH_OK;
}

// Pages each group must still hand out for the request to grow by n_new tokens.
BWH_EXPORT int bwh_pages_needed(void* cache, int h, long long n_new, int* out) {
    Cache* c = (Cache*)cache;
    Request* r = get(c, h);
    if (!r || n_new < 0) return BWH_BAD_ARG;
    for (size_t g = 0; g < c->groups.size(); ++g) out[g] = pages_short(c, *r, (int)g, r->length + n_new);
    return BWH_OK;
}

// The same for R requests that each grow by n_new tokens: the sums per group.
BWH_EXPORT int bwh_pages_needed_many(void* cache, int R, const int* handles, long long n_new, int* out) {
    Cache* c = (Cache*)cache;
    if (R < 0 || n_new < 0) return BWH_BAD_ARG;
    for (size_t g = 0; g < c->groups.size(); ++g) out[g] = 0;
    for (int i = 0; i < R; ++i) {
        Request* r = get(c, handles[i]);
        if (!r) return BWH_BAD_ARG;
        for (size_t g = 0; g < c->groups.size(); ++g) out[g] += pages_short(c, *r, (int)g, r->length + n_new);
    }
    return BWH_OK;
}

// Grows the request by n_new tokens: its old length, or BWH_OUT_OF_PAGES with nothing changed.
BWH_EXPORT long long bwh_append(void* cache, int h, long long n_new) {
    Cache* c = (Cache*)cache;
    Request* r = get(c, h);
    if (!r || n_new <= 0) return BWH_BAD_ARG;
    for (size_t g = 0; g < c->groups.size(); ++g)
        if (pages_short(c, *r, (int)g, r->length + n_new) > (int)c->groups[g].free.size()) return BWH_OUT_OF_PAGES;
    const long long old = r->length;
    grow(c, *r, n_new);
    return old;
}

// Gives back the pages that every later query's window has passed; returns how many.
BWH_EXPORT int bwh_release_passed(void* cache, int h) {
    Cache* c = (Cache*)cache;
    Request* r = get(c, h);
    if (!r) return BWH_BAD_ARG;
    int freed = 0;
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        Group& g = c->groups[gi];
        if (g.window <= 0) continue;
        const int keep_from = first_needed_block(c, g, r->length);   // the next query sits at position `length`
        int& first = r->first_live[gi];
        for (int i = first; i < keep_from && i < (int)r->blocks[gi].size(); ++i) {
            int& p = r->blocks[gi][i];
            if (p >= 0) { const int rc = free_pages_of(g, &p, 1); if (rc) return rc; ++freed; p = -1; }
        }
        if (keep_from > first) first = keep_from;
    }
    return freed;
}

// Rolls the request back to new_length tokens and gives back the pages behind it.
BWH_EXPORT int bwh_truncate(void* cache, int h, long long new_length) {
    Cache* c = (Cache*)cache;
    Request* r = get(c, h);
    if (!r || new_length < 0 || new_length > r->length) return BWH_BAD_ARG;
    const long long keep = ceil_div(new_length, c->page_size);
    for (size_t gi = 0; gi < c->groups.size(); ++gi)
        if (c->groups[gi].window > 0 && r->first_live[gi] > first_needed_block(c, c->groups[gi], new_length))
            return BWH_WINDOW_RELEASED;
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        std::vector<int>& b = r->blocks[gi];
        // from the back, as the reference pops them (src/core/paging/paged_kv_cache.h:196-208): the page
        // nearest to the kept prefix is the next to be handed out
        for (long long i = (long long)b.size() - 1; i >= keep; --i)
            if (b[i] >= 0) { const int rc = free_pages_of(c->groups[gi], &b[i], 1); if (rc) return rc; }
        if ((long long)b.size() > keep) b.resize(keep);
        if (r->first_live[gi] > keep) r->first_live[gi] = (int)keep;
    }
    r->length = new_length;
    return BWH_OK;
}

// The request ends: its pages and its slot are given back.  Returns the slot.
BWH_EXPORT int bwh_free_request(void* cache, int h) {
    Cache* c = (Cache*)cache;
    Request* r = get(c, h);
    if (!r) return BWH_BAD_ARG;
    for (size_t gi = 0; gi < c->groups.size(); ++gi)
        for (int& p : r->blocks[gi])
            if (p >= 0) { const int rc = free_pages_of(c->groups[gi], &p, 1); if (rc) return rc; p = -1; }
    const int slot = r->slot;
    if (c->slot_free[slot]) return BWH_FREED_TWICE;
    c->slot_free[slot] = 1; c->free_slots.push_back(slot);
    r->live = false; r->blocks.clear(); r->first_live.clear();
    c->free_handles.push_back(h);
    return slot;
}

BWH_EXPORT int bwh_num_blocks(void* cache, int h, int group) {
    Cache* c = (Cache*)cache;
    Request* r = get(c, h);
    if (!r || group < 0 || group >= (int)c->groups.size()) return BWH_BAD_ARG;
    return (int)r->blocks[group].size();
}

// Copies the block table of (request, group) into out[0..cap); returns its length.
BWH_EXPORT int bwh_blocks(void* cache, int h, int group, int* out, int cap) {
    Cache* c = (Cache*)cache;
    Request* r = get(c, h);
    if (!r || group < 0 || group >= (int)c->groups.size()) return BWH_BAD_ARG;
    const std::vector<int>& b = r->blocks[group];
    if ((int)b.size() > cap) return BWH_TOO_SMALL;
    if (!b.empty()) std::memcpy(out, b.data(), b.size() * sizeof(int));
    return (int)b.size();
}

// No page lost, none held twice, no held page on a free list, every slot accounted for.
BWH_EXPORT int bwh_check(void* cache) {
    Cache* c = (Cache*)cache;
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        Group& g = c->groups[gi];
        std::vector<uint8_t> held(g.num_pages, 0);
        long long n_held = 0;
        for (const Request& r : c->requests) {
            if (!r.live) continue;
            for (int p : r.blocks[gi]) {
                if (p < 0) continue;
                if (p >= g.num_pages) return BWH_BAD_ARG;
                if (held[p]) return BWH_PAGE_HELD_TWICE;
                if (g.is_free[p]) return BWH_HELD_PAGE_FREE;
                held[p] = 1; ++n_held;
            }
        }
        if (n_held + (long long)g.free.size() != g.num_pages) return BWH_PAGE_LOST;
    }
    int live = 0;
    for (const Request& r : c->requests) live += r.live ? 1 : 0;
    if (live + (int)c->free_slots.size() != c->max_requests) return BWH_PAGE_LOST;
    return BWH_OK;
}

// One step: R entries; handles[i] < 0 asks for a new request (its handle is written back).  Checks
// the token ids (0 <= id < vocab) and the wanted places, then reserves the pages for ALL tokens of
// the step in every group, or changes nothing and returns BWH_OUT_OF_PAGES / BWH_NO_SLOT.  Then the
// requests grow and the step is written into out[0..cap) in this order, all int32:
//   token ids [T], positions [T], request of token [T], cu_q [R + 1], q_start [R], kv_len [R],
//   slot [R], logit rows [n_want], and per group a block table [R, width_g] padded with -1,
// width_g = max(min_blocks, 1, longest table of the step).  meta: T, n_want, total words,
// n_new, then width per group.  new_slots[0..n_new): the slots of the new requests (their state
// must be zeroed by the caller).  Returns the number of words written, or an error.
BWH_EXPORT long long bwh_pack_step(void* cache, int R, int* handles, const int* n_tok, const int* tokens,
                                   const int* n_want, const int* want, int vocab, int min_blocks,
                                   long long max_tokens, int* out, long long cap, long long* meta, int* new_slots) {
    Cache* c = (Cache*)cache;
    const int G = (int)c->groups.size();
    if (R <= 0) return BWH_BAD_ARG;
    long long T = 0, W = 0;
    int n_new = 0;
    if (c->mark.size() < c->requests.size()) c->mark.resize(c->requests.size(), 0);
    int rc = BWH_OK;
    for (int i = 0; i < R && rc == BWH_OK; ++i) {
        if (n_tok[i] <= 0 || n_want[i] < 0) { rc = BWH_BAD_ARG; break; }
        for (int t = 0; t < n_tok[i]; ++t) if (tokens[T + t] < 0 || tokens[T + t] >= vocab) rc = BWH_BAD_TOKEN;
        for (int w = 0; w < n_want[i]; ++w) if (want[W + w] < 0 || want[W + w] >= n_tok[i]) rc = BWH_BAD_WANT;
        if (handles[i] < 0) ++n_new;
        else if (!get(c, handles[i])) rc = BWH_BAD_ARG;
        else if (c->mark[handles[i]]) rc = BWH_TWICE;
        else c->mark[handles[i]] = 1;
        T += n_tok[i]; W += n_want[i];
    }
    for (int i = 0; i < R; ++i) if (handles[i] >= 0 && handles[i] < (int)c->mark.size()) c->mark[handles[i]] = 0;
    if (rc != BWH_OK) return rc;
    if (T > max_tokens) return BWH_TOO_MANY_TOKENS;
    if (n_new > (int)c->free_slots.size()) return BWH_NO_SLOT;
    // pages for the whole step, all or nothing
    for (int g = 0; g < G; ++g) {
        long long need = 0;
        for (int i = 0; i < R; ++i) {
            if (handles[i] < 0) need += ceil_div(n_tok[i], c->page_size);
            else need += pages_short(c, c->requests[handles[i]], g, c->requests[handles[i]].length + n_tok[i]);
        }
        if (need > (long long)c->groups[g].free.size()) return BWH_OUT_OF_PAGES;
    }
    // sizes, before anything changes
    std::vector<long long> width(G, 0);
    for (int g = 0; g < G; ++g) {
        long long w = min_blocks > 1 ? min_blocks : 1;
        for (int i = 0; i < R; ++i) {
            const long long len = (handles[i] < 0 ? 0 : c->requests[handles[i]].length) + n_tok[i];
            const long long blocks = ceil_div(len, c->page_size);
            if (blocks > w) w = blocks;
        }
        width[g] = w;
    }
    long long total = 3 * T + (R + 1) + 3LL * R + W;
    for (int g = 0; g < G; ++g) total += (long long)R * width[g];
    if (total > cap) return BWH_TOO_SMALL;

    int k_new = 0;
    for (int i = 0; i < R; ++i)
        if (handles[i] < 0) { handles[i] = add_request(c); new_slots[k_new++] = c->requests[handles[i]].slot; }
    int* tok = out; int* pos = tok + T; int* req = pos + T; int* cu = req + T; int* qs = cu + R + 1;
    int* kv = qs + R; int* sl = kv + R; int* lr = sl + R; int* bt = lr + W;
    long long t0 = 0, w0 = 0;
    cu[0] = 0;
    for (int i = 0; i < R; ++i) {
        Request& r = c->requests[handles[i]];
        const long long q_start = r.length;
        grow(c, r, n_tok[i]);
        for (int t = 0; t < n_tok[i]; ++t) {
            tok[t0 + t] = tokens[t0 + t];
            pos[t0 + t] = (int)(q_start + t);
            req[t0 + t] = i;
        }
        for (int w = 0; w < n_want[i]; ++w) lr[w0 + w] = (int)(t0 + want[w0 + w]);
        t0 += n_tok[i]; w0 += n_want[i];
        cu[i + 1] = (int)t0; qs[i] = (int)q_start; kv[i] = (int)r.length; sl[i] = r.slot;
    }
    for (int g = 0; g < G; ++g) {
        for (int i = 0; i < R; ++i) {
            const std::vector<int>& b = c->requests[handles[i]].blocks[g];
            int* row = bt + (long long)i * width[g];
            const long long n = (long long)b.size();
            if (n) std::memcpy(row, b.data(), n * sizeof(int));
            for (long long k = n; k < width[g]; ++k) row[k] = -1;
        }
        bt += (long long)R * width[g];
    }
    meta[0] = T; meta[1] = W; meta[2] = total; meta[3] = n_new;
    for (int g = 0; g < G; ++g) meta[4 + g] = width[g];
    return total;
}

// release_passed for every request of a step (after it ran); returns the pages freed.
BWH_EXPORT int bwh_release_passed_many(void* cache, int R, const int* handles) {
    int freed = 0;
    for (int i = 0; i < R; ++i) {
        const int n = bwh_release_passed(cache, handles[i]);
        if (n < 0) return n;
        freed += n;
    }
    return freed;
}
