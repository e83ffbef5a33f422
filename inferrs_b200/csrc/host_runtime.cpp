// Host side of the cache in native code: page pools, block tables, state slots, and the description of a
// replayed decode step.  No CUDA here; the Python package drives it through the C interface at the end
// (inferrs_b200/cache/manager.py is its front, and says what each call means).
//
// The reference keeps the same book in Rust: a pool of fixed-size blocks with a FIFO free list
// (inferrs-models/src/kv_cache.rs:80-139), a table per request (:154-222), release at the request's end
// (inferrs/src/engine.rs:746-748).  Here there is one pool and one table per *group* of caches with the same
// needs; a group with a window gives pages back as soon as every later query's window has passed them.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

constexpr int RELEASED = -1;

// return codes of the C interface
constexpr int OK = 0;
constexpr int ERR_UNKNOWN_REQUEST = -1;
constexpr int ERR_ALREADY_LIVE = -2;
constexpr int ERR_NO_SLOT = -3;
constexpr int ERR_OUT_OF_PAGES = -4;
constexpr int ERR_BAD_COUNT = -5;
constexpr int ERR_BEYOND_RESERVED = -6;
constexpr int ERR_DOUBLE_FREE = -7;
constexpr int ERR_ARGUMENT = -8;
constexpr int ERR_TOKEN = -9;
constexpr int ERR_POSITIONS = -10;
constexpr int ERR_TABLE_WIDTH = -11;

struct Pool {
    int n_pages = 0;
    std::deque<int> free_list;   // taken from the front, given back to the back
    std::vector<char> held;

    explicit Pool(int n) : n_pages(n), held(n, 0) {
        for (int i = 0; i < n; ++i) free_list.push_back(i);
    }
    int n_free() const { return (int)free_list.size(); }
    int take() {
        const int id = free_list.front();
        free_list.pop_front();
        held[id] = 1;
        return id;
    }
    bool give_back(int id) {
        if (id < 0 || id >= n_pages || !held[id]) return false;
        held[id] = 0;
        free_list.push_back(id);
        return true;
    }
};

struct Request {
    int slot = 0;
    int n_tokens = 0;     // tokens whose keys and values are in the cache
    int n_reserved = 0;   // tokens that pages have been taken for
    std::vector<std::vector<int>> tables;   // per group: page number -> page id or RELEASED
};

struct Cache {
    int page_size = 0, max_requests = 0;
    std::vector<int> windows;   // per group, -1: all keys stay visible
    std::vector<Pool> pools;
    std::deque<int> free_slots;
    std::unordered_map<int64_t, Request> requests;

    int pages_for(int n_tokens) const { return (n_tokens + page_size - 1) / page_size; }

    // the request gets a state slot (returned, >= 0) and empty block tables
    int admit(int64_t rid) {
        if (requests.count(rid)) return ERR_ALREADY_LIVE;
        if (free_slots.empty()) return ERR_NO_SLOT;
        Request r;
        r.slot = free_slots.front();
        free_slots.pop_front();
        r.tables.resize(pools.size());
        const int slot = r.slot;
        requests.emplace(rid, std::move(r));
        return slot;
    }

    // Free[g] pages of every group are still unspoken for; request i would take the pages for n_new[i] more
    // tokens.  Subtracts what each one needs from free_pages[] as long as it fits and stops at the first that
    // does not; returns how many fitted.  Nothing is taken from the pools.
    int fit_in_order(int n, const int64_t* rids, const int* n_new, int* free_pages) {
        std::vector<int> need(pools.size());
        for (int i = 0; i < n; ++i) {
            Request* r = get(rids[i]);
            if (r == nullptr) return ERR_UNKNOWN_REQUEST;
            pages_needed(*r, n_new[i], need.data());
            for (size_t g = 0; g < pools.size(); ++g)
                if (need[g] > free_pages[g]) return i;
            for (size_t g = 0; g < pools.size(); ++g) free_pages[g] -= need[g];
        }
        return n;
    }

    Request* get(int64_t rid) {
        auto it = requests.find(rid);
        return it == requests.end() ? nullptr : &it->second;
    }

    // pages that each group has to take so that n_new more tokens of the request fit
    void pages_needed(const Request& r, int n_new, int* out) const {
        const int total = pages_for(r.n_tokens + n_new);
        for (size_t g = 0; g < pools.size(); ++g) {
            const int have = (int)r.tables[g].size();
            out[g] = total > have ? total - have : 0;
        }
    }

    int can_reserve(int n, const int64_t* rids, const int* n_new) {
        std::vector<int> need(pools.size(), 0), one(pools.size());
        for (int i = 0; i < n; ++i) {
            Request* r = get(rids[i]);
            if (r == nullptr) return ERR_UNKNOWN_REQUEST;
            pages_needed(*r, n_new[i], one.data());
            for (size_t g = 0; g < pools.size(); ++g) need[g] += one[g];
        }
        for (size_t g = 0; g < pools.size(); ++g)
            if (need[g] > pools[g].n_free()) return 0;
        return 1;
    }

    int reserve(int n, const int64_t* rids, const int* n_new) {
        for (int i = 0; i < n; ++i)
            if (n_new[i] <= 0) return ERR_BAD_COUNT;
        const int can = can_reserve(n, rids, n_new);
        if (can < 0) return can;
        if (can == 0) return ERR_OUT_OF_PAGES;
        std::vector<int> one(pools.size());
        for (int i = 0; i < n; ++i) {
            Request* r = get(rids[i]);
            pages_needed(*r, n_new[i], one.data());
            for (size_t g = 0; g < pools.size(); ++g)
                for (int k = 0; k < one[g]; ++k) r->tables[g].push_back(pools[g].take());
            r->n_reserved = r->n_tokens + n_new[i];
        }
        return OK;
    }

    int commit(int64_t rid, int n_new) {
        Request* r = get(rid);
        if (r == nullptr) return ERR_UNKNOWN_REQUEST;
        if (r->n_tokens + n_new > r->n_reserved) return ERR_BEYOND_RESERVED;
        r->n_tokens += n_new;
        for (size_t g = 0; g < pools.size(); ++g) {
            if (windows[g] < 0) continue;
            // the next query stands at position >= n_tokens and sees keys >= n_tokens - window + 1
            const int first_needed = r->n_tokens - windows[g] + 1;
            if (first_needed <= 0) continue;
            int dead = first_needed / page_size;   // pages 0..dead-1 hold only keys before first_needed
            if (dead > (int)r->tables[g].size()) dead = (int)r->tables[g].size();
            for (int i = 0; i < dead; ++i) {
                int& p = r->tables[g][i];
                if (p != RELEASED) {
                    if (!pools[g].give_back(p)) return ERR_DOUBLE_FREE;
                    p = RELEASED;
                }
            }
        }
        return OK;
    }

    int release(int64_t rid) {
        auto it = requests.find(rid);
        if (it == requests.end()) return ERR_UNKNOWN_REQUEST;
        Request& r = it->second;
        for (size_t g = 0; g < pools.size(); ++g)
            for (int p : r.tables[g])
                if (p != RELEASED && !pools[g].give_back(p)) return ERR_DOUBLE_FREE;
        free_slots.push_back(r.slot);
        requests.erase(it);
        return OK;
    }

    // No page lost, none held by two requests, free list and tables disjoint; the same for the slots.
    int check(std::string& msg) const {
        for (size_t g = 0; g < pools.size(); ++g) {
            const Pool& pool = pools[g];
            std::vector<int64_t> owner(pool.n_pages, INT64_MIN);
            int n_seen = 0;
            for (const auto& kv : requests) {
                for (int p : kv.second.tables[g]) {
                    if (p == RELEASED) continue;
                    if (p < 0 || p >= pool.n_pages) { msg = "a block table holds a page id outside its pool"; return 1; }
                    if (owner[p] != INT64_MIN) { msg = "a page is held by two requests"; return 1; }
                    if (!pool.held[p]) { msg = "a page of a request is marked free"; return 1; }
                    owner[p] = kv.first;
                    ++n_seen;
                }
            }
            std::vector<char> in_free(pool.n_pages, 0);
            for (int p : pool.free_list) {
                if (in_free[p]) { msg = "a page is twice in the free list"; return 1; }
                in_free[p] = 1;
                if (owner[p] != INT64_MIN) { msg = "a held page is in the free list"; return 1; }
            }
            if ((int)pool.free_list.size() + n_seen != pool.n_pages) { msg = "pages are lost"; return 1; }
        }
        std::vector<char> slot_used(max_requests, 0);
        size_t n = 0;
        for (const auto& kv : requests) {
            const int s = kv.second.slot;
            if (s < 0 || s >= max_requests || slot_used[s]) { msg = "state slots are lost or held twice"; return 1; }
            slot_used[s] = 1;
            ++n;
        }
        for (int s : free_slots) {
            if (s < 0 || s >= max_requests || slot_used[s]) { msg = "state slots are lost or held twice"; return 1; }
            slot_used[s] = 1;
            ++n;
        }
        if ((int)n != max_requests) { msg = "state slots are lost or held twice"; return 1; }
        return 0;
    }
};

}  // namespace

#define IBH_EXPORT extern "C" __attribute__((visibility("default")))

// windows[g] < 0: group g keeps all keys.  Returns nullptr for sizes that make no sense.
IBH_EXPORT void* ibh_cache_new(int n_groups, const int* windows, const int* n_pages, int page_size, int max_requests) {
    if (n_groups <= 0 || page_size <= 0 || max_requests <= 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (n_pages[g] <= 0 || windows[g] == 0) return nullptr;
    Cache* c = new Cache();
    c->page_size = page_size;
    c->max_requests = max_requests;
    for (int g = 0; g < n_groups; ++g) {
        c->windows.push_back(windows[g] < 0 ? -1 : windows[g]);
        c->pools.emplace_back(n_pages[g]);
    }
    for (int s = 0; s < max_requests; ++s) c->free_slots.push_back(s);
    return c;
}

IBH_EXPORT void ibh_cache_delete(void* h) { delete static_cast<Cache*>(h); }

// The request gets a state slot (returned, >= 0) and empty block tables.
IBH_EXPORT int ibh_cache_admit(void* h, int64_t rid) { return static_cast<Cache*>(h)->admit(rid); }

IBH_EXPORT int ibh_cache_has(void* h, int64_t rid) { return static_cast<Cache*>(h)->requests.count(rid) ? 1 : 0; }
IBH_EXPORT int ibh_cache_n_live(void* h) { return (int)static_cast<Cache*>(h)->requests.size(); }
IBH_EXPORT int ibh_cache_n_free_slots(void* h) { return (int)static_cast<Cache*>(h)->free_slots.size(); }
IBH_EXPORT int ibh_cache_n_free_pages(void* h, int g) { return static_cast<Cache*>(h)->pools[g].n_free(); }

IBH_EXPORT int ibh_cache_slot(void* h, int64_t rid) {
    Request* r = static_cast<Cache*>(h)->get(rid);
    return r == nullptr ? ERR_UNKNOWN_REQUEST : r->slot;
}

IBH_EXPORT int ibh_cache_n_tokens(void* h, int64_t rid) {
    Request* r = static_cast<Cache*>(h)->get(rid);
    return r == nullptr ? ERR_UNKNOWN_REQUEST : r->n_tokens;
}

// Copies the request's block table of group g to out (at most cap entries); returns its length.
IBH_EXPORT int ibh_cache_block_table(void* h, int64_t rid, int g, int* out, int cap) {
    Cache* c = static_cast<Cache*>(h);
    Request* r = c->get(rid);
    if (r == nullptr) return ERR_UNKNOWN_REQUEST;
    if (g < 0 || g >= (int)c->pools.size()) return ERR_ARGUMENT;
    const std::vector<int>& t = r->tables[g];
    const int n = (int)t.size() < cap ? (int)t.size() : cap;
    if (n > 0) std::memcpy(out, t.data(), (size_t)n * sizeof(int));
    return (int)t.size();
}

IBH_EXPORT int ibh_cache_pages_needed(void* h, int64_t rid, int n_new, int* out) {
    Cache* c = static_cast<Cache*>(h);
    Request* r = c->get(rid);
    if (r == nullptr) return ERR_UNKNOWN_REQUEST;
    c->pages_needed(*r, n_new, out);
    return OK;
}

// 1 if the pages for n_new[i] more tokens of every request rids[i] are free, 0 if not.
IBH_EXPORT int ibh_cache_can_reserve(void* h, int n, const int64_t* rids, const int* n_new) {
    return static_cast<Cache*>(h)->can_reserve(n, rids, n_new);
}

// Takes those pages, or changes nothing and says why.
IBH_EXPORT int ibh_cache_reserve(void* h, int n, const int64_t* rids, const int* n_new) {
    return static_cast<Cache*>(h)->reserve(n, rids, n_new);
}

IBH_EXPORT int ibh_cache_commit(void* h, int64_t rid, int n_new) { return static_cast<Cache*>(h)->commit(rid, n_new); }
IBH_EXPORT int ibh_cache_release(void* h, int64_t rid) { return static_cast<Cache*>(h)->release(rid); }

IBH_EXPORT int ibh_cache_check(void* h, char* msg, int cap) {
    std::string m;
    const int bad = static_cast<Cache*>(h)->check(m);
    if (bad && cap > 0) std::snprintf(msg, (size_t)cap, "%s", m.c_str());
    return bad;
}

// The description of a step in which each of the n requests brings one token, padded to `bucket` requests, in
// the layout that the captured graphs read (every part starts on a multiple of four numbers):
//   token ids [bucket] | positions [bucket] | request of each row [bucket] | first row of each request [bucket + 1]
//   | keys each request sees [bucket] | state slots [bucket] | rows whose logits are made [bucket]
//   | per group: block tables [bucket, fixed_pages[g]]
// A request that only fills the batch has token 0 at position 0, one key, no pages (-1 everywhere) and state slot
// max_requests, which no request ever gets (the state tensors have that one slot more).
// The pages for the step's tokens are reserved already.  Returns the count of numbers written, or an error with
// the index of the offending entry in *bad.
IBH_EXPORT int ibh_describe_decode(void* h, int n, const int64_t* rids, const int* tokens, int bucket,
                                   const int* fixed_pages, int vocab_size, int max_positions, int* out, int cap,
                                   int* bad) {
    Cache* c = static_cast<Cache*>(h);
    if (n <= 0 || n > bucket || out == nullptr) return ERR_ARGUMENT;
    const int n_groups = (int)c->pools.size();
    auto round4 = [](int v) { return (v + 3) / 4 * 4; };
    int off[8];
    off[0] = 0;
    off[1] = off[0] + round4(bucket);
    off[2] = off[1] + round4(bucket);
    off[3] = off[2] + round4(bucket);
    off[4] = off[3] + round4(bucket + 1);
    off[5] = off[4] + round4(bucket);
    off[6] = off[5] + round4(bucket);
    off[7] = off[6] + round4(bucket);
    int total = off[7];
    for (int g = 0; g < n_groups; ++g) total += round4(bucket * fixed_pages[g]);
    if (total > cap) return ERR_ARGUMENT;
    std::memset(out, 0, (size_t)total * sizeof(int));
    for (int i = 0; i < bucket; ++i) {
        out[off[2] + i] = i;
        out[off[3] + i] = i;
        out[off[4] + i] = 1;
        out[off[5] + i] = c->max_requests;   // a request that only fills the batch: the slot that no request ever gets
        out[off[6] + i] = i;
    }
    out[off[3] + bucket] = bucket;
    int at = off[7];
    std::vector<int> table_at(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        table_at[g] = at;
        const int count = bucket * fixed_pages[g];
        for (int k = 0; k < count; ++k) out[at + k] = RELEASED;
        at += round4(count);
    }
    for (int i = 0; i < n; ++i) {
        if (bad != nullptr) *bad = i;
        Request* r = c->get(rids[i]);
        if (r == nullptr) return ERR_UNKNOWN_REQUEST;
        if (tokens[i] < 0 || tokens[i] >= vocab_size) return ERR_TOKEN;
        if (r->n_tokens + 1 > max_positions) return ERR_POSITIONS;
        out[off[0] + i] = tokens[i];
        out[off[1] + i] = r->n_tokens;
        out[off[4] + i] = r->n_tokens + 1;
        out[off[5] + i] = r->slot;
        for (int g = 0; g < n_groups; ++g) {
            const std::vector<int>& t = r->tables[g];
            if ((int)t.size() > fixed_pages[g]) return ERR_TABLE_WIDTH;
            if (!t.empty()) std::memcpy(out + table_at[g] + (size_t)i * fixed_pages[g], t.data(), t.size() * sizeof(int));
        }
    }
    return total;
}

// The description of a step of any portions, padded to a fixed shape (the layout that the captured graphs of
// such steps read; every part starts on a multiple of four numbers):
//   token ids [pad_rows] | positions [pad_rows] | request of each row [pad_rows] | first row of each request
//   [pad_requests + 1] | keys each request sees [pad_requests] | state slots [pad_requests] | rows whose logits
//   are made [pad_wanted] | per group: block tables [pad_requests, fixed_pages[g]] | per tile size: request and
//   first row of every attention tile [pad_rows / size + pad_requests each] | rows and requests of the requests
//   that bring a single token [pad_requests each]
// Request i brings n_tok[i] tokens (concatenated in `tokens`) and wants the logits at n_want[i] of its places
// (concatenated in `wants`).  The rows that fill the step up belong to one more request without pages, at position
// 0; the requests after it are empty.  -1 marks table entries, tiles and single-token places that are not there.
// A tile size with tile_portions[k] != 0 leaves the single-token requests out.  A tile list has room for
// pad_rows / tile_tokens[k] + tile_pad tiles (tile_pad: the most requests that may bring tiles); the tiles stand at its
// end, the one that sees the fewest keys first (the attention kernels start at the end: the longest tile first, the
// places without a tile last).  The pages for the step's tokens are reserved already.  Returns the count of numbers
// written, or an error with the offending entry in *bad.
IBH_EXPORT int ibh_describe_step(void* h, int n, const int64_t* rids, const int* n_tok, const int* tokens,
                                 const int* n_want, const int* wants, int pad_rows, int pad_requests, int pad_wanted,
                                 const int* fixed_pages, int n_tile_sizes, const int* tile_tokens,
                                 const int* tile_portions, int tile_pad, int vocab_size, int max_positions, int* out,
                                 int cap, int* bad) {
    Cache* c = static_cast<Cache*>(h);
    if (n <= 0 || n + 1 > pad_requests || out == nullptr || pad_rows <= 0 || pad_wanted < 0 || tile_pad < 0)
        return ERR_ARGUMENT;
    const int n_groups = (int)c->pools.size();
    auto round4 = [](int v) { return (v + 3) / 4 * 4; };
    int total_rows = 0, total_want = 0;
    for (int i = 0; i < n; ++i) {
        if (n_tok[i] <= 0 || n_want[i] < 0) { if (bad) *bad = i; return ERR_BAD_COUNT; }
        total_rows += n_tok[i];
        total_want += n_want[i];
    }
    if (total_rows > pad_rows || total_want > pad_wanted) return ERR_ARGUMENT;
    // where the parts start
    std::vector<int> off;
    int at = 0;
    auto part = [&](int count) { off.push_back(at); at += round4(count); };
    part(pad_rows); part(pad_rows); part(pad_rows); part(pad_requests + 1); part(pad_requests); part(pad_requests);
    part(pad_wanted);
    for (int g = 0; g < n_groups; ++g) part(pad_requests * fixed_pages[g]);
    std::vector<int> t_max(n_tile_sizes);
    for (int k = 0; k < n_tile_sizes; ++k) {
        if (tile_tokens[k] <= 0) return ERR_ARGUMENT;
        t_max[k] = pad_rows / tile_tokens[k] + tile_pad;
        part(t_max[k]);
        part(t_max[k]);
    }
    part(pad_requests);
    part(pad_requests);
    if (at > cap) return ERR_ARGUMENT;
    std::memset(out, 0, (size_t)at * sizeof(int));
    int* ids = out + off[0];
    int* pos = out + off[1];
    int* row_req = out + off[2];
    int* q_start = out + off[3];
    int* kv_len = out + off[4];
    int* slots = out + off[5];
    int* logit_rows = out + off[6];
    for (int g = 0; g < n_groups; ++g) {
        int* t = out + off[7 + g];
        for (int k = 0; k < pad_requests * fixed_pages[g]; ++k) t[k] = RELEASED;
    }
    const int tiles_at = 7 + n_groups;
    for (int k = 0; k < n_tile_sizes; ++k)
        for (int j = 0; j < t_max[k]; ++j) out[off[tiles_at + 2 * k] + j] = -1;
    int* single_rows = out + off[tiles_at + 2 * n_tile_sizes];
    int* single_reqs = out + off[tiles_at + 2 * n_tile_sizes + 1];
    for (int j = 0; j < pad_requests; ++j) single_rows[j] = single_reqs[j] = -1;
    for (int j = 0; j < pad_requests; ++j) slots[j] = c->max_requests;   // the slot that no request ever gets

    struct Tile { int last_pos, req, row0; };
    std::vector<std::vector<Tile>> tiles(n_tile_sizes);
    int row = 0, tok_at = 0, want_at = 0, n_logit = 0, n_single = 0;
    for (int i = 0; i < n; ++i) {
        if (bad != nullptr) *bad = i;
        Request* r = c->get(rids[i]);
        if (r == nullptr) return ERR_UNKNOWN_REQUEST;
        const int t = n_tok[i];
        if (r->n_tokens + t > max_positions) return ERR_POSITIONS;
        q_start[i] = row;
        kv_len[i] = r->n_tokens + t;
        slots[i] = r->slot;
        for (int j = 0; j < t; ++j) {
            const int id = tokens[tok_at + j];
            if (id < 0 || id >= vocab_size) return ERR_TOKEN;
            ids[row + j] = id;
            pos[row + j] = r->n_tokens + j;
            row_req[row + j] = i;
        }
        for (int j = 0; j < n_want[i]; ++j) {
            const int w = wants[want_at + j];
            if (w < 0 || w >= t) return ERR_BAD_COUNT;
            logit_rows[n_logit++] = row + w;
        }
        for (int g = 0; g < n_groups; ++g) {
            const std::vector<int>& table = r->tables[g];
            if ((int)table.size() > fixed_pages[g]) return ERR_TABLE_WIDTH;
            if (!table.empty())
                std::memcpy(out + off[7 + g] + (size_t)i * fixed_pages[g], table.data(), table.size() * sizeof(int));
        }
        for (int k = 0; k < n_tile_sizes; ++k) {
            if (tile_portions[k] && t == 1) continue;
            for (int s0 = 0; s0 < t; s0 += tile_tokens[k]) {
                const int s1 = s0 + tile_tokens[k] < t ? s0 + tile_tokens[k] : t;
                tiles[k].push_back({r->n_tokens + s1 - 1, i, row + s0});
            }
            if ((int)tiles[k].size() > t_max[k]) return ERR_ARGUMENT;   // more requests bring tiles than tile_pad allows
        }
        if (t == 1) {
            single_rows[n_single] = row;
            single_reqs[n_single] = i;
            ++n_single;
        }
        row += t;
        tok_at += t;
        want_at += n_want[i];
    }
    for (int k = 0; k < n_tile_sizes; ++k) {
        std::stable_sort(tiles[k].begin(), tiles[k].end(), [](const Tile& a, const Tile& b) { return a.last_pos < b.last_pos; });
        const int first = t_max[k] - (int)tiles[k].size();
        for (size_t j = 0; j < tiles[k].size(); ++j) {
            out[off[tiles_at + 2 * k] + first + (int)j] = tiles[k][j].req;
            out[off[tiles_at + 2 * k + 1] + first + (int)j] = tiles[k][j].row0;
        }
    }
    // the request that takes the rows that fill the step up, then the empty ones
    const int extra = pad_rows - row;
    for (int j = 0; j < extra; ++j) row_req[row + j] = n;
    for (int i = n; i < pad_requests; ++i) {
        const int k = i == n ? extra : 0;
        q_start[i] = i == n ? row : pad_rows;
        kv_len[i] = k > 1 ? k : 1;
    }
    q_start[pad_requests] = pad_rows;
    return at;
}

// For a scheduler that walks its requests in order: free[g] pages of every group are still unspoken for; request
// i would take the pages for n_new[i] more tokens.  Goes through the requests in the order given, subtracts what
// each one needs from free[] as long as it fits, and stops at the first that does not.  Returns how many fitted
// (n if all did); free[] then holds what is left after those.  Nothing is taken from the pools.
IBH_EXPORT int ibh_cache_fit_in_order(void* h, int n, const int64_t* rids, const int* n_new, int* free_pages) {
    return static_cast<Cache*>(h)->fit_in_order(n, rids, n_new, free_pages);
}

// ---------------------------------------------------------------------------------------------------------
// The scheduler's decisions in native code: which requests run in the next step and with how many tokens.
//
// The reference's loop admits requests while fewer than max_batch_size are active, runs one forward pass per
// sequence per turn, never cuts a prompt and fails a request when blocks run out
// (inferrs/src/engine.rs:1380-1912, :2093-2095).  Here every step is one batch under a token budget: decoded
// tokens first, then portions of running prompts, then admissions, first come first served; when pages run
// out the youngest running request is preempted and recomputed later.  The scheduler knows requests by number
// and by their counts only; token ids, sampling options and results stay with the Python front
// (inferrs_b200/engine/scheduler.py), which says what each call means.
// ---------------------------------------------------------------------------------------------------------
namespace {

constexpr int ERR_EMPTY_PROMPT = -20;
constexpr int ERR_PROMPT_TOO_LONG = -21;
constexpr int ERR_NEVER_FITS = -22;
constexpr int ERR_IN_FLIGHT = -23;
constexpr int ERR_CAPACITY = -24;
constexpr int ERR_NOT_RUNNING = -25;

enum { WAITING = 0, RUNNING = 1, FINISHED = 2 };
enum { REASON_NONE = 0, REASON_STOP = 1, REASON_LENGTH = 2 };

struct SchedRequest {
    int n_prompt = 0, n_output = 0;
    int n_computed = 0;    // tokens that launched steps have run
    int n_in_flight = 0;   // tokens that launched steps have sampled and nobody has delivered yet
    int max_tokens = 0, ignore_eos = 0;
    std::vector<int> stop_ids;
    long order = 0;        // arrival number: smaller is older
    int n_preempted = 0;
    int state = WAITING;
    int n_pending() const { return n_prompt + n_output + n_in_flight - n_computed; }
};

struct Scheduler {
    Cache* cache = nullptr;
    int max_batch = 0, budget = 0, chunk = 0, max_positions = 0;
    std::vector<int> eos;
    std::unordered_map<int64_t, SchedRequest> requests;
    std::deque<int64_t> waiting;
    std::vector<int64_t> running;   // in the order of their admission
    long arrivals = 0;
    int n_preemptions = 0;

    SchedRequest* get(int64_t rid) {
        auto it = requests.find(rid);
        return it == requests.end() ? nullptr : &it->second;
    }

    void drop_running(int64_t rid) {
        for (size_t i = 0; i < running.size(); ++i)
            if (running[i] == rid) {
                running.erase(running.begin() + i);
                return;
            }
    }

    int add(int64_t rid, int n_prompt, int max_tokens, int ignore_eos, const int* stop, int n_stop) {
        if (requests.count(rid)) return ERR_ALREADY_LIVE;
        if (n_prompt <= 0) return ERR_EMPTY_PROMPT;
        if (n_prompt >= max_positions) return ERR_PROMPT_TOO_LONG;
        const int pages = cache->pages_for(n_prompt + 1);
        for (const Pool& pool : cache->pools)
            if (pages > pool.n_pages) return ERR_NEVER_FITS;
        SchedRequest r;
        r.n_prompt = n_prompt;
        r.max_tokens = max_tokens;
        r.ignore_eos = ignore_eos;
        r.stop_ids.assign(stop, stop + n_stop);
        r.order = arrivals++;
        requests.emplace(rid, std::move(r));
        waiting.push_back(rid);
        return OK;
    }

    // 1: it was running (pages and slot are free again), 2: it was waiting, 0: unknown or over already
    int abort(int64_t rid) {
        SchedRequest* r = get(rid);
        if (r == nullptr) return 0;
        int was = 0;
        if (r->state == RUNNING) {
            drop_running(rid);
            cache->release(rid);
            was = 1;
        } else if (r->state == WAITING) {
            for (size_t i = 0; i < waiting.size(); ++i)
                if (waiting[i] == rid) {
                    waiting.erase(waiting.begin() + i);
                    break;
                }
            was = 2;
        }
        requests.erase(rid);
        return was;
    }

    // The youngest running request other than `keep` gives its pages and slot back and returns to the head of
    // the waiting queue; everything it has (prompt and generated tokens) is run again later.
    bool preempt_youngest(int64_t keep, std::vector<int64_t>& preempted) {
        int64_t victim = -1;
        long youngest = -1;
        for (int64_t rid : running) {
            if (rid == keep) continue;
            const SchedRequest& r = requests[rid];
            if (r.order > youngest) {
                youngest = r.order;
                victim = rid;
            }
        }
        if (victim < 0) return false;
        drop_running(victim);
        cache->release(victim);
        SchedRequest& v = requests[victim];
        v.n_computed = 0;
        v.n_preempted += 1;
        v.state = WAITING;
        n_preemptions += 1;
        waiting.push_front(victim);
        preempted.push_back(victim);
        return true;
    }

    struct Entry {
        int64_t rid;
        int start, n, samples;
    };

    // 0: planned; 1: not planned, because it would take a running request's pages or end one and may_preempt is 0
    // (nothing has changed then); < 0: an error.
    int plan(int may_preempt, std::vector<Entry>& out, std::vector<int64_t>& preempted, std::vector<int64_t>& ended,
             std::vector<int64_t>& admitted) {
        const int n_groups = (int)cache->pools.size();
        std::vector<int> free_pages(n_groups), need(n_groups);
        std::vector<int64_t> order;
        std::vector<int> counts;
        while (true) {
            int left = budget;
            for (int g = 0; g < n_groups; ++g) free_pages[g] = cache->pools[g].n_free();
            out.clear();
            // decoded tokens first, then portions of prompts, oldest first
            std::vector<int64_t> by_age(running);
            std::stable_sort(by_age.begin(), by_age.end(),
                             [&](int64_t a, int64_t b) { return requests[a].order < requests[b].order; });
            order.clear();
            for (int64_t rid : by_age)
                if (requests[rid].n_pending() == 1) order.push_back(rid);
            for (int64_t rid : by_age)
                if (requests[rid].n_pending() > 1) order.push_back(rid);
            counts.clear();
            for (int64_t rid : order) {
                if (left <= 0) break;
                int n = requests[rid].n_pending();
                if (n > left) n = left;
                if (n > chunk) n = chunk;
                counts.push_back(n);
                left -= n;
            }
            order.resize(counts.size());
            int fitted = 0;
            if (!order.empty()) {
                fitted = cache->fit_in_order((int)order.size(), order.data(), counts.data(), free_pages.data());
                if (fitted < 0) return fitted;
            }
            for (int i = 0; i < fitted; ++i) {
                const SchedRequest& r = requests[order[i]];
                out.push_back({order[i], r.n_computed, counts[i], counts[i] == r.n_pending() ? 1 : 0});
            }
            if (fitted < (int)order.size()) {
                const int64_t starved = order[fitted];
                if (!may_preempt) {
                    out.clear();
                    return 1;
                }
                for (int64_t rid : running)
                    if (requests[rid].n_in_flight) return ERR_IN_FLIGHT;
                if (preempt_youngest(starved, preempted)) continue;   // plan again with the pages that came back
                // the request is alone and still does not fit: it has outgrown the cache
                drop_running(starved);
                cache->release(starved);
                requests.erase(starved);
                ended.push_back(starved);
                continue;
            }
            // admission, first come first served
            while (!waiting.empty() && left > 0 && (int)running.size() < max_batch && !cache->free_slots.empty()) {
                const int64_t rid = waiting.front();
                SchedRequest& r = requests[rid];
                int n = r.n_pending();
                if (n > left) n = left;
                if (n > chunk) n = chunk;
                const int slot = cache->admit(rid);
                if (slot < 0) return slot;
                cache->pages_needed(*cache->get(rid), n, need.data());
                bool fits = true;
                for (int g = 0; g < n_groups; ++g) fits = fits && need[g] <= free_pages[g];
                if (!fits) {
                    cache->release(rid);
                    break;
                }
                for (int g = 0; g < n_groups; ++g) free_pages[g] -= need[g];
                waiting.pop_front();
                running.push_back(rid);
                r.state = RUNNING;
                admitted.push_back(rid);
                out.push_back({rid, r.n_computed, n, n == r.n_pending() ? 1 : 0});
                left -= n;
            }
            return 0;
        }
    }

    int advance(int n, const int64_t* rids, const int* n_tok, const int* samples) {
        for (int i = 0; i < n; ++i)
            if (get(rids[i]) == nullptr) return ERR_UNKNOWN_REQUEST;
        for (int i = 0; i < n; ++i) {
            SchedRequest& r = requests[rids[i]];
            r.n_computed += n_tok[i];
            if (samples[i]) r.n_in_flight += 1;
        }
        return OK;
    }

    int stop_reason(const SchedRequest& r, int token) const {
        if (!r.ignore_eos) {
            for (int t : eos)
                if (t == token) return REASON_STOP;
            for (int t : r.stop_ids)
                if (t == token) return REASON_STOP;
        }
        if (r.n_output >= r.max_tokens) return REASON_LENGTH;
        if (r.n_prompt + r.n_output >= max_positions) return REASON_LENGTH;
        return REASON_NONE;
    }

    // one sampled token per request named; reasons[i] says whether and why request i is over with it
    int deliver(int n, const int64_t* rids, const int* tokens, int* reasons) {
        for (int i = 0; i < n; ++i) {
            SchedRequest* r = get(rids[i]);
            if (r == nullptr) return ERR_UNKNOWN_REQUEST;
            if (r->state != RUNNING || r->n_in_flight <= 0) return ERR_NOT_RUNNING;
        }
        for (int i = 0; i < n; ++i) {
            SchedRequest& r = requests[rids[i]];
            r.n_in_flight -= 1;
            r.n_output += 1;
            reasons[i] = stop_reason(r, tokens[i]);
            if (reasons[i] != REASON_NONE) {
                drop_running(rids[i]);
                cache->release(rids[i]);
                requests.erase(rids[i]);
            }
        }
        return OK;
    }
};

}  // namespace

IBH_EXPORT void* ibh_sched_new(void* cache, int max_batch, int budget, int chunk, int max_positions, const int* eos,
                               int n_eos) {
    if (cache == nullptr || max_batch <= 0 || budget <= 0 || chunk <= 0 || n_eos < 0) return nullptr;
    Scheduler* s = new Scheduler();
    s->cache = static_cast<Cache*>(cache);
    s->max_batch = max_batch;
    s->budget = budget;
    s->chunk = chunk;
    s->max_positions = max_positions;
    s->eos.assign(eos, eos + n_eos);
    return s;
}

IBH_EXPORT void ibh_sched_delete(void* h) { delete static_cast<Scheduler*>(h); }

IBH_EXPORT int ibh_sched_add(void* h, int64_t rid, int n_prompt, int max_tokens, int ignore_eos, const int* stop,
                             int n_stop) {
    return static_cast<Scheduler*>(h)->add(rid, n_prompt, max_tokens, ignore_eos, stop, n_stop < 0 ? 0 : n_stop);
}

IBH_EXPORT int ibh_sched_abort(void* h, int64_t rid) { return static_cast<Scheduler*>(h)->abort(rid); }

// The next step.  entries[3 * i ..] = (start, tokens, samples) of request rids[i], for i < *n_entries; then the
// requests that were preempted, ended ("length": alone and still too large for the cache) and admitted while
// planning, each list in the order in which it happened.  cap bounds every list.  Returns 0, 1 (not planned:
// see Scheduler::plan) or an error.
IBH_EXPORT int ibh_sched_plan(void* h, int may_preempt, int cap, int64_t* rids, int* entries, int* n_entries,
                              int64_t* preempted, int* n_preempted, int64_t* ended, int* n_ended, int64_t* admitted,
                              int* n_admitted) {
    Scheduler* s = static_cast<Scheduler*>(h);
    std::vector<Scheduler::Entry> out;
    std::vector<int64_t> pre, end, adm;
    const int code = s->plan(may_preempt, out, pre, end, adm);
    *n_entries = *n_preempted = *n_ended = *n_admitted = 0;
    if (code != 0) return code;
    if ((int)out.size() > cap || (int)pre.size() > cap || (int)end.size() > cap || (int)adm.size() > cap) return ERR_CAPACITY;
    for (size_t i = 0; i < out.size(); ++i) {
        rids[i] = out[i].rid;
        entries[3 * i] = out[i].start;
        entries[3 * i + 1] = out[i].n;
        entries[3 * i + 2] = out[i].samples;
    }
    std::copy(pre.begin(), pre.end(), preempted);
    std::copy(end.begin(), end.end(), ended);
    std::copy(adm.begin(), adm.end(), admitted);
    *n_entries = (int)out.size();
    *n_preempted = (int)pre.size();
    *n_ended = (int)end.size();
    *n_admitted = (int)adm.size();
    return 0;
}

IBH_EXPORT int ibh_sched_advance(void* h, int n, const int64_t* rids, const int* n_tok, const int* samples) {
    return static_cast<Scheduler*>(h)->advance(n, rids, n_tok, samples);
}

IBH_EXPORT int ibh_sched_deliver(void* h, int n, const int64_t* rids, const int* tokens, int* reasons) {
    return static_cast<Scheduler*>(h)->deliver(n, rids, tokens, reasons);
}

// counts of one request: out = (n_prompt, n_output, n_computed, n_in_flight, n_preempted, state); -1 if unknown
IBH_EXPORT int ibh_sched_counts(void* h, int64_t rid, int* out) {
    SchedRequest* r = static_cast<Scheduler*>(h)->get(rid);
    if (r == nullptr) return ERR_UNKNOWN_REQUEST;
    out[0] = r->n_prompt; out[1] = r->n_output; out[2] = r->n_computed; out[3] = r->n_in_flight;
    out[4] = r->n_preempted; out[5] = r->state;
    return OK;
}

IBH_EXPORT int ibh_sched_n_waiting(void* h) { return (int)static_cast<Scheduler*>(h)->waiting.size(); }
IBH_EXPORT int ibh_sched_n_running(void* h) { return (int)static_cast<Scheduler*>(h)->running.size(); }
IBH_EXPORT int ibh_sched_n_preemptions(void* h) { return static_cast<Scheduler*>(h)->n_preemptions; }
