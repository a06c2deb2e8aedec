// Host-side core of the cache manager in C++: pools of pages, block tables per request and per
// group, window release, state slots, and the packing of a step's batch into one int32 buffer.
//
// The bookkeeping rules are those of cache/manager.py (which remains as the reference
// implementation and runs the same tests): a page id addresses the same page in every entry of its
// group; pages are taken when a step is about to write them, in every group or in none; they are
// given back when the request ends or when a group's window has passed them; the most recently
// freed unit is handed out first (the reference's allocator is a LIFO free list too,
// crates/core/src/scheduler/memory/allocator.rs:51-110); a unit freed twice is an error.
//
// C interface (ctypes): every function returns 0 or a negative VC_* code; nothing throws across
// the boundary.  Requests are named by 64-bit keys chosen by the caller.
#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <algorithm>
#include <vector>

namespace {

enum : int {
    VC_OK = 0,
    VC_NO_SPACE = -1,        // not enough free pages or slots; nothing was changed
    VC_UNKNOWN = -2,         // no such request / group
    VC_EXISTS = -3,          // the request already holds a cache
    VC_DOUBLE_FREE = -4,     // a unit was freed twice or never handed out
    VC_ARGUMENT = -5,
    VC_GONE = -6,            // a position lies in a page that was given back
    VC_TOO_LONG = -8,        // a request would grow beyond the caller's limit; nothing was changed
    VC_CORRUPT = -7          // the books do not balance (check)
};

struct Pool {
    std::vector<int> free_list;      // back() is handed out next
    std::vector<char> held;
    explicit Pool(int size = 0) : held(size, 0) {
        free_list.reserve(size);
        for (int i = size - 1; i >= 0; --i) free_list.push_back(i);   // 0 first
    }
    int size() const { return (int)held.size(); }
    int free_count() const { return (int)free_list.size(); }
    bool allocate(int n, std::vector<int>& out) {
        if (n < 0 || n > free_count()) return false;
        for (int i = 0; i < n; ++i) {
            const int u = free_list.back();
            free_list.pop_back();
            held[u] = 1;
            out.push_back(u);
        }
        return true;
    }
    int release(const int* units, int n) {
        for (int i = 0; i < n; ++i) {
            const int u = units[i];
            if (u < 0 || u >= size() || !held[u]) return VC_DOUBLE_FREE;
        }
        for (int i = 0; i < n; ++i) held[units[i]] = 0;
        for (int i = n - 1; i >= 0; --i) free_list.push_back(units[i]);     // first of the list comes out first
        return VC_OK;
    }
};

struct Request {
    int state_slot = -1;
    long long num_tokens = 0;
    std::vector<std::vector<int>> tables;     // per paged group; -1 = given back
};

struct Core {
    int page_size = 16;
    std::vector<Pool> pools;
    std::vector<int> windows;                 // per group, 0 = none
    Pool slots;
    std::unordered_map<long long, Request> requests;
    std::vector<int> fresh_slots;

    int pages_needed(const Request& r, long long count, int g) const {
        const long long want = (r.num_tokens + count + page_size - 1) / page_size;
        const long long have = (long long)r.tables[g].size();
        return want > have ? (int)(want - have) : 0;
    }
};

inline int align4(int n) { return (n + 3) & ~3; }

}  // namespace

extern "C" {

void* vc_create(int page_size, int num_groups, const int* pages_per_group, const int* windows, int max_requests) {
    if (page_size <= 0 || num_groups < 0 || max_requests < 0) return nullptr;
    Core* c = new Core();
    c->page_size = page_size;
    for (int g = 0; g < num_groups; ++g) {
        if (pages_per_group[g] < 0) { delete c; return nullptr; }
        c->pools.emplace_back(pages_per_group[g]);
        c->windows.push_back(windows ? windows[g] : 0);
    }
    c->slots = Pool(max_requests);
    return c;
}

void vc_destroy(void* h) { delete static_cast<Core*>(h); }

int vc_admit(void* h, long long key, int* state_slot) {
    Core* c = static_cast<Core*>(h);
    if (c->requests.count(key)) return VC_EXISTS;
    std::vector<int> got;
    if (!c->slots.allocate(1, got)) return VC_NO_SPACE;
    Request r;
    r.state_slot = got[0];
    r.tables.resize(c->pools.size());
    c->requests.emplace(key, std::move(r));
    c->fresh_slots.push_back(got[0]);
    if (state_slot) *state_slot = got[0];
    return VC_OK;
}

int vc_free(void* h, long long key) {
    Core* c = static_cast<Core*>(h);
    auto it = c->requests.find(key);
    if (it == c->requests.end()) return VC_UNKNOWN;
    Request& r = it->second;
    for (size_t g = 0; g < c->pools.size(); ++g) {
        std::vector<int> held;
        for (int p : r.tables[g]) if (p >= 0) held.push_back(p);
        const int rc = c->pools[g].release(held.data(), (int)held.size());
        if (rc) return rc;
    }
    const int rc = c->slots.release(&r.state_slot, 1);
    if (rc) return rc;
    for (size_t i = 0; i < c->fresh_slots.size(); ++i)
        if (c->fresh_slots[i] == r.state_slot) { c->fresh_slots.erase(c->fresh_slots.begin() + i); break; }
    c->requests.erase(it);
    return VC_OK;
}

int vc_has(void* h, long long key) { return static_cast<Core*>(h)->requests.count(key) ? 1 : 0; }

// need[g] = pages group g must still take before `count` more tokens fit
int vc_pages_needed(void* h, long long key, long long count, int* need) {
    Core* c = static_cast<Core*>(h);
    auto it = c->requests.find(key);
    if (it == c->requests.end()) return VC_UNKNOWN;
    for (size_t g = 0; g < c->pools.size(); ++g) need[g] = c->pages_needed(it->second, count, (int)g);
    return VC_OK;
}

// Takes the pages `count` more tokens need, in every group or in none; *start = position of the first new token.
int vc_append(void* h, long long key, long long count, long long* start) {
    Core* c = static_cast<Core*>(h);
    if (count <= 0) return VC_ARGUMENT;
    auto it = c->requests.find(key);
    if (it == c->requests.end()) return VC_UNKNOWN;
    Request& r = it->second;
    for (size_t g = 0; g < c->pools.size(); ++g)
        if (c->pages_needed(r, count, (int)g) > c->pools[g].free_count()) return VC_NO_SPACE;
    for (size_t g = 0; g < c->pools.size(); ++g) c->pools[g].allocate(c->pages_needed(r, count, (int)g), r.tables[g]);
    if (start) *start = r.num_tokens;
    r.num_tokens += count;
    return VC_OK;
}

// Gives back the pages that no later query of the request can read: the next query sits at
// position num_tokens and reads from num_tokens - window + 1 on.  *freed = pages returned.
int vc_release_behind_window(void* h, long long key, int* freed) {
    Core* c = static_cast<Core*>(h);
    auto it = c->requests.find(key);
    if (it == c->requests.end()) return VC_UNKNOWN;
    Request& r = it->second;
    int total = 0;
    for (size_t g = 0; g < c->pools.size(); ++g) {
        const int w = c->windows[g];
        if (w <= 0) continue;
        long long first_needed = r.num_tokens - w + 1;
        if (first_needed < 0) first_needed = 0;
        long long dead = first_needed / c->page_size;
        if (dead > (long long)r.tables[g].size()) dead = (long long)r.tables[g].size();
        std::vector<int> gone;
        for (long long b = 0; b < dead; ++b)
            if (r.tables[g][b] >= 0) { gone.push_back(r.tables[g][b]); r.tables[g][b] = -1; }
        const int rc = c->pools[g].release(gone.data(), (int)gone.size());
        if (rc) return rc;
        total += (int)gone.size();
    }
    if (freed) *freed = total;
    return VC_OK;
}

int vc_request_info(void* h, long long key, long long* num_tokens, int* state_slot) {
    Core* c = static_cast<Core*>(h);
    auto it = c->requests.find(key);
    if (it == c->requests.end()) return VC_UNKNOWN;
    if (num_tokens) *num_tokens = it->second.num_tokens;
    if (state_slot) *state_slot = it->second.state_slot;
    return VC_OK;
}

// Length of the block table of a group (out == nullptr) or a copy of it (up to capacity entries).
int vc_block_table(void* h, long long key, int group, int* out, int capacity) {
    Core* c = static_cast<Core*>(h);
    auto it = c->requests.find(key);
    if (it == c->requests.end() || group < 0 || group >= (int)c->pools.size()) return VC_UNKNOWN;
    const std::vector<int>& t = it->second.tables[group];
    if (out) std::memcpy(out, t.data(), sizeof(int) * (size_t)((int)t.size() < capacity ? (int)t.size() : capacity));
    return (int)t.size();
}

int vc_slot_of(void* h, long long key, int group, long long position, long long* slot) {
    Core* c = static_cast<Core*>(h);
    auto it = c->requests.find(key);
    if (it == c->requests.end() || group < 0 || group >= (int)c->pools.size()) return VC_UNKNOWN;
    const std::vector<int>& t = it->second.tables[group];
    const long long blk = position / c->page_size;
    if (position < 0 || blk >= (long long)t.size()) return VC_ARGUMENT;
    if (t[blk] < 0) return VC_GONE;
    *slot = (long long)t[blk] * c->page_size + position % c->page_size;
    return VC_OK;
}

int vc_pool_counts(void* h, int group, int* size, int* free_count) {      // group -1: the state slots
    Core* c = static_cast<Core*>(h);
    const Pool* p = group < 0 ? &c->slots : (group < (int)c->pools.size() ? &c->pools[group] : nullptr);
    if (!p) return VC_UNKNOWN;
    if (size) *size = p->size();
    if (free_count) *free_count = p->free_count();
    return VC_OK;
}

int vc_is_held(void* h, int group, int unit) {
    Core* c = static_cast<Core*>(h);
    const Pool* p = group < 0 ? &c->slots : (group < (int)c->pools.size() ? &c->pools[group] : nullptr);
    if (!p || unit < 0 || unit >= p->size()) return VC_UNKNOWN;
    return p->held[unit] ? 1 : 0;
}

// Copies the slots handed out since the last call (up to capacity) and forgets them; returns their number.
int vc_take_fresh_slots(void* h, int* out, int capacity) {
    Core* c = static_cast<Core*>(h);
    const int n = (int)c->fresh_slots.size() < capacity ? (int)c->fresh_slots.size() : capacity;
    if (out) std::memcpy(out, c->fresh_slots.data(), sizeof(int) * (size_t)n);
    c->fresh_slots.erase(c->fresh_slots.begin(), c->fresh_slots.begin() + n);
    return n;
}

int vc_num_requests(void* h) { return (int)static_cast<Core*>(h)->requests.size(); }

// No page lost, none held twice, none both free and held; slots and requests agree.
int vc_check(void* h) {
    Core* c = static_cast<Core*>(h);
    for (size_t g = 0; g < c->pools.size(); ++g) {
        const Pool& p = c->pools[g];
        std::vector<char> seen(p.size(), 0);
        for (int u : p.free_list) {
            if (u < 0 || u >= p.size() || seen[u] || p.held[u]) return VC_CORRUPT;
            seen[u] = 1;
        }
        int in_tables = 0, held = 0;
        for (char b : p.held) held += b;
        if (held + p.free_count() != p.size()) return VC_CORRUPT;
        std::vector<char> owned(p.size(), 0);
        for (const auto& kv : c->requests)
            for (int pg : kv.second.tables[g]) {
                if (pg < 0) continue;
                if (pg >= p.size() || owned[pg] || !p.held[pg]) return VC_CORRUPT;
                owned[pg] = 1;
                ++in_tables;
            }
        if (in_tables != held) return VC_CORRUPT;
    }
    std::vector<char> slot_seen(c->slots.size(), 0);
    for (const auto& kv : c->requests) {
        const int s = kv.second.state_slot;
        if (s < 0 || s >= c->slots.size() || slot_seen[s] || !c->slots.held[s]) return VC_CORRUPT;
        slot_seen[s] = 1;
    }
    if ((int)c->requests.size() != c->slots.size() - c->slots.free_count()) return VC_CORRUPT;
    return VC_OK;
}

// ---- packing a step ---------------------------------------------------------------------------
// The batch of a step as one int32 buffer of 16-byte aligned sections:
//   tokens[T] positions[T] req_index[T] cu_seqlens[B+1] state_slots[B] logit_rows[R] tiles[4*NT]
//   single_tokens[ND], and per group g: slots[T] table[B * max_blocks[g]]
// tiles: up to tile_rows (0: no list) consecutive tokens of a request that brings more than one token (for the
// prefill attention kernel); single_tokens: indices of the tokens of requests that bring exactly
// one (for the decode attention kernel) when the step holds both kinds.
// B, T, R are the padded sizes (pad_to > 0: a decode step padded to pad_to requests; padded tokens
// sit at position -1 with slot -1 and read nothing).  max_blocks[g] in: 0 = widest table of the
// step (at least 1), else the fixed width.  offsets receives 8 + 2 * groups section offsets; the
// return value is the number of int32 words used (or needed, when capacity is too small: then
// nothing is written), or a negative code.
//   keys[B], counts[B], starts[B]  one entry per request (starts = position of its first new token)
//   tokens                         all new tokens, entry after entry
//   want_offsets[B+1], wants       places (within an entry's tokens) whose logits are wanted
long long vc_pack_step(void* h, int B_real, const long long* keys, const int* counts, const long long* starts,
                       const int* tokens, const int* want_offsets, const int* wants, int pad_to, int tile_rows,
                       int* max_blocks, int* out, long long capacity, int* offsets, int* sizes) {
    Core* c = static_cast<Core*>(h);
    const int G = (int)c->pools.size();
    if (B_real <= 0) return VC_ARGUMENT;
    std::vector<const Request*> reqs(B_real);
    long long T_real = 0;
    for (int b = 0; b < B_real; ++b) {
        auto it = c->requests.find(keys[b]);
        if (it == c->requests.end()) return VC_UNKNOWN;
        reqs[b] = &it->second;
        if (counts[b] <= 0) return VC_ARGUMENT;
        T_real += counts[b];
    }
    const int R_real = want_offsets[B_real];
    const int B = pad_to > 0 ? pad_to : B_real;
    const long long T = pad_to > 0 ? pad_to : T_real;
    const int R = pad_to > 0 ? pad_to : R_real;
    if (pad_to > 0 && (B_real > pad_to || T_real != B_real || R_real != B_real)) return VC_ARGUMENT;
    int num_tiles = 0, num_single = 0;
    if (tile_rows > 0 && pad_to <= 0) {
        for (int b = 0; b < B_real; ++b) {
            if (counts[b] > 1) num_tiles += (counts[b] + tile_rows - 1) / tile_rows;
            else ++num_single;
        }
        if (num_tiles == 0) num_single = 0;          // a step of single tokens only needs no list
    }
    for (int g = 0; g < G; ++g) {
        if (max_blocks[g] <= 0) {
            int widest = 1;
            for (int b = 0; b < B_real; ++b) widest = widest > (int)reqs[b]->tables[g].size() ? widest : (int)reqs[b]->tables[g].size();
            max_blocks[g] = widest;
        }
    }
    long long cursor = 0;
    int si = 0;
    auto section = [&](long long n) {
        offsets[si] = (int)cursor;
        sizes[si] = (int)n;
        ++si;
        cursor += align4((int)(n > 0 ? n : 1));
    };
    section(T); section(T); section(T); section(B + 1); section(B); section(R); section(4LL * num_tiles);
    section(num_single);
    for (int g = 0; g < G; ++g) { section(T); section((long long)B * max_blocks[g]); }
    if (cursor > capacity) return cursor;
    for (long long i = 0; i < cursor; ++i) out[i] = -1;
    int* tok = out + offsets[0];
    int* pos = out + offsets[1];
    int* req = out + offsets[2];
    int* cu = out + offsets[3];
    int* sslot = out + offsets[4];
    int* rows = out + offsets[5];
    int* tiles = out + offsets[6];
    int* single = out + offsets[7];
    if (pad_to > 0) {
        for (long long i = 0; i < T; ++i) { tok[i] = 0; req[i] = 0; rows[i] = (int)i; }
        for (int b = 0; b <= B; ++b) cu[b] = (int)T_real;
        for (int b = 0; b < B; ++b) sslot[b] = 0;
    }
    cu[0] = 0;
    long long t = 0;
    int r = 0, ti = 0, si1 = 0;
    for (int b = 0; b < B_real; ++b) {
        const int n = counts[b];
        for (int i = 0; i < n; ++i) {
            tok[t + i] = tokens[t + i];
            pos[t + i] = (int)(starts[b] + i);
            req[t + i] = b;
        }
        for (int w = want_offsets[b]; w < want_offsets[b + 1]; ++w) {
            if (wants[w] < 0 || wants[w] >= n) return VC_ARGUMENT;
            rows[r++] = (int)(t + wants[w]);
        }
        if (num_tiles > 0 && n > 1)
            for (int lo = 0; lo < n; lo += tile_rows) {
                tiles[4 * ti] = b; tiles[4 * ti + 1] = (int)(t + lo);
                tiles[4 * ti + 2] = n - lo < tile_rows ? n - lo : tile_rows; tiles[4 * ti + 3] = (int)(starts[b] + lo);
                ++ti;
            }
        if (num_single > 0 && n == 1) single[si1++] = (int)t;
        sslot[b] = reqs[b]->state_slot;
        t += n;
        cu[b + 1] = (int)t;
    }
    for (int g = 0; g < G; ++g) {
        int* sl = out + offsets[8 + 2 * g];
        int* tb = out + offsets[9 + 2 * g];
        const int mb = max_blocks[g];
        long long tt = 0;
        for (int b = 0; b < B_real; ++b) {
            const std::vector<int>& table = reqs[b]->tables[g];
            const int len = (int)table.size() < mb ? (int)table.size() : mb;
            std::memcpy(tb + (long long)b * mb, table.data(), sizeof(int) * (size_t)len);
            for (int i = 0; i < counts[b]; ++i) {
                const long long p = starts[b] + i;
                const long long blk = p / c->page_size;
                if (blk >= (long long)table.size() || table[blk] < 0) return VC_GONE;
                sl[tt + i] = (int)((long long)table[blk] * c->page_size + p % c->page_size);
            }
            tt += counts[b];
        }
    }
    return cursor;
}

// A decode step in one call: every request brings one token and wants its logits.  Checks that
// the pools can take all the tokens (else VC_NO_SPACE, nothing changed), appends them, packs the
// batch as vc_pack_step does (padded to pad_to requests, block tables max_blocks_fixed wide) and
// gives back the pages that windows have passed.  starts_out[b] receives the position of request
// b's token.  A request that would grow beyond max_tokens: VC_TOO_LONG, nothing changed.
long long vc_decode_step(void* h, int B, const long long* keys, const int* tokens, int pad_to, int max_blocks_fixed,
                         long long max_tokens, int* out, long long capacity, int* offsets, int* sizes,
                         long long* starts_out) {
    Core* c = static_cast<Core*>(h);
    const int G = (int)c->pools.size();
    if (B <= 0 || pad_to < B || max_blocks_fixed <= 0) return VC_ARGUMENT;
    std::vector<Request*> reqs(B);
    std::vector<int> need(G, 0);
    for (int b = 0; b < B; ++b) {
        auto it = c->requests.find(keys[b]);
        if (it == c->requests.end()) return VC_UNKNOWN;
        reqs[b] = &it->second;
        for (int a = 0; a < b; ++a)
            if (reqs[a] == reqs[b]) return VC_ARGUMENT;
        if (reqs[b]->num_tokens + 1 > max_tokens) return VC_TOO_LONG;
        for (int g = 0; g < G; ++g) need[g] += c->pages_needed(*reqs[b], 1, g);
    }
    for (int g = 0; g < G; ++g)
        if (need[g] > c->pools[g].free_count()) return VC_NO_SPACE;
    long long required = 3LL * align4(pad_to) + align4(pad_to + 1) + 2LL * align4(pad_to) + 2LL * align4(1);
    for (int g = 0; g < G; ++g) required += align4(pad_to) + align4(pad_to * max_blocks_fixed);
    if (required > capacity) return required;        // nothing changed: call again with a larger buffer
    std::vector<int> counts(B, 1), want_offsets(B + 1), wants(B, 0), max_blocks(G > 0 ? G : 1, max_blocks_fixed);
    std::vector<long long> starts(B);
    for (int b = 0; b < B; ++b) {
        Request& r = *reqs[b];
        for (int g = 0; g < G; ++g) c->pools[g].allocate(c->pages_needed(r, 1, g), r.tables[g]);
        starts[b] = r.num_tokens;
        r.num_tokens += 1;
        want_offsets[b] = b;
        if (starts_out) starts_out[b] = starts[b];
    }
    want_offsets[B] = B;
    const long long used = vc_pack_step(h, B, keys, counts.data(), starts.data(), tokens, want_offsets.data(),
                                        wants.data(), pad_to, 0, max_blocks.data(), out, capacity, offsets, sizes);
    if (used < 0 || used > capacity) return used;
    for (int b = 0; b < B; ++b) {
        const int rc = vc_release_behind_window(h, keys[b], nullptr);
        if (rc) return rc;
    }
    return used;
}

// ---- the scheduler's decision ---------------------------------------------------------------------
// What one step holds, decided from the state of the queues and of the pools (engine/scheduler.py
// states the policy and is the reference implementation; both run the same tests).  Nothing is
// changed here: the caller applies the answer (pre-empts the victims, moves the admitted).
//   Sequences are numbered 0 .. n_run + n_wait - 1: the running ones in order of arrival, then the
//   queue from its head.  remaining[i] = tokens not yet in the cache (1: decoding), computed[i] =
//   tokens in the cache, keys[i] = the cache's key of the request or 0 when it holds nothing,
//   arrival[i] = its arrival number.
//   A step holds the next token of every decoding request, then portions of running prompts, then
//   admissions from the head of the queue, under max_num_batched_tokens / max_num_seqs /
//   prefill_chunk_size (the last bounds a prompt's portion only in a step that also decodes); a running sequence that cannot get its pages makes the most recently arrived
//   running sequence a victim (its pages count as free, it goes back to the head of the queue with
//   all its tokens to compute) and the step is composed again.
//   Out: entries (sequence number, tokens) in step order, victims in the order they were chosen, and
//   admitted sequence numbers in order.  Returns the number of entries, or VC_NO_SPACE when a sequence
//   that runs alone cannot get its pages, VC_ARGUMENT for inconsistent input.
int vs_schedule(void* h, int max_num_seqs, long long max_num_batched_tokens, long long prefill_chunk_size,
                int n_run, int n_wait, const long long* remaining, const long long* computed, const long long* keys,
                const long long* arrival, int* entry_seq, long long* entry_count, int* n_entries,
                int* victims, int* n_victims, int* admitted, int* n_admitted) {
    Core* c = static_cast<Core*>(h);
    const int G = (int)c->pools.size();
    const long long ps = c->page_size;
    if (n_run < 0 || n_wait < 0 || max_num_seqs <= 0 || max_num_batched_tokens <= 0 || prefill_chunk_size <= 0) return VC_ARGUMENT;
    const int n = n_run + n_wait;
    std::vector<long long> rem(remaining, remaining + n), comp(computed, computed + n);
    std::vector<char> holds(n, 0);                   // the sequence holds pages (and a slot) in the cache
    std::vector<int> running, waiting;
    for (int i = 0; i < n; ++i) {
        if (keys[i]) {
            if (!c->requests.count(keys[i])) return VC_UNKNOWN;
            holds[i] = 1;
        }
        (i < n_run ? running : waiting).push_back(i);
    }
    std::vector<int> extra_free(G, 0);               // pages of the victims chosen so far
    int extra_slots = 0;
    *n_victims = 0;
    auto pages_for = [&](int i, long long count) {    // the blocks that count more positions open
        const long long held = holds[i] ? comp[i] : 0;
        return (int)((held + count + ps - 1) / ps - (held + ps - 1) / ps);
    };
    bool capped = true;                              // prefill_chunk_size bounds portions only beside decoding requests
    auto chunk = [&](int i, long long room) {
        long long k = rem[i] < room ? rem[i] : room;
        if (rem[i] > 1 && capped && k > prefill_chunk_size) k = prefill_chunk_size;
        return k;
    };
    for (;;) {
        capped = false;
        for (int i : running) capped = capped || rem[i] == 1;
        std::vector<int> free(G);
        for (int g = 0; g < G; ++g) free[g] = c->pools[g].free_count() + extra_free[g];
        int free_slots = c->slots.free_count() + extra_slots;
        long long room = max_num_batched_tokens;
        std::vector<int> es;
        std::vector<long long> ec;
        std::vector<int> run_now = running, wait_now = waiting, adm;
        int starved = -1;
        std::vector<int> order;
        for (int i : run_now) if (rem[i] == 1) order.push_back(i);
        for (int i : run_now) if (rem[i] > 1) order.push_back(i);
        for (int i : order) {
            const long long k = chunk(i, room);
            if (k <= 0) continue;
            const int need = pages_for(i, k);
            bool fits = true;
            for (int g = 0; g < G; ++g) fits = fits && need <= free[g];
            if (!fits) {
                if (run_now.size() == 1 && es.empty()) return VC_NO_SPACE;
                starved = i;
                break;
            }
            for (int g = 0; g < G; ++g) free[g] -= need;
            room -= k;
            es.push_back(i); ec.push_back(k);
        }
        if (starved < 0) {
            size_t head = 0;
            while (head < wait_now.size() && room > 0 && (int)run_now.size() < max_num_seqs) {
                const int i = wait_now[head];
                const long long k = chunk(i, room);
                const int need = pages_for(i, k);
                bool fits = true;
                for (int g = 0; g < G; ++g) fits = fits && need <= free[g];
                if (!fits || (!holds[i] && free_slots < 1)) break;     // head of line: never admit what cannot get pages
                ++head;
                run_now.push_back(i);
                if (!holds[i]) --free_slots;
                for (int g = 0; g < G; ++g) free[g] -= need;
                room -= k;
                es.push_back(i); ec.push_back(k);
                adm.push_back(i);
            }
            *n_entries = (int)es.size();
            for (size_t e = 0; e < es.size(); ++e) { entry_seq[e] = es[e]; entry_count[e] = ec[e]; }
            *n_admitted = (int)adm.size();
            for (size_t a = 0; a < adm.size(); ++a) admitted[a] = adm[a];
            return (int)es.size();
        }
        // the most recently arrived running sequence yields
        int v = running[0];
        for (int i : running) if (arrival[i] > arrival[v]) v = i;
        running.erase(std::find(running.begin(), running.end(), v));
        if (holds[v]) {
            const Request& r = c->requests[keys[v]];
            for (int g = 0; g < G; ++g)
                for (int page : r.tables[g]) if (page >= 0) ++extra_free[g];
            ++extra_slots;
            holds[v] = 0;
        }
        rem[v] += comp[v];                            // everything is computed again
        comp[v] = 0;
        waiting.insert(waiting.begin(), v);
        victims[(*n_victims)++] = v;
    }
}

}  // extern "C"
