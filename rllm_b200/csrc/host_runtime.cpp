// Host runtime of the engine in C++: page allocator, cache manager (groups of layers with their
// own page pools, block tables per request, windows that give pages back, state slots) and the
// builder that turns a step's items into the flat int32 arrays the kernels read, written straight
// into the pinned staging buffer.  No CUDA in this file; Python reaches it through the extern "C"
// functions at the end (ctypes).
//
// Behaviour follows AxiomOperator/rllm's host crates: BlockAllocator and SeqKv
// (crates/rllm-kv/src/lib.rs:17-133: free list popped lowest id first, all-or-nothing append,
// slot = page * block_size + offset) and the batch flattening of KvPool::step_sampled
// (crates/rllm-model/src/generate.rs:85-139: tokens, positions, token -> request, logit rows,
// block tables; pre-checks before any mutation).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

struct Allocator {
    std::vector<int> free_list;      // back() is the lowest free id
    std::vector<int> ref;
    explicit Allocator(int n) : ref(n, 0) {
        free_list.reserve(n);
        for (int i = n - 1; i >= 0; --i) free_list.push_back(i);
    }
    int n_free() const { return (int)free_list.size(); }
    int take() {
        int b = free_list.back();
        free_list.pop_back();
        ref[b] = 1;
        return b;
    }
    bool release(int b) {
        if (b < 0 || b >= (int)ref.size() || ref[b] <= 0) return false;
        if (--ref[b] == 0) free_list.push_back(b);
        return true;
    }
};

struct Request {
    int length = 0;
    int state_slot = -1;
    std::vector<std::vector<int>> tables;   // per group: page per logical block, -1 = given back
};

struct Group {
    int window;
    Allocator alloc;
    int n_blocks;                    // pages of this group's pool
    Group(int w, int nb) : window(w), alloc(nb), n_blocks(nb) {}
};

enum : int { OK = 0, ERR_OUT_OF_PAGES = 1, ERR_OUT_OF_SLOTS = 2, ERR_UNKNOWN_REQUEST = 3, ERR_BAD_ARG = 4,
             ERR_DOUBLE_FREE = 5, ERR_INVARIANT = 6, ERR_LIVE_TWICE = 7, ERR_BUFFER = 8, ERR_TOO_LONG = 9 };

// Pages of a windowed group are given back in runs of this many keys: the attention kernels
// round the start of a window down to their key tile (at most 128 keys) and load whole tiles,
// so a page is only handed to another request once no tile that is still read touches it.
constexpr int RELEASE_ALIGN = 128;

struct Cache {
    int block_size, n_blocks, max_requests;
    std::vector<Group> groups;
    std::vector<int> free_slots;
    std::unordered_map<int64_t, Request> requests;
    int last_need = 0, last_free = 0;        // of the most recent refusal
    int max_length = 0;                      // most tokens a request may hold (0: no limit)

    // group_blocks: pages of each group's pool (null: nb for all; a windowed group may have fewer)
    Cache(int n_groups, const int* windows, int bs, int nb, int mr, const int* group_blocks = nullptr)
        : block_size(bs), n_blocks(nb), max_requests(mr) {
        for (int g = 0; g < n_groups; ++g) groups.emplace_back(windows[g], group_blocks ? group_blocks[g] : nb);
        for (int s = mr - 1; s >= 0; --s) free_slots.push_back(s);
    }
    int blocks_for(int tokens) const { return (tokens + block_size - 1) / block_size; }

    void pages_needed(int64_t rid, int n_new, int* out) const {
        auto it = requests.find(rid);
        const int length = it == requests.end() ? 0 : it->second.length;
        for (size_t g = 0; g < groups.size(); ++g) {
            const int have = it == requests.end() ? 0 : (int)it->second.tables[g].size();
            out[g] = std::max(0, blocks_for(length + n_new) - have);
        }
    }
    // 0 if all items can be appended together, else an error code (nothing is taken either way)
    int check_append(int n_items, const int64_t* rids, const int* n_new) {
        std::vector<int> need(groups.size(), 0), one(groups.size());
        int new_requests = 0;
        for (int i = 0; i < n_items; ++i) {
            if (n_new[i] <= 0) return ERR_BAD_ARG;
            auto it = requests.find(rids[i]);
            if (it == requests.end()) ++new_requests;
            const int length = (it == requests.end() ? 0 : it->second.length) + n_new[i];
            if (max_length > 0 && length > max_length) { last_need = length; last_free = max_length; return ERR_TOO_LONG; }
            pages_needed(rids[i], n_new[i], one.data());
            for (size_t g = 0; g < groups.size(); ++g) need[g] += one[g];
        }
        if (new_requests > (int)free_slots.size()) {
            last_need = new_requests; last_free = (int)free_slots.size();
            return ERR_OUT_OF_SLOTS;
        }
        for (size_t g = 0; g < groups.size(); ++g)
            if (need[g] > groups[g].alloc.n_free()) {
                last_need = need[g]; last_free = groups[g].alloc.n_free();
                return ERR_OUT_OF_PAGES;
            }
        return OK;
    }
    int add_request(int64_t rid) {
        if (requests.count(rid)) return ERR_LIVE_TWICE;
        if (free_slots.empty()) { last_need = 1; last_free = 0; return ERR_OUT_OF_SLOTS; }
        Request r;
        r.state_slot = free_slots.back();
        free_slots.pop_back();
        r.tables.resize(groups.size());
        requests.emplace(rid, std::move(r));
        return OK;
    }
    // slots_out: [group][n_new]
    int append(int64_t rid, int n_new, int* slots_out, int* is_new) {
        int st = check_append(1, &rid, &n_new);
        if (st) return st;
        if (is_new) *is_new = 0;
        if (!requests.count(rid)) {
            st = add_request(rid);
            if (st) return st;
            if (is_new) *is_new = 1;
        }
        Request& r = requests[rid];
        for (size_t g = 0; g < groups.size(); ++g) {
            auto& table = r.tables[g];
            const int want = blocks_for(r.length + n_new);
            while ((int)table.size() < want) table.push_back(groups[g].alloc.take());
            if (slots_out)
                for (int i = 0; i < n_new; ++i) {
                    const int p = r.length + i;
                    slots_out[g * n_new + i] = table[p / block_size] * block_size + p % block_size;
                }
        }
        r.length += n_new;
        return OK;
    }
    int release_passed(int64_t rid, int* released) {
        auto it = requests.find(rid);
        if (it == requests.end()) return ERR_UNKNOWN_REQUEST;
        int count = 0;
        for (size_t g = 0; g < groups.size(); ++g) {
            if (groups[g].window <= 0) continue;
            const int first = std::max(0, it->second.length + 1 - groups[g].window) / RELEASE_ALIGN * RELEASE_ALIGN / block_size;
            auto& table = it->second.tables[g];
            for (int b = 0; b < std::min(first, (int)table.size()); ++b)
                if (table[b] >= 0) {
                    if (!groups[g].alloc.release(table[b])) return ERR_DOUBLE_FREE;
                    table[b] = -1;
                    ++count;
                }
        }
        if (released) *released = count;
        return OK;
    }
    int free_request(int64_t rid) {
        auto it = requests.find(rid);
        if (it == requests.end()) return ERR_UNKNOWN_REQUEST;
        for (size_t g = 0; g < groups.size(); ++g)
            for (int b : it->second.tables[g])
                if (b >= 0 && !groups[g].alloc.release(b)) return ERR_DOUBLE_FREE;
        free_slots.push_back(it->second.state_slot);
        requests.erase(it);
        return OK;
    }
    int truncate(int64_t rid, int length) {
        auto it = requests.find(rid);
        if (it == requests.end()) return ERR_UNKNOWN_REQUEST;
        if (length > it->second.length || length < 0) return ERR_BAD_ARG;
        const int keep = blocks_for(length);
        for (size_t g = 0; g < groups.size(); ++g) {
            auto& table = it->second.tables[g];
            while ((int)table.size() > keep) {
                if (table.back() >= 0 && !groups[g].alloc.release(table.back())) return ERR_DOUBLE_FREE;
                table.pop_back();
            }
        }
        it->second.length = length;
        return OK;
    }
    int check_invariants() const {
        for (size_t g = 0; g < groups.size(); ++g) {
            const int nb = groups[g].n_blocks;
            std::vector<int> seen(nb, 0);
            int held = 0;
            for (auto& kv : requests)
                for (int b : kv.second.tables[g])
                    if (b >= 0) { if (b >= nb || seen[b]++) return ERR_INVARIANT; ++held; }
            for (int b : groups[g].alloc.free_list) { if (b < 0 || b >= nb || seen[b]++) return ERR_INVARIANT; }
            if (held + groups[g].alloc.n_free() != nb) return ERR_INVARIANT;
        }
        std::vector<int> slot_seen(max_requests, 0);
        for (auto& kv : requests) {
            const int s = kv.second.state_slot;
            if (s < 0 || s >= max_requests || slot_seen[s]++) return ERR_INVARIANT;
        }
        for (int s : free_slots) if (s < 0 || s >= max_requests || slot_seen[s]++) return ERR_INVARIANT;
        if ((int)requests.size() + (int)free_slots.size() != max_requests) return ERR_INVARIANT;
        return OK;
    }
};

inline int round4(int n) { return (n + 3) / 4 * 4; }

}  // namespace

#define API extern "C" __attribute__((visibility("default")))

API void* rllm_cache_create(int n_groups, const int* windows, int block_size, int n_blocks, int max_requests,
                            const int* group_blocks) {
    if (n_groups < 0 || block_size <= 0 || n_blocks < 0 || max_requests < 0) return nullptr;
    return new Cache(n_groups, windows, block_size, n_blocks, max_requests, group_blocks);
}
API void rllm_cache_destroy(void* c) { delete static_cast<Cache*>(c); }
API int rllm_cache_has(void* c, int64_t rid) { return (int)static_cast<Cache*>(c)->requests.count(rid); }
API int rllm_cache_length(void* c, int64_t rid) {
    auto& r = static_cast<Cache*>(c)->requests;
    auto it = r.find(rid);
    return it == r.end() ? -1 : it->second.length;
}
API void rllm_cache_set_max_length(void* c, int n) { static_cast<Cache*>(c)->max_length = n; }
API int rllm_cache_n_requests(void* c) { return (int)static_cast<Cache*>(c)->requests.size(); }
API int rllm_cache_state_slot(void* c, int64_t rid) {
    auto& r = static_cast<Cache*>(c)->requests;
    auto it = r.find(rid);
    return it == r.end() ? -1 : it->second.state_slot;
}
API int rllm_cache_n_free_pages(void* c, int group) { return static_cast<Cache*>(c)->groups[group].alloc.n_free(); }
API int rllm_cache_n_free_slots(void* c) { return (int)static_cast<Cache*>(c)->free_slots.size(); }
API void rllm_cache_pages_needed(void* c, int64_t rid, int n_new, int* out) { static_cast<Cache*>(c)->pages_needed(rid, n_new, out); }
API int rllm_cache_check_append(void* c, int n_items, const int64_t* rids, const int* n_new) {
    return static_cast<Cache*>(c)->check_append(n_items, rids, n_new);
}
API void rllm_cache_last_refusal(void* c, int* need, int* free_) {
    *need = static_cast<Cache*>(c)->last_need;
    *free_ = static_cast<Cache*>(c)->last_free;
}
API int rllm_cache_add_request(void* c, int64_t rid) { return static_cast<Cache*>(c)->add_request(rid); }
API int rllm_cache_append(void* c, int64_t rid, int n_new, int* slots_out, int* is_new) {
    return static_cast<Cache*>(c)->append(rid, n_new, slots_out, is_new);
}
API int rllm_cache_release_passed(void* c, int64_t rid, int* released) { return static_cast<Cache*>(c)->release_passed(rid, released); }
API int rllm_cache_free(void* c, int64_t rid) { return static_cast<Cache*>(c)->free_request(rid); }
API int rllm_cache_truncate(void* c, int64_t rid, int length) { return static_cast<Cache*>(c)->truncate(rid, length); }
API int rllm_cache_check_invariants(void* c) { return static_cast<Cache*>(c)->check_invariants(); }
// Copies the block table of (rid, group) into out (capacity cap); returns its length; pages given back read as 0.
API int rllm_cache_block_table(void* c, int64_t rid, int group, int* out, int cap, int raw) {
    auto& r = static_cast<Cache*>(c)->requests;
    auto it = r.find(rid);
    if (it == r.end()) return -1;
    const auto& t = it->second.tables[group];
    for (int i = 0; i < (int)t.size() && i < cap; ++i) out[i] = raw ? t[i] : std::max(t[i], 0);
    return (int)t.size();
}

// Builds the flat arrays of a step in `out` (int32, every array starting at a multiple of 4
// entries): tokens[n], positions[n], seq_ids[n], cu_q[R+1], ctx_lens[R], state_slots[R],
// logit_rows[m], then per group slots[n], then per group block_table[R, width].
// Appends every item's tokens to its request first (all-or-nothing: on an error nothing changed).
// pad_requests > 0 gives the step the padded shape of a captured graph: the items with one token
// are padded to that many requests (padding rows: token 0, position 0, slot -1, context 1), the
// tables to pad_width columns.  Every item may have one token (a decode step: all n rows are logit
// rows), or all but the LAST, which is then a portion of a prompt and comes behind the padding
// rows: [one-token items][padding][portion]; the logit rows are the pad_requests one-token rows and
// the portion's last row.  `offsets` receives the start of each array, `meta` = {n, R, m, width,
// total, longest}.  `new_flags[i]` tells whether item i created its request (its state slot must be zeroed).
API int rllm_step_build(void* cv, int n_items, const int64_t* rids, const int* n_tok, const int* tokens_flat,
                        const int* n_want, const int* want_flat, int vocab, int pad_requests, int pad_width,
                        int pad_quantum, int32_t* out, int out_cap, int* offsets, int* meta, int* new_flags) {
    Cache* c = static_cast<Cache*>(cv);
    if (n_items <= 0) return ERR_BAD_ARG;
    int n_real = 0, m = 0;
    {
        int t = 0, w = 0;
        for (int i = 0; i < n_items; ++i) {
            if (n_tok[i] <= 0) return ERR_BAD_ARG;
            for (int j = 0; j < n_tok[i]; ++j) if (tokens_flat[t + j] < 0 || tokens_flat[t + j] >= vocab) return ERR_BAD_ARG;
            for (int j = 0; j < n_want[i]; ++j) if (want_flat[w + j] < 0 || want_flat[w + j] >= n_tok[i]) return ERR_BAD_ARG;
            for (int k = 0; k < i; ++k) if (rids[k] == rids[i]) return ERR_LIVE_TWICE;
            t += n_tok[i]; w += n_want[i];
            n_real += n_tok[i]; m += n_want[i];
        }
    }
    // the padded shape: one-token items first, at most one portion, and that one last
    const bool portion = pad_requests > 0 && n_tok[n_items - 1] > 1;
    const int n_single = portion ? n_items - 1 : n_items;
    if (pad_requests > 0) {
        for (int i = 0; i < n_single; ++i) if (n_tok[i] != 1) return ERR_BAD_ARG;
        if (n_single > pad_requests) return ERR_BAD_ARG;
    }
    int st = c->check_append(n_items, rids, n_tok);
    if (st) return st;
    const int G = (int)c->groups.size();
    const int n_pad = pad_requests > 0 ? pad_requests - n_single : 0;      // padding rows (and requests)
    const int R = n_items + n_pad;
    const int n = n_real + n_pad;
    if (pad_requests) m = pad_requests + (portion ? 1 : 0);
    // table width after the append
    int width = std::max(1, pad_width), longest = 0;
    for (int i = 0; i < n_items; ++i) {
        auto it = c->requests.find(rids[i]);
        const int len = (it == c->requests.end() ? 0 : it->second.length) + n_tok[i];
        longest = std::max(longest, len);
        width = std::max(width, c->blocks_for(len));
    }
    // pad_quantum: the tables are as wide as the longest request rounded up to that many tokens
    if (pad_quantum > 0) width = std::max(width, c->blocks_for((longest + pad_quantum - 1) / pad_quantum * pad_quantum));
    meta[5] = longest;
    int off = 0, k = 0;
    auto place = [&](int count) { offsets[k++] = off; off += round4(count); return offsets[k - 1]; };
    const int o_tok = place(n), o_pos = place(n), o_seq = place(n), o_cu = place(R + 1), o_ctx = place(R),
              o_state = place(R), o_rows = place(m);
    std::vector<int> o_slots(G), o_tab(G);
    for (int g = 0; g < G; ++g) o_slots[g] = place(n);
    for (int g = 0; g < G; ++g) o_tab[g] = place(R * width);
    const int total = std::max(off, 4);
    meta[0] = n; meta[1] = R; meta[2] = m; meta[3] = width; meta[4] = total;
    if (total > out_cap) return ERR_BUFFER;           // nothing appended yet: the caller grows the buffer and retries
    std::memset(out, 0, sizeof(int32_t) * total);
    std::vector<int> slots;
    int base = 0, t = 0, w = 0, row = 0, r = 0;      // r: the request's row in the step
    out[o_cu] = 0;
    for (int i = 0; i < n_items; ++i) {
        if (i == n_single) {
            // padding rows, behind the one-token items (and before the portion, if there is one)
            for (int q = 0; q < n_pad; ++q, ++r, ++base) {
                out[o_seq + base] = r;
                for (int g = 0; g < G; ++g) out[o_slots[g] + base] = -1;
                out[o_cu + r + 1] = base + 1;
                out[o_ctx + r] = 1;
                out[o_state + r] = c->max_requests;     // the state slot that belongs to no request
            }
        }
        const int cnt = n_tok[i];
        auto it = c->requests.find(rids[i]);
        const int start = it == c->requests.end() ? 0 : it->second.length;
        slots.assign((size_t)G * cnt, -1);
        st = c->append(rids[i], cnt, slots.data(), &new_flags[i]);
        if (st) return ERR_INVARIANT;                   // cannot happen after check_append
        for (int j = 0; j < cnt; ++j) {
            out[o_tok + base + j] = tokens_flat[t + j];
            out[o_pos + base + j] = start + j;
            out[o_seq + base + j] = r;
            for (int g = 0; g < G; ++g) out[o_slots[g] + base + j] = slots[(size_t)g * cnt + j];
        }
        if (!pad_requests)
            for (int j = 0; j < n_want[i]; ++j) out[o_rows + row++] = base + want_flat[w + j];
        out[o_cu + r + 1] = base + cnt;
        out[o_ctx + r] = start + cnt;
        const Request& rq = c->requests[rids[i]];
        out[o_state + r] = rq.state_slot;
        for (int g = 0; g < G; ++g) {
            const auto& tab = rq.tables[g];
            for (size_t b = 0; b < tab.size(); ++b) out[o_tab[g] + r * width + (int)b] = std::max(tab[b], 0);
        }
        base += cnt; t += cnt; w += n_want[i];
        ++r;
    }
    if (n_single == n_items)
        for (int q = 0; q < n_pad; ++q, ++r, ++base) {  // padding rows at the end of a decode step
            out[o_seq + base] = r;
            for (int g = 0; g < G; ++g) out[o_slots[g] + base] = -1;
            out[o_cu + r + 1] = base + 1;
            out[o_ctx + r] = 1;
            out[o_state + r] = c->max_requests;
        }
    if (pad_requests) {
        for (int j = 0; j < pad_requests; ++j) out[o_rows + j] = j;
        if (portion) out[o_rows + pad_requests] = n - 1;
    }
    return OK;
}

// ---------------------------------------------------------------------------------------------
// Replay of recorded launches.  A step that is not replayed from a CUDA graph launches the kernels
// of one layer from Python and records them (ops.Trace); the other layers of the same build launch
// the same kernels with their own weights and cache planes.  The record comes here as a list of
// calls: for each, the packed-argument form of its launcher (`name_packed` in the kernel libraries:
// one 64-bit word per argument) and its words.  `rllm_trace_replay` makes all the calls again with
// the words that hold a layer's addresses replaced: `swap_at[i]` is the index of such a word,
// `swap_role[i]` which of the layer's addresses (in the order the caller keeps) stands there.
namespace {
typedef int (*PackedFn)(const unsigned long long*);
struct Recorded {
    std::vector<PackedFn> fns;
    std::vector<int> first;                 // index of a call's first word
    std::vector<unsigned long long> words;
    std::vector<int> swap_at, swap_role;
};
}  // namespace

API void* rllm_trace_create(int n_calls, void* const* fns, const int* n_args, const unsigned long long* words,
                            int n_swap, const int* swap_at, const int* swap_role) {
    if (n_calls < 0 || n_swap < 0) return nullptr;
    Recorded* r = new Recorded;
    int total = 0;
    for (int i = 0; i < n_calls; ++i) {
        r->fns.push_back(reinterpret_cast<PackedFn>(fns[i]));
        r->first.push_back(total);
        total += n_args[i];
    }
    r->words.assign(words, words + total);
    r->swap_at.assign(swap_at, swap_at + n_swap);
    r->swap_role.assign(swap_role, swap_role + n_swap);
    for (int i = 0; i < n_swap; ++i)
        if (swap_at[i] < 0 || swap_at[i] >= total || swap_role[i] < 0) { delete r; return nullptr; }
    return r;
}
API void rllm_trace_destroy(void* t) { delete static_cast<Recorded*>(t); }

// Makes the recorded calls with the layer's addresses `roles[0 .. n_roles)` in their places.
// Returns 0, or the first launcher status that was not 0, with the call's index in *failed_call.
API int rllm_trace_replay(void* t, const unsigned long long* roles, int n_roles, int* failed_call) {
    Recorded* r = static_cast<Recorded*>(t);
    for (size_t i = 0; i < r->swap_at.size(); ++i) {
        if (r->swap_role[i] >= n_roles) return ERR_BAD_ARG;
        r->words[r->swap_at[i]] = roles[r->swap_role[i]];
    }
    for (size_t i = 0; i < r->fns.size(); ++i) {
        const int st = r->fns[i](r->words.data() + r->first[i]);
        if (st) {
            if (failed_call) *failed_call = (int)i;
            return st;
        }
    }
    return OK;
}
