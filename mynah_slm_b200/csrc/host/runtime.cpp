// The host-side runtime behind include/mynah_slm_b200_host.h: page pools, slots, the books of what every live
// sequence holds in every storage group, and the packing of a step's batch description. No device code.
//
// A page holds 64 positions of one storage group. Pages are handed out when a sequence grows into them and given
// back when it ends or, in a group that keeps only a window, as soon as every position of the page has left the
// window. Freed pages and slots are the next to be handed out, so reuse happens at once.
#include "../../include/mynah_slm_b200_host.h"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <map>
#include <new>
#include <thread>
#include <vector>

namespace {

thread_local char g_error[512] = "";

int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return -1;
}

constexpr int PAGE = MYNAH_PAGE_TOKENS;
constexpr int FREE = -1;

}  // namespace

int mynah_page_tokens(void) { return MYNAH_PAGE_TOKENS; }

// ---------------------------------------------------------------- random weights on the host
// The same numbers as the device's mynah_randn_fill, for writing a model folder where there is no device.
#include "../../include/mynah_random_normal.h"

int mynah_randn_fill_host(void* out, int dtype, long long n, unsigned long long seed, unsigned long long tensor_key,
                          double mean, double std) {
    if (n < 0 || (n > 0 && out == nullptr)) return fail("randn_fill_host: bad size %lld", n);
    if (dtype != 0 && dtype != 1) return fail("randn_fill_host: unsupported dtype %d (0: float32, 1: bfloat16)", dtype);
    const uint64_t state = mynah_rn_state(seed, tensor_key);
    auto fill = [=](long long lo, long long hi) {
        if (dtype == 0) {
            float* o = static_cast<float*>(out);
            for (long long i = lo; i < hi; i++) o[i] = mynah_rn_value(state, (uint64_t)i, mean, std);
        } else {
            uint16_t* o = static_cast<uint16_t*>(out);
            for (long long i = lo; i < hi; i++) o[i] = mynah_rn_bf16_bits(mynah_rn_value(state, (uint64_t)i, mean, std));
        }
    };
    // every element stands alone, so large tensors are shared out among threads
    const unsigned hw = std::thread::hardware_concurrency();
    const int n_threads = n < (1 << 20) ? 1 : (int)std::min<long long>(std::max(1u, std::min(hw, 32u)), n >> 18);
    if (n_threads <= 1) {
        fill(0, n);
    } else {
        std::vector<std::thread> pool;
        const long long per = (n + n_threads - 1) / n_threads;
        for (int t = 0; t < n_threads; t++) pool.emplace_back(fill, std::min(n, t * per), std::min(n, (t + 1) * per));
        for (auto& th : pool) th.join();
    }
    return 0;
}

struct mynah_pool {
    int n_pages;
    std::vector<int32_t> free_stack;   // page 0 is handed out first
    std::vector<int32_t> owner;        // FREE or a slot
};

struct mynah_slots {
    int n_slots;
    std::vector<int32_t> free_stack;
    std::vector<char> used;
};

namespace {

struct Held {
    std::vector<int32_t> pages;
    int base = 0;                      // logical index of pages[0]
};

struct Sequence {
    int length = 0;
    std::vector<Held> held;            // one per group
};

void pool_init(mynah_pool& p, int n) {
    p.n_pages = n;
    p.free_stack.resize(n);
    for (int i = 0; i < n; i++) p.free_stack[i] = n - 1 - i;
    p.owner.assign(n, FREE);
}

int pool_take(mynah_pool& p, int n, int owner, int32_t* out) {
    if (n < 0) return fail("cannot take %d pages", n);
    if (n > (int)p.free_stack.size())
        return fail("the cache is full: %d pages wanted, %d of %d free", n, (int)p.free_stack.size(), p.n_pages);
    for (int i = 0; i < n; i++) {
        const int32_t pg = p.free_stack.back();
        if (p.owner[pg] != FREE) return fail("page %d was free and owned by slot %d at once", pg, p.owner[pg]);
        p.free_stack.pop_back();
        p.owner[pg] = owner;
        out[i] = pg;
    }
    return 0;
}

int pool_give_back(mynah_pool& p, const int32_t* pages, int n, int owner) {
    for (int i = 0; i < n; i++) {
        const int32_t pg = pages[i];
        if (pg < 0 || pg >= p.n_pages) return fail("page %d does not exist", pg);
        if (p.owner[pg] != owner) {
            if (p.owner[pg] == FREE) return fail("slot %d gives back page %d, which is free", owner, pg);
            return fail("slot %d gives back page %d, which belongs to slot %d", owner, pg, p.owner[pg]);
        }
        p.owner[pg] = FREE;
        p.free_stack.push_back(pg);
    }
    return 0;
}

void slots_init(mynah_slots& s, int n) {
    s.n_slots = n;
    s.free_stack.resize(n);
    for (int i = 0; i < n; i++) s.free_stack[i] = n - 1 - i;
    s.used.assign(n, 0);
}

}  // namespace

struct mynah_books {
    std::vector<int32_t> windows;      // 0: every position is kept
    std::vector<mynah_pool> pools;
    mynah_slots slots;
    std::map<int, Sequence> live;      // by slot, ascending
};

extern "C" {

const char* mynah_host_last_error(void) { return g_error; }

// ------------------------------------------------------------------ pools
mynah_pool* mynah_pool_create(int n_pages) {
    if (n_pages < 1) {
        fail("a page pool needs at least one page, got %d", n_pages);
        return nullptr;
    }
    mynah_pool* p = new (std::nothrow) mynah_pool();
    if (p != nullptr) pool_init(*p, n_pages);
    return p;
}
void mynah_pool_destroy(mynah_pool* p) { delete p; }
int mynah_pool_take(mynah_pool* p, int n, int owner, int32_t* out) { return pool_take(*p, n, owner, out); }
int mynah_pool_give_back(mynah_pool* p, const int32_t* pages, int n, int owner) { return pool_give_back(*p, pages, n, owner); }
int mynah_pool_owner(const mynah_pool* p, int page) { return page < 0 || page >= p->n_pages ? -2 : p->owner[page]; }
int mynah_pool_n_free(const mynah_pool* p) { return (int)p->free_stack.size(); }
int mynah_pool_n_pages(const mynah_pool* p) { return p->n_pages; }

// ------------------------------------------------------------------ slots
mynah_slots* mynah_slots_create(int n_slots) {
    if (n_slots < 1) {
        fail("a slot table needs at least one slot, got %d", n_slots);
        return nullptr;
    }
    mynah_slots* s = new (std::nothrow) mynah_slots();
    if (s != nullptr) slots_init(*s, n_slots);
    return s;
}
void mynah_slots_destroy(mynah_slots* s) { delete s; }
int mynah_slots_take(mynah_slots* s) {
    if (s->free_stack.empty()) return fail("all %d sequence slots are in use", s->n_slots);
    const int slot = s->free_stack.back();
    s->free_stack.pop_back();
    s->used[slot] = 1;
    return slot;
}
int mynah_slots_give_back(mynah_slots* s, int slot) {
    if (slot < 0 || slot >= s->n_slots || !s->used[slot]) return fail("slot %d is not in use", slot);
    s->used[slot] = 0;
    s->free_stack.push_back(slot);
    return 0;
}
int mynah_slots_in_use(const mynah_slots* s, int slot) { return slot >= 0 && slot < s->n_slots && s->used[slot]; }
int mynah_slots_n_free(const mynah_slots* s) { return (int)s->free_stack.size(); }
int mynah_slots_n_slots(const mynah_slots* s) { return s->n_slots; }

// ------------------------------------------------------------------ books
mynah_books* mynah_books_create(int n_groups, const int32_t* windows, int n_pages, int max_seqs) {
    if (n_groups < 0 || n_pages < 1 || max_seqs < 1) {
        fail("books need pages and slots: %d groups, %d pages, %d slots", n_groups, n_pages, max_seqs);
        return nullptr;
    }
    mynah_books* b = new (std::nothrow) mynah_books();
    if (b == nullptr) return nullptr;
    b->windows.assign(windows, windows + n_groups);
    b->pools.resize(n_groups);
    for (auto& p : b->pools) pool_init(p, n_pages);
    slots_init(b->slots, max_seqs);
    return b;
}
void mynah_books_destroy(mynah_books* b) { delete b; }

int mynah_books_open(mynah_books* b) {
    const int slot = mynah_slots_take(&b->slots);
    if (slot < 0) return -1;
    Sequence& s = b->live[slot];
    s.length = 0;
    s.held.assign(b->pools.size(), Held());
    return slot;
}

int mynah_books_close(mynah_books* b, int slot) {
    auto it = b->live.find(slot);
    if (it == b->live.end()) return fail("slot %d is not open", slot);
    for (size_t g = 0; g < b->pools.size(); g++) {
        Held& h = it->second.held[g];
        if (pool_give_back(b->pools[g], h.pages.data(), (int)h.pages.size(), slot)) return -1;
    }
    b->live.erase(it);
    return mynah_slots_give_back(&b->slots, slot);
}

int mynah_books_length(const mynah_books* b, int slot) {
    auto it = b->live.find(slot);
    return it == b->live.end() ? -1 : it->second.length;
}

int mynah_books_pages_needed(const mynah_books* b, int slot, int n_new) {
    auto it = b->live.find(slot);
    if (it == b->live.end()) return fail("slot %d is not open", slot);
    const int need_total = (it->second.length + n_new + PAGE - 1) / PAGE;
    int most = 0;
    for (const Held& h : it->second.held) most = std::max(most, need_total - (h.base + (int)h.pages.size()));
    return most;
}

int mynah_books_reserve(mynah_books* b, int slot, int n_new) {
    auto it = b->live.find(slot);
    if (it == b->live.end()) return fail("slot %d is not open", slot);
    if (n_new < 0) return fail("cannot reserve a negative number of positions");
    const int need_total = (it->second.length + n_new + PAGE - 1) / PAGE;
    const size_t G = b->pools.size();
    std::vector<int> wants(G);
    for (size_t g = 0; g < G; g++) {               // all or nothing
        const Held& h = it->second.held[g];
        wants[g] = std::max(0, need_total - (h.base + (int)h.pages.size()));
        if (wants[g] > (int)b->pools[g].free_stack.size())
            return fail("the cache is full: %d pages wanted, %d of %d free", wants[g], (int)b->pools[g].free_stack.size(), b->pools[g].n_pages);
    }
    for (size_t g = 0; g < G; g++) {
        Held& h = it->second.held[g];
        const size_t n0 = h.pages.size();
        h.pages.resize(n0 + wants[g]);
        if (pool_take(b->pools[g], wants[g], slot, h.pages.data() + n0)) return -1;
    }
    return 0;
}

int mynah_books_commit(mynah_books* b, int slot, int n_new) {
    auto it = b->live.find(slot);
    if (it == b->live.end()) return fail("slot %d is not open", slot);
    const int n = it->second.length + n_new;
    for (size_t g = 0; g < b->pools.size(); g++) {
        Held& h = it->second.held[g];
        if ((long long)(h.base + (int)h.pages.size()) * PAGE < n)
            return fail("slot %d advanced to %d positions without pages for them", slot, n);
        const int w = b->windows[g];
        if (w > 0) {
            const int first_needed = std::max(0, n - w + 1) / PAGE;
            const int drop = std::min(first_needed - h.base, (int)h.pages.size());
            if (drop > 0) {
                if (pool_give_back(b->pools[g], h.pages.data(), drop, slot)) return -1;
                h.pages.erase(h.pages.begin(), h.pages.begin() + drop);
                h.base += drop;
            }
        }
    }
    it->second.length = n;
    return 0;
}

int mynah_books_held(const mynah_books* b, int slot, int group, int32_t* pages_out, int cap, int32_t* base_out) {
    auto it = b->live.find(slot);
    if (it == b->live.end()) return fail("slot %d is not open", slot);
    if (group < 0 || group >= (int)b->pools.size()) return fail("group %d does not exist", group);
    const Held& h = it->second.held[group];
    if (base_out != nullptr) *base_out = h.base;
    const int n = (int)h.pages.size();
    if (pages_out != nullptr) {
        if (n > cap) return fail("slot %d holds %d pages, the buffer takes %d", slot, n, cap);
        std::copy(h.pages.begin(), h.pages.end(), pages_out);
    }
    return n;
}

int mynah_books_live_slots(const mynah_books* b, int32_t* out, int cap) {
    int n = 0;
    for (const auto& kv : b->live) {
        if (out != nullptr && n < cap) out[n] = kv.first;
        n++;
    }
    return n;
}

const mynah_pool* mynah_books_pool(const mynah_books* b, int group) {
    return group < 0 || group >= (int)b->pools.size() ? nullptr : &b->pools[group];
}
const mynah_slots* mynah_books_slots(const mynah_books* b) { return &b->slots; }

// ------------------------------------------------------------------ the step's description
int mynah_step_fill(const mynah_books* b, int32_t* buf, const int32_t* off, int T, int B, int W, const int32_t* ids_cap,
                    int n_entries, const int32_t* slot, const int32_t* n_tok, const int32_t* tokens,
                    const int32_t* n_want, const int32_t* want, int32_t* n_rows) {
    if (n_entries > B) return fail("%d sequences do not fit a step description of %d", n_entries, B);
    int32_t* tok = buf + off[0];
    int32_t* tok_seq = buf + off[1];
    int32_t* tok_pos = buf + off[2];
    int32_t* cu_q = buf + off[3];
    int32_t* kv_len = buf + off[4];
    int32_t* slots_o = buf + off[5];
    int32_t* want_o = buf + off[6];
    int row = 0, wi = 0, max_q = 0, ti = 0, wj = 0;
    cu_q[0] = 0;
    for (int e = 0; e < n_entries; e++) {
        auto it = b->live.find(slot[e]);
        if (it == b->live.end()) return fail("slot %d is not open", slot[e]);
        const int n = n_tok[e], past = it->second.length;
        if (row + n > T) return fail("%d tokens do not fit a step description of %d", row + n, T);
        for (int j = 0; j < n; j++) {
            tok[row + j] = tokens[ti + j];
            tok_seq[row + j] = e;
            tok_pos[row + j] = past + j;
        }
        const int nw = n_want != nullptr ? n_want[e] : 0;
        if (wi + nw > W) return fail("%d wanted rows do not fit a step description of %d", wi + nw, W);
        for (int j = 0; j < nw; j++) want_o[wi++] = row + want[wj + j];
        wj += nw;
        ti += n;
        row += n;
        cu_q[e + 1] = row;
        kv_len[e] = past + n;
        slots_o[e] = slot[e];
        max_q = std::max(max_q, n);
    }
    for (int e = n_entries; e < B; e++) {          // padding sequences and rows
        cu_q[e + 1] = row;
        kv_len[e] = 0;
        slots_o[e] = -1;
    }
    for (int r = row; r < T; r++) {
        tok[r] = 0;
        tok_seq[r] = -1;
        tok_pos[r] = 0;
    }
    for (size_t g = 0; g < b->pools.size(); g++) {
        int32_t* indptr = buf + off[7 + 3 * g];
        int32_t* base = buf + off[8 + 3 * g];
        int32_t* ids = buf + off[9 + 3 * g];
        int n_ids = 0;
        indptr[0] = 0;
        for (int e = 0; e < n_entries; e++) {
            const Held& h = b->live.find(slot[e])->second.held[g];
            if (n_ids + (int)h.pages.size() > ids_cap[g]) return fail("the page lists of this step outgrow their buffer");
            std::copy(h.pages.begin(), h.pages.end(), ids + n_ids);
            n_ids += (int)h.pages.size();
            indptr[e + 1] = n_ids;
            base[e] = h.base;
        }
        for (int e = n_entries; e < B; e++) {
            indptr[e + 1] = n_ids;
            base[e] = 0;
        }
    }
    if (n_rows != nullptr) *n_rows = wi;
    return max_q;
}

int mynah_decode_prepare(mynah_books* b, int n, const int32_t* slot, const int32_t* token, int vocab, int max_positions,
                         int32_t* buf, const int32_t* off, int T, int B, int W, const int32_t* ids_cap) {
    if (n < 1) return fail("a step needs at least one sequence");
    int max_kv = 0;
    for (int i = 0; i < n; i++) {
        auto it = b->live.find(slot[i]);
        if (it == b->live.end()) return fail("slot %d is not open", slot[i]);
        for (int j = 0; j < i; j++)
            if (slot[j] == slot[i]) return fail("slot %d appears twice in one step", slot[i]);
        if (token[i] < 0 || token[i] >= vocab) return fail("token id %d lies outside the vocabulary of %d", token[i], vocab);
        if (it->second.length + 1 > max_positions)
            return fail("slot %d would grow to %d positions, the model allows %d", slot[i], it->second.length + 1, max_positions);
        max_kv = std::max(max_kv, it->second.length + 1);
    }
    for (int i = 0; i < n; i++)
        if (mynah_books_reserve(b, slot[i], 1)) return -1;
    std::vector<int32_t> ones(n, 1);
    if (mynah_step_fill(b, buf, off, T, B, W, ids_cap, n, slot, ones.data(), token, nullptr, nullptr, nullptr) < 0) return -1;
    return max_kv;
}

int mynah_books_commit_many(mynah_books* b, int n, const int32_t* slot, int n_new) {
    for (int i = 0; i < n; i++)
        if (mynah_books_commit(b, slot[i], n_new)) return -1;
    return 0;
}

}  // extern "C"
