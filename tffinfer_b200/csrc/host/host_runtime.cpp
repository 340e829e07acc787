// See host_runtime.h.
#include "host_runtime.h"

#include <algorithm>
#include <cstdio>
#include <numeric>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

constexpr int NO_PAGE = -1;
constexpr int64_t NOBODY = INT64_MIN;        // owner of a free page or slot

// A fixed number of pages (or slots), a last-in-first-out free list and an owner per page, so that a page
// held twice or freed twice is an error and not a wrong result.
struct Pool {
    int total = 0;
    int high_water = 0;
    std::vector<int> free_list;              // back() is handed out next; page 0 first
    std::vector<int64_t> owner;

    void init(int n) {
        total = n;
        free_list.resize(n);
        for (int i = 0; i < n; ++i) free_list[i] = n - 1 - i;
        owner.assign(n, NOBODY);
    }
    int num_free() const { return (int)free_list.size(); }
    int num_used() const { return total - num_free(); }
    // takes one page; the caller has checked that one is free
    bool take(int64_t who, int* page, std::string& err) {
        const int p = free_list.back();
        if (owner[p] != NOBODY) {
            err = "page " + std::to_string(p) + " on the free list has an owner";
            return false;
        }
        free_list.pop_back();
        owner[p] = who;
        high_water = std::max(high_water, num_used());
        *page = p;
        return true;
    }
    bool give_back(int p, int64_t who, std::string& err) {
        if (p < 0 || p >= total) { err = "page " + std::to_string(p) + " does not exist"; return false; }
        if (owner[p] == NOBODY) { err = "page " + std::to_string(p) + " freed twice"; return false; }
        if (owner[p] != who) { err = "page " + std::to_string(p) + " freed by a request that does not own it"; return false; }
        owner[p] = NOBODY;
        free_list.push_back(p);
        return true;
    }
    bool check(std::string& err) const {
        std::vector<char> seen(total, 0);
        for (int p : free_list) {
            if (p < 0 || p >= total || seen[p]) { err = "a page is on the free list twice"; return false; }
            seen[p] = 1;
            if (owner[p] != NOBODY) { err = "free page " + std::to_string(p) + " has an owner"; return false; }
        }
        int owned = 0;
        for (int64_t o : owner) owned += o != NOBODY;
        if (owned + num_free() != total) { err = "pages lost: owned + free != total"; return false; }
        return true;
    }
};

struct RequestCache {
    int slot = 0;
    int num_tokens = 0;                      // tokens whose keys and values are in the cache
    int reserved_tokens = 0;                 // tokens a step may write up to
    std::vector<std::vector<int>> tables;    // per group: physical page of each logical block
};

struct Cache {
    int page_size = 0;
    std::vector<int> windows;                // per group; 0 = all keys are kept
    std::vector<Pool> pools;
    Pool slots;
    std::unordered_map<int64_t, RequestCache> requests;
    std::string error;

    int fail(int code, const std::string& what) { error = what; return code; }
    RequestCache* find(int64_t req) {
        auto it = requests.find(req);
        return it == requests.end() ? nullptr : &it->second;
    }
    // first logical block that a query at position >= num_tokens can still read
    int first_needed_block(int g, int num_tokens) const {
        const int w = windows[g];
        if (w <= 0) return 0;
        return std::max(0, num_tokens - w + 1) / page_size;      // a query at p sees keys p-w+1 .. p
    }
    void pages_needed(const RequestCache& rc, int n_new, int* per_group) const {
        const int blocks = (rc.num_tokens + n_new + page_size - 1) / page_size;
        for (size_t g = 0; g < pools.size(); ++g)
            per_group[g] = std::max(0, blocks - (int)rc.tables[g].size());
    }
};

Cache* as_cache(void* p) { return static_cast<Cache*>(p); }

}  // namespace

TFFH_API void* tffh_cache_create(int num_groups, const int* windows, int page_size, const int* pages_per_group,
                                 int max_live_requests) {
    if (num_groups < 0 || page_size <= 0 || max_live_requests <= 0) return nullptr;
    for (int g = 0; g < num_groups; ++g)
        if (pages_per_group[g] <= 0) return nullptr;
    Cache* c = new Cache();
    c->page_size = page_size;
    c->windows.assign(windows, windows + num_groups);
    c->pools.resize(num_groups);
    for (int g = 0; g < num_groups; ++g) c->pools[g].init(pages_per_group[g]);
    c->slots.init(max_live_requests);
    return c;
}

TFFH_API void tffh_cache_destroy(void* cache) { delete as_cache(cache); }

TFFH_API const char* tffh_last_error(void* cache) { return cache ? as_cache(cache)->error.c_str() : "no cache"; }

TFFH_API int tffh_admit(void* cache, int64_t req) {
    Cache* c = as_cache(cache);
    if (req == NOBODY) return c->fail(TFFH_ERR_ARGUMENT, "this handle is kept for free pages");
    if (c->find(req)) return c->fail(TFFH_ERR_LIVE, "request " + std::to_string(req) + " is already live");
    if (c->slots.num_free() == 0) return -100;
    int slot;
    if (!c->slots.take(req, &slot, c->error)) return TFFH_ERR_ACCOUNTING;
    RequestCache rc;
    rc.slot = slot;
    rc.tables.resize(c->pools.size());
    c->requests.emplace(req, std::move(rc));
    return slot;
}

TFFH_API int tffh_is_live(void* cache, int64_t req) { return as_cache(cache)->find(req) != nullptr; }

TFFH_API int tffh_num_tokens(void* cache, int64_t req) {
    Cache* c = as_cache(cache);
    RequestCache* rc = c->find(req);
    return rc ? rc->num_tokens : c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(req) + " is not live");
}

TFFH_API int tffh_slot_of(void* cache, int64_t req) {
    Cache* c = as_cache(cache);
    RequestCache* rc = c->find(req);
    return rc ? rc->slot : c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(req) + " is not live");
}

TFFH_API int tffh_pages_needed(void* cache, int64_t req, int n_new, int* per_group) {
    Cache* c = as_cache(cache);
    RequestCache* rc = c->find(req);
    if (!rc) return c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(req) + " is not live");
    if (n_new < 0) return c->fail(TFFH_ERR_ARGUMENT, "n_new must be >= 0");
    c->pages_needed(*rc, n_new, per_group);
    return 0;
}

TFFH_API int tffh_reserve(void* cache, int64_t req, int n_new) {
    Cache* c = as_cache(cache);
    RequestCache* rc = c->find(req);
    if (!rc) return c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(req) + " is not live");
    if (n_new < 0) return c->fail(TFFH_ERR_ARGUMENT, "n_new must be >= 0");
    std::vector<int> need(c->pools.size());
    c->pages_needed(*rc, n_new, need.data());
    for (size_t g = 0; g < need.size(); ++g)
        if (need[g] > c->pools[g].num_free()) return 0;          // all groups or none
    for (size_t g = 0; g < need.size(); ++g)
        for (int i = 0; i < need[g]; ++i) {
            int page;
            if (!c->pools[g].take(req, &page, c->error)) return TFFH_ERR_ACCOUNTING;
            rc->tables[g].push_back(page);
        }
    rc->reserved_tokens = std::max(rc->reserved_tokens, rc->num_tokens + n_new);
    return 1;
}

TFFH_API int tffh_commit(void* cache, int64_t req, int n_new) {
    Cache* c = as_cache(cache);
    RequestCache* rc = c->find(req);
    if (!rc) return c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(req) + " is not live");
    if (n_new < 0) return c->fail(TFFH_ERR_ARGUMENT, "n_new must be >= 0");
    if (rc->num_tokens + n_new > rc->reserved_tokens)
        return c->fail(TFFH_ERR_ACCOUNTING, "request " + std::to_string(req) + ": " + std::to_string(n_new) +
                                                " tokens committed beyond the " + std::to_string(rc->reserved_tokens) +
                                                " reserved");
    rc->num_tokens += n_new;
    // pages that the window of every later query has passed go back to their pool
    for (size_t g = 0; g < c->pools.size(); ++g) {
        std::vector<int>& t = rc->tables[g];
        const int first = std::min(c->first_needed_block((int)g, rc->num_tokens), (int)t.size());
        for (int b = 0; b < first; ++b) {
            if (t[b] == NO_PAGE) continue;
            if (!c->pools[g].give_back(t[b], req, c->error)) return TFFH_ERR_ACCOUNTING;
            t[b] = NO_PAGE;
        }
    }
    return 0;
}

TFFH_API int tffh_release(void* cache, int64_t req) {
    Cache* c = as_cache(cache);
    auto it = c->requests.find(req);
    if (it == c->requests.end()) return c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(req) + " is not live");
    RequestCache rc = std::move(it->second);
    c->requests.erase(it);
    for (size_t g = 0; g < rc.tables.size(); ++g)
        for (int p : rc.tables[g])
            if (p != NO_PAGE && !c->pools[g].give_back(p, req, c->error)) return TFFH_ERR_ACCOUNTING;
    if (!c->slots.give_back(rc.slot, req, c->error)) return TFFH_ERR_ACCOUNTING;
    return 0;
}

TFFH_API int tffh_block_table(void* cache, int64_t req, int group, int* out, int capacity) {
    Cache* c = as_cache(cache);
    RequestCache* rc = c->find(req);
    if (!rc) return c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(req) + " is not live");
    if (group < 0 || group >= (int)c->pools.size()) return c->fail(TFFH_ERR_ARGUMENT, "no such group");
    const std::vector<int>& t = rc->tables[group];
    if (out != nullptr) {
        if ((int)t.size() > capacity) return c->fail(TFFH_ERR_TOO_SMALL, "block table longer than the buffer given");
        std::copy(t.begin(), t.end(), out);
    }
    return (int)t.size();
}

TFFH_API int tffh_count(void* cache, int what, int group) {
    Cache* c = as_cache(cache);
    if (what >= 0 && what <= 2) {
        if (group < 0 || group >= (int)c->pools.size()) return c->fail(TFFH_ERR_ARGUMENT, "no such group");
        const Pool& p = c->pools[group];
        return what == 0 ? p.total : what == 1 ? p.num_free() : p.high_water;
    }
    if (what == 3) return c->slots.num_free();
    if (what == 4) return (int)c->requests.size();
    return c->fail(TFFH_ERR_ARGUMENT, "no such count");
}

// No page lost, none held twice, owners consistent with the block tables.
TFFH_API int tffh_check(void* cache) {
    Cache* c = as_cache(cache);
    for (size_t g = 0; g < c->pools.size(); ++g) {
        const Pool& pool = c->pools[g];
        if (!pool.check(c->error)) return TFFH_ERR_ACCOUNTING;
        std::vector<char> seen(pool.total, 0);
        int held = 0;
        for (const auto& kv : c->requests)
            for (int p : kv.second.tables[g]) {
                if (p == NO_PAGE) continue;
                if (p < 0 || p >= pool.total || seen[p])
                    return c->fail(TFFH_ERR_ACCOUNTING, "group " + std::to_string(g) + ": page " + std::to_string(p) +
                                                            " is held twice");
                if (pool.owner[p] != kv.first)
                    return c->fail(TFFH_ERR_ACCOUNTING, "group " + std::to_string(g) + ": page " + std::to_string(p) +
                                                            " is in the table of a request that does not own it");
                seen[p] = 1;
                ++held;
            }
        if (held != pool.num_used())
            return c->fail(TFFH_ERR_ACCOUNTING, "group " + std::to_string(g) + ": " + std::to_string(pool.num_used()) +
                                                    " pages taken, " + std::to_string(held) + " in block tables");
    }
    if (!c->slots.check(c->error)) return TFFH_ERR_ACCOUNTING;
    int slots_held = 0;
    for (const auto& kv : c->requests) {
        if (c->slots.owner[kv.second.slot] != kv.first) return c->fail(TFFH_ERR_ACCOUNTING, "a slot has the wrong owner");
        ++slots_held;
    }
    if (slots_held != c->slots.num_used()) return c->fail(TFFH_ERR_ACCOUNTING, "slots lost");
    return 0;
}

TFFH_API int64_t tffh_pack_step(void* cache, int n, const int64_t* reqs, const int* q_lens, const int* tokens,
                                const int* want_start, const int* want, const int* tok_src,
                                int pad_requests, int* widths, const int* dummy_pages, int dummy_slot,
                                int* out, int64_t out_capacity, int* info) {
    Cache* c = as_cache(cache);
    if (n <= 0) return c->fail(TFFH_ERR_ARGUMENT, "a step needs at least one request");
    const int G = (int)c->pools.size();
    const int npad = std::max(0, pad_requests - n);
    const int B = n + npad;
    std::vector<const RequestCache*> rcs(n);
    int64_t T = 0;
    for (int i = 0; i < n; ++i) {
        if (q_lens[i] <= 0) return c->fail(TFFH_ERR_ARGUMENT, "every request needs at least one token");
        rcs[i] = c->find(reqs[i]);
        if (!rcs[i]) return c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(reqs[i]) + " is not live");
        T += q_lens[i];
    }
    const int64_t real_tokens = T;
    T += npad;
    const int real_rows = want_start[n];
    const int R = real_rows + npad;
    for (int g = 0; g < G; ++g) {
        int widest = 1;
        for (int i = 0; i < n; ++i) widest = std::max(widest, (int)rcs[i]->tables[g].size());
        if (widths[g] <= 0) widths[g] = widest;
        else if (widest > widths[g])
            return c->fail(TFFH_ERR_ARGUMENT, "a block table is wider than the batch layout allows");
    }
    int64_t total = 3 * T + (B + 1) + 3 * (int64_t)B + R + B + T;
    for (int g = 0; g < G; ++g) total += (int64_t)B * widths[g];
    if (out == nullptr || out_capacity < total) {
        info[0] = (int)total;
        return c->fail(TFFH_ERR_TOO_SMALL, "the buffer given does not hold the batch");
    }
    int* token_ids = out;
    int* positions = token_ids + T;
    int* tok_req = positions + T;
    int* q_start = tok_req + T;
    int* pos_start = q_start + B + 1;
    int* kv_len = pos_start + B;
    int* slot_arr = kv_len + B;
    int* rows = slot_arr + B;
    int* req_order = rows + R;
    int* src = req_order + B;
    int* tables = src + T;

    int max_q = 1, max_kv = 0, has_src = 0;
    int64_t t = 0;
    q_start[0] = 0;
    for (int i = 0; i < B; ++i) {
        const bool real = i < n;
        const int q = real ? q_lens[i] : 1;
        const int start = real ? rcs[i]->num_tokens : 0;
        pos_start[i] = start;
        kv_len[i] = start + q;
        slot_arr[i] = real ? rcs[i]->slot : dummy_slot;
        max_q = std::max(max_q, q);
        if (real) max_kv = std::max(max_kv, kv_len[i]);
        for (int j = 0; j < q; ++j, ++t) {
            int s = (real && tok_src != nullptr) ? tok_src[t] : -1;
            src[t] = s;
            has_src |= s >= 0;
            token_ids[t] = real ? (s >= 0 ? 0 : tokens[t]) : 0;
            positions[t] = start + j;
            tok_req[t] = i;
        }
        q_start[i + 1] = (int)t;
    }
    if (npad > 0) max_kv = std::max(max_kv, 1);
    int r = 0;
    for (int i = 0; i < n; ++i)
        for (int k = want_start[i]; k < want_start[i + 1]; ++k) {
            if (want[k] < 0 || want[k] >= q_lens[i])
                return c->fail(TFFH_ERR_ARGUMENT, "request " + std::to_string(reqs[i]) + ": wanted place " +
                                                      std::to_string(want[k]) + " is outside its " +
                                                      std::to_string(q_lens[i]) + " tokens");
            rows[r++] = q_start[i] + want[k];
        }
    for (int j = 0; j < npad; ++j) rows[r++] = q_start[n + j];
    // by the number of new tokens, and among equals the longest context first (ties: the earlier request):
    // the attention launches take their requests in this order
    std::iota(req_order, req_order + B, 0);
    std::stable_sort(req_order, req_order + B, [&](int a, int b) {
        const int qa = q_start[a + 1] - q_start[a], qb = q_start[b + 1] - q_start[b];
        if (qa != qb) return qa < qb;
        return kv_len[a] > kv_len[b];
    });
    for (int g = 0; g < G; ++g) {
        const int w = widths[g];
        for (int i = 0; i < B; ++i) {
            int* row = tables + (int64_t)i * w;
            if (i < n) {
                const std::vector<int>& tb = rcs[i]->tables[g];
                std::copy(tb.begin(), tb.end(), row);
                std::fill(row + tb.size(), row + w, NO_PAGE);
            } else {
                std::fill(row, row + w, dummy_pages != nullptr ? dummy_pages[g] : NO_PAGE);
            }
        }
        tables += (int64_t)B * w;
    }
    info[0] = (int)T; info[1] = B; info[2] = R; info[3] = max_q; info[4] = max_kv; info[5] = has_src;
    info[6] = real_tokens == n ? 1 : 0;
    info[7] = real_rows;
    return total;
}

// ---------------------------------------------------------------------------------------------- planning
namespace {
struct Candidate {
    int uid;            // index into running[] or n_running + index into waiting[]
    int64_t handle;
    int len;            // prompt + generated tokens
    int prompt_len;
};
}  // namespace

TFFH_API int tffh_plan_step(void* cache, int budget_tokens, int max_model_len,
                            int n_running, const int64_t* running, const int* running_len,
                            int n_waiting, const int64_t* waiting, const int* waiting_len, const int* waiting_prompt_len,
                            int* events, int capacity) {
    Cache* c = as_cache(cache);
    const int G = (int)c->pools.size();
    std::vector<Candidate> run, wait;
    for (int i = 0; i < n_running; ++i) {
        if (!c->find(running[i])) return c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(running[i]) + " is not live");
        run.push_back({i, running[i], running_len[i], 1});      // a live request has a prompt
    }
    for (int j = 0; j < n_waiting; ++j) wait.push_back({n_running + j, waiting[j], waiting_len[j], waiting_prompt_len[j]});
    int n_events = 0;
    auto emit = [&](int kind, int uid, int a, int b) -> bool {
        if (n_events >= capacity) return false;
        int* e = events + 4 * n_events++;
        e[0] = kind; e[1] = uid; e[2] = a; e[3] = b;
        return true;
    };
    const char* too_many = "more events than the buffer given holds";
    // Whether a request of ``len`` tokens can ever run, alone: in a group that keeps all keys it holds pages for
    // all of them; in a group that keeps a window, for the window and one step's tokens (whose pages are taken
    // before those behind the window go back), with a page of slack at either ragged end.
    auto fits_alone = [&](int len) -> bool {
        for (int g = 0; g < G; ++g) {
            const int w = c->windows[g];
            int64_t most = len;
            if (w > 0) most = std::min<int64_t>(most, (int64_t)w + budget_tokens + 2 * (int64_t)c->page_size);
            if (most > (int64_t)c->pools[g].total * c->page_size) return false;
        }
        return true;
    };

    std::vector<std::pair<int, int>> chosen;        // (position in run, tokens)
    std::vector<int> free_pages(G), need(G);
    for (;;) {
        int budget = budget_tokens;
        for (int g = 0; g < G; ++g) free_pages[g] = c->pools[g].num_free();
        chosen.clear();
        bool ok = true;
        // running requests, oldest admission first: decoded tokens (one each), then portions of prompts
        for (int pass = 0; pass < 2 && ok; ++pass)
            for (int i = 0; i < (int)run.size(); ++i) {
                const RequestCache* rc = c->find(run[i].handle);
                const int left = run[i].len - rc->num_tokens;
                if (pass == 0 ? left != 1 : left <= 1) continue;
                if (budget <= 0) { pass = 2; break; }
                const int n = std::min(left, budget);
                c->pages_needed(*rc, n, need.data());
                for (int g = 0; g < G; ++g) ok = ok && need[g] <= free_pages[g];
                if (!ok) break;
                for (int g = 0; g < G; ++g) free_pages[g] -= need[g];
                budget -= n;
                chosen.emplace_back(i, n);
            }
        if (!ok) {
            // pages ran out: the request admitted last gives way (alone, it is too large for the pool)
            const Candidate victim = run.back();
            run.pop_back();
            if (tffh_release(cache, victim.handle) < 0) return TFFH_ERR_ACCOUNTING;
            if (run.empty()) {
                if (!emit(TFFH_EVENT_FINISH, victim.uid, TFFH_REASON_OUT_OF_MEMORY, 1)) return c->fail(TFFH_ERR_TOO_SMALL, too_many);
            } else {
                if (!emit(TFFH_EVENT_PREEMPT, victim.uid, 0, 0)) return c->fail(TFFH_ERR_TOO_SMALL, too_many);
                wait.insert(wait.begin(), victim);
            }
            continue;
        }
        // admissions, in arrival order, while a slot, budget and pages are there
        size_t w = 0;
        while (w < wait.size() && budget > 0) {
            const Candidate r = wait[w];
            if (r.prompt_len == 0 || r.len > max_model_len) {
                if (!emit(TFFH_EVENT_FINISH, r.uid, r.prompt_len ? TFFH_REASON_TOO_LONG : TFFH_REASON_EMPTY_PROMPT, 0))
                    return c->fail(TFFH_ERR_TOO_SMALL, too_many);
                ++w;
                continue;
            }
            if (!fits_alone(r.len)) {
                if (!emit(TFFH_EVENT_FINISH, r.uid, TFFH_REASON_OUT_OF_MEMORY, 0)) return c->fail(TFFH_ERR_TOO_SMALL, too_many);
                ++w;
                continue;
            }
            if (c->slots.num_free() == 0) break;
            const int n = std::min(r.len, budget);
            const int blocks = (n + c->page_size - 1) / c->page_size;
            bool fits = true;
            for (int g = 0; g < G; ++g) fits = fits && blocks <= free_pages[g];
            if (!fits) break;
            const int slot = tffh_admit(cache, r.handle);
            if (slot < 0) return slot == -100 ? c->fail(TFFH_ERR_ACCOUNTING, "a free slot vanished") : slot;
            if (!emit(TFFH_EVENT_ADMIT, r.uid, slot, 0)) return c->fail(TFFH_ERR_TOO_SMALL, too_many);
            for (int g = 0; g < G; ++g) free_pages[g] -= blocks;
            budget -= n;
            run.push_back(r);
            chosen.emplace_back((int)run.size() - 1, n);
            ++w;
        }
        break;
    }
    for (const auto& ch : chosen) {
        const Candidate& r = run[ch.first];
        const int start = c->find(r.handle)->num_tokens;
        const int got = tffh_reserve(cache, r.handle, ch.second);
        if (got < 0) return got;
        if (got == 0) return c->fail(TFFH_ERR_ACCOUNTING, "pages were counted but could not be taken");
        if (!emit(TFFH_EVENT_RUN, r.uid, ch.second, start)) return c->fail(TFFH_ERR_TOO_SMALL, too_many);
    }
    return n_events;
}

// ------------------------------------------------------------------------------- a whole step at once
TFFH_API int tffh_reserve_step(void* cache, int n, const int64_t* reqs, const int* q_lens, int max_model_len,
                               int* detail) {
    Cache* c = as_cache(cache);
    const int G = (int)c->pools.size();
    std::vector<RequestCache*> rcs(n);
    std::vector<int> total(G, 0), need(G);
    for (int i = 0; i < n; ++i) {
        detail[0] = i;
        rcs[i] = c->find(reqs[i]);
        if (!rcs[i]) return c->fail(TFFH_ERR_UNKNOWN, "request " + std::to_string(reqs[i]) + " is not live");
        for (int j = 0; j < i; ++j)
            if (reqs[j] == reqs[i]) return c->fail(TFFH_ERR_DUPLICATE, "a request appears twice in one step");
        if (q_lens[i] <= 0) return c->fail(TFFH_ERR_ARGUMENT, "a request brings no tokens");
        if (max_model_len > 0 && rcs[i]->num_tokens + q_lens[i] > max_model_len)
            return c->fail(TFFH_ERR_TOO_LONG, "a request would exceed the maximum length");
        c->pages_needed(*rcs[i], q_lens[i], need.data());
        for (int g = 0; g < G; ++g) total[g] += need[g];
    }
    for (int g = 0; g < G; ++g)
        if (total[g] > c->pools[g].num_free()) {            // all or nothing over the whole step
            detail[0] = g; detail[1] = total[g]; detail[2] = c->pools[g].num_free();
            return 0;
        }
    for (int i = 0; i < n; ++i) {
        const int got = tffh_reserve(cache, reqs[i], q_lens[i]);
        if (got <= 0) return got < 0 ? got : c->fail(TFFH_ERR_ACCOUNTING, "pages were counted but could not be taken");
    }
    return 1;
}

TFFH_API int tffh_commit_step(void* cache, int n, const int64_t* reqs, const int* counts) {
    for (int i = 0; i < n; ++i) {
        const int st = tffh_commit(cache, reqs[i], counts[i]);
        if (st < 0) return st;
    }
    return 0;
}
