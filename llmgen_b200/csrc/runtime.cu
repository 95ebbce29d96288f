// The host side of the engine in C++: the cache manager (pages, block tables, groups of layers with
// different needs, slots of per-request state), the batch scheduler (both policies, preemption by
// recompute) and the filling of a decode step's metadata.  No device code lives here; the file is
// built like the kernel modules and bound through the same C ABI (`llmr_*`), the Python classes in
// `llmgen_b200/cache/manager.py` and `llmgen_b200/engine/scheduler.py` are thin shells over it.
//
// What the reference has, in Zig: `BlockManager` (src/runner/block.zig:5-80: one pool, a LIFO free
// stack that hands out 0, 1, 2, ... when fresh, ensure / canEnsure / deallocate), `Sequence` and
// `BatchScheduler` (src/runner/batching.zig:18-356: prefill_first and chunked, the last running
// sequence is preempted when pages run out and goes back to the front of the queue), and the
// executor's `fillMeta` (src/executor.zig:772-861).  Kept: those rules.  Added: groups (a window
// group gives pages back as the window passes them), state slots, all-or-nothing over groups.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#define LLMR_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

thread_local char g_error[512] = "";

enum { KIND_FULL = 0, KIND_WINDOW = 1 };
enum { ST_WAITING = 0, ST_RUNNING = 1, ST_FINISHED = 2 };
enum { POLICY_PREFILL_FIRST = 0, POLICY_CHUNKED = 1 };

// ------------------------------------------------------------------------------ page pool
struct Pool {
    int num_pages = 0;
    std::vector<int> free_;          // a stack; a fresh pool pops 0, 1, 2, ...
    std::vector<char> is_free;

    explicit Pool(int n) : num_pages(n), free_(n), is_free(n, 1) {
        for (int i = 0; i < n; ++i) free_[i] = n - 1 - i;
    }
    int num_free() const { return (int)free_.size(); }
    bool take(int n, std::vector<int>* out) {
        if (n > (int)free_.size()) return false;
        for (int i = 0; i < n; ++i) {
            const int p = free_.back();
            free_.pop_back();
            is_free[p] = 0;
            out->push_back(p);
        }
        return true;
    }
    // 0 ok, 1 page outside the pool, 2 page freed twice
    int give(const int* pages, int n) {
        for (int i = 0; i < n; ++i) {
            const int p = pages[i];
            if (p < 0 || p >= num_pages) {
                snprintf(g_error, sizeof(g_error), "page %d does not belong to this pool of %d", p, num_pages);
                return 1;
            }
            if (is_free[p]) {
                snprintf(g_error, sizeof(g_error), "page %d freed twice", p);
                return 2;
            }
            is_free[p] = 1;
            free_.push_back(p);
        }
        return 0;
    }
};

// ----------------------------------------------------------------------- one group of layers
struct Group {
    int kind, window, page_size;
    Pool pool;
    std::unordered_map<int64_t, std::vector<int>> tables;
    std::unordered_map<int64_t, int64_t> births;     // which table of the group's history a request's table is
    int64_t born = 0;

    Group(int kind_, int window_, int pages, int page_size_) : kind(kind_), window(window_), page_size(page_size_), pool(pages) {}

    int first_needed(int start) const { return kind == KIND_WINDOW ? std::max(0, start - window + 1) : 0; }

    // pages to give back (indices into the table), number of new pages, number of skipped indices
    void plan(int64_t req, int start, int end, std::vector<int>* give, int* fresh, int* skipped) const {
        static const std::vector<int> none;
        auto it = tables.find(req);
        const std::vector<int>& table = it == tables.end() ? none : it->second;
        const int first_live_page = first_needed(start) / page_size;
        const int upto = std::min(first_live_page, (int)table.size());
        for (int i = 0; i < upto; ++i)
            if (table[i] >= 0) give->push_back(i);
        const int need_pages = (end + page_size - 1) / page_size;
        const int more = std::max(0, need_pages - (int)table.size());
        // positions between the end of the table and the first live page need no real page
        *skipped = std::max(0, std::min(first_live_page, need_pages) - (int)table.size());
        *fresh = more - *skipped;
    }
    bool can_reserve(int64_t req, int start, int end) const {
        std::vector<int> give;
        int fresh, skipped;
        plan(req, start, end, &give, &fresh, &skipped);
        return fresh <= pool.num_free() + (int)give.size();
    }
    bool reserve(int64_t req, int start, int end) {
        std::vector<int> give;
        int fresh, skipped;
        plan(req, start, end, &give, &fresh, &skipped);
        if (fresh > pool.num_free() + (int)give.size()) return false;
        auto it = tables.find(req);
        if (it == tables.end()) {
            it = tables.emplace(req, std::vector<int>()).first;
            births[req] = ++born;
        }
        std::vector<int>& table = it->second;
        for (int i : give) {
            pool.give(&table[i], 1);
            table[i] = -1;
        }
        table.insert(table.end(), skipped, -1);
        pool.take(fresh, &table);
        return true;
    }
    void release(int64_t req) {
        auto it = tables.find(req);
        if (it != tables.end()) {
            const std::vector<int>& t = it->second;
            for (int i = (int)t.size() - 1; i >= 0; --i)
                if (t[i] >= 0) pool.give(&t[i], 1);
            tables.erase(it);
        }
        births.erase(req);
    }
    const std::vector<int>* table(int64_t req) const {
        auto it = tables.find(req);
        return it == tables.end() ? nullptr : &it->second;
    }
    // changes whenever the table's contents may have changed; -1: a window group (its pages go away too)
    int64_t stamp(int64_t req) const {
        if (kind == KIND_WINDOW) return -1;
        auto it = births.find(req);
        const std::vector<int>* t = table(req);
        return ((it == births.end() ? 0 : it->second) << 24) | (int64_t)(t ? t->size() : 0);
    }
};

// ------------------------------------------------------------------------------ state slots
struct Slots {
    int num_slots;
    std::vector<int> free_;
    std::unordered_map<int64_t, int> owner;
    explicit Slots(int n) : num_slots(n), free_(n) {
        for (int i = 0; i < n; ++i) free_[i] = n - 1 - i;
    }
    int take(int64_t req) {
        auto it = owner.find(req);
        if (it != owner.end()) return it->second;
        if (free_.empty()) return -1;
        const int s = free_.back();
        free_.pop_back();
        owner[req] = s;
        return s;
    }
    void give(int64_t req) {
        auto it = owner.find(req);
        if (it == owner.end()) return;
        free_.push_back(it->second);
        owner.erase(it);
    }
    int slot(int64_t req) const {
        auto it = owner.find(req);
        return it == owner.end() ? -1 : it->second;
    }
};

// ---------------------------------------------------------------------------- cache manager
struct Cache {
    int page_size;
    std::vector<Group*> groups;
    Slots slots;
    std::vector<int> fresh;          // slots handed out since the executor last looked

    Cache(int n_groups, const int* kinds, const int* windows, const int* pages, int page_size_, int n_slots)
        : page_size(page_size_), slots(n_slots) {
        for (int i = 0; i < n_groups; ++i) groups.push_back(new Group(kinds[i], windows[i], pages[i], page_size_));
    }
    ~Cache() {
        for (Group* g : groups) delete g;
    }
    int admit(int64_t req) {
        const bool known = slots.owner.count(req) != 0;
        const int s = slots.take(req);
        if (s >= 0 && !known) fresh.push_back(s);
        return s;
    }
    bool can_reserve(int64_t req, int start, int end) const {
        for (const Group* g : groups)
            if (!g->can_reserve(req, start, end)) return false;
        return true;
    }
    bool reserve(int64_t req, int start, int end) {
        if (!can_reserve(req, start, end)) return false;
        for (Group* g : groups) g->reserve(req, start, end);
        return true;
    }
    void release_pages(int64_t req) {
        for (Group* g : groups) g->release(req);
    }
    void release(int64_t req) {
        release_pages(req);
        slots.give(req);
    }
};

// -------------------------------------------------------------------------------- scheduler
struct Req {
    int64_t id;
    int length;          // prompt + generated tokens known so far
    int num_prompt;
    int computed;
    int max_tokens;
    bool ignore_eos;
    int status;
    int preemptions;
    int pending = 0;         // tokens of launched steps that the host has not read yet
    bool reported = false;   // its last token has been named
};

struct Item {
    int64_t req;
    int q_start, q_len;
};

struct Sched {
    Cache* cache;
    int policy, max_num_seqs, max_batched, chunk;
    std::vector<int> eos;
    std::deque<int64_t> waiting;
    std::vector<int64_t> running;
    std::unordered_map<int64_t, Req> reqs;
    int num_preemptions = 0;
    std::vector<int64_t> preempted_now;     // requests preempted by the last schedule()

    bool admit(Req& r, int upto) {
        if ((int)running.size() >= max_num_seqs) return false;
        if (cache->admit(r.id) < 0) return false;
        if (!cache->reserve(r.id, 0, upto)) {
            cache->release(r.id);
            return false;
        }
        return true;
    }
    void preempt(Req& r) {
        r.status = ST_WAITING;
        r.computed = 0;
        r.preemptions += 1;
        cache->release(r.id);
        waiting.push_front(r.id);
        num_preemptions += 1;
        preempted_now.push_back(r.id);
    }
    // Preempt from the tail of `running` until positions [start, upto) of running[index] can be
    // reserved; false if the sequence had to preempt itself.
    bool make_room(int index, int start, int upto) {
        const int64_t id = running[index];
        while (!cache->can_reserve(id, start, upto)) {
            if ((int)running.size() - 1 > index) {
                const int64_t last = running.back();
                running.pop_back();
                preempt(reqs[last]);
            } else {
                running.erase(running.begin() + index);
                preempt(reqs[id]);
                return false;
            }
        }
        return true;
    }
    // The request leaves the queues and gives back what it holds; its record stays until the tokens
    // it still expects have been read.
    void finish(Req& r) {
        r.status = ST_FINISHED;
        cache->release(r.id);
        auto pos = std::find(running.begin(), running.end(), r.id);
        if (pos != running.end()) running.erase(pos);
        auto wpos = std::find(waiting.begin(), waiting.end(), r.id);
        if (wpos != waiting.end()) waiting.erase(wpos);
    }
    void start_running(Req& r) {
        waiting.pop_front();
        r.status = ST_RUNNING;
        r.computed = 0;
        running.push_back(r.id);
    }
    void schedule_prefill_first(std::vector<Item>* out) {
        int tokens = 0;
        while (!waiting.empty() && (int)out->size() < max_num_seqs) {
            Req& r = reqs[waiting.front()];
            const int n = r.length;
            if (tokens + n > max_batched) break;
            if (!admit(r, n)) break;
            start_running(r);
            out->push_back({r.id, 0, n});
            tokens += n;
        }
        if (!out->empty()) return;
        int i = 0;
        while (i < (int)running.size() && (int)out->size() < max_num_seqs) {
            Req& r = reqs[running[i]];
            const int n = r.length;
            if (!make_room(i, n - 1, n)) break;
            cache->reserve(r.id, n - 1, n);
            out->push_back({r.id, n - 1, 1});
            ++i;
        }
    }
    void schedule_chunked(std::vector<Item>* out) {
        int budget = max_batched, prefill_budget = chunk;
        const int preemptions_before = num_preemptions;
        int i = 0;
        while (i < (int)running.size() && (int)out->size() < max_num_seqs && budget > 0) {
            Req& r = reqs[running[i]];
            const int remaining = r.length - r.computed;
            const bool in_prefill = remaining > 1;
            int q_len = std::min(remaining, budget);
            if (in_prefill) q_len = std::min(q_len, prefill_budget);
            if (q_len == 0) {
                ++i;
                continue;
            }
            const int start = r.computed;
            if (!make_room(i, start, start + q_len)) break;
            cache->reserve(r.id, start, start + q_len);
            out->push_back({r.id, start, q_len});
            budget -= q_len;
            if (in_prefill) prefill_budget -= q_len;
            ++i;
        }
        if (num_preemptions != preemptions_before) return;
        while (!waiting.empty() && (int)out->size() < max_num_seqs && budget > 0 && prefill_budget > 0) {
            Req& r = reqs[waiting.front()];
            const int q_len = std::min(r.length, std::min(budget, prefill_budget));
            if (!admit(r, q_len)) break;
            start_running(r);
            out->push_back({r.id, 0, q_len});
            budget -= q_len;
            prefill_budget -= q_len;
        }
    }
};

int copy_out(const std::vector<int>& v, int* out, int cap) {
    const int n = std::min((int)v.size(), cap);
    if (n > 0 && out) memcpy(out, v.data(), n * sizeof(int));
    return (int)v.size();
}

}  // namespace

LLMR_EXPORT const char* llmr_last_error() { return g_error; }
// also under the name every kernel module exports, so that the loader treats this module like the others
LLMR_EXPORT const char* llmk_last_error() { return g_error; }

// ------------------------------------------------------------------------ C ABI: page pool
LLMR_EXPORT void* llmr_pool_new(int n) { return n < 0 ? nullptr : new Pool(n); }
LLMR_EXPORT void llmr_pool_delete(void* p) { delete static_cast<Pool*>(p); }
LLMR_EXPORT int llmr_pool_num_free(void* p) { return static_cast<Pool*>(p)->num_free(); }
LLMR_EXPORT int llmr_pool_take(void* p, int n, int* out) {
    std::vector<int> got;
    if (!static_cast<Pool*>(p)->take(n, &got)) return 0;
    if (n > 0) memcpy(out, got.data(), n * sizeof(int));
    return 1;
}
LLMR_EXPORT int llmr_pool_give(void* p, const int* pages, int n) { return static_cast<Pool*>(p)->give(pages, n); }
LLMR_EXPORT int llmr_pool_free_list(void* p, int* out, int cap) { return copy_out(static_cast<Pool*>(p)->free_, out, cap); }

// --------------------------------------------------------------------------- C ABI: group
LLMR_EXPORT void* llmr_group_new(int kind, int window, int pages, int page_size) {
    if (pages < 0 || page_size <= 0 || (kind == KIND_WINDOW && window <= 0) || (kind != KIND_FULL && kind != KIND_WINDOW))
        return nullptr;
    return new Group(kind, window, pages, page_size);
}
LLMR_EXPORT void llmr_group_delete(void* g) { delete static_cast<Group*>(g); }
LLMR_EXPORT void* llmr_group_pool(void* g) { return &static_cast<Group*>(g)->pool; }
LLMR_EXPORT int llmr_group_can_reserve(void* g, long long req, int start, int end) {
    return static_cast<Group*>(g)->can_reserve(req, start, end) ? 1 : 0;
}
LLMR_EXPORT int llmr_group_reserve(void* g, long long req, int start, int end) {
    return static_cast<Group*>(g)->reserve(req, start, end) ? 1 : 0;
}
LLMR_EXPORT void llmr_group_release(void* g, long long req) { static_cast<Group*>(g)->release(req); }
// length of the table, -1 when the request has none; up to `cap` entries are copied
LLMR_EXPORT int llmr_group_table(void* g, long long req, int* out, int cap) {
    const std::vector<int>* t = static_cast<Group*>(g)->table(req);
    return t ? copy_out(*t, out, cap) : -1;
}
LLMR_EXPORT long long llmr_group_stamp(void* g, long long req) { return static_cast<Group*>(g)->stamp(req); }
LLMR_EXPORT int llmr_group_num_tables(void* g) { return (int)static_cast<Group*>(g)->tables.size(); }
LLMR_EXPORT int llmr_group_first_needed(void* g, int start) { return static_cast<Group*>(g)->first_needed(start); }
// 0 when no page is lost, held twice, or both held and free; otherwise a message is left
LLMR_EXPORT int llmr_group_check(void* gp, int index) {
    Group* g = static_cast<Group*>(gp);
    std::vector<char> seen(g->pool.num_pages, 0);
    int held = 0;
    for (const auto& kv : g->tables)
        for (int p : kv.second) {
            if (p < 0) continue;
            if (p >= g->pool.num_pages || seen[p]) {
                snprintf(g_error, sizeof(g_error), "group %d: a page is held twice", index);
                return 1;
            }
            seen[p] = 1;
            ++held;
        }
    std::vector<char> on_stack(g->pool.num_pages, 0);
    for (int p : g->pool.free_) {
        if (on_stack[p]) {
            snprintf(g_error, sizeof(g_error), "group %d: a page is on the free stack twice", index);
            return 2;
        }
        on_stack[p] = 1;
        if (seen[p]) {
            snprintf(g_error, sizeof(g_error), "group %d: a page is both held and free", index);
            return 3;
        }
    }
    if (held + (int)g->pool.free_.size() != g->pool.num_pages) {
        snprintf(g_error, sizeof(g_error), "group %d: %d page(s) lost", index, g->pool.num_pages - held - (int)g->pool.free_.size());
        return 4;
    }
    return 0;
}

// --------------------------------------------------------------------------- C ABI: slots
LLMR_EXPORT void* llmr_slots_new(int n) { return n < 0 ? nullptr : new Slots(n); }
LLMR_EXPORT void llmr_slots_delete(void* s) { delete static_cast<Slots*>(s); }
LLMR_EXPORT int llmr_slots_take(void* s, long long req) { return static_cast<Slots*>(s)->take(req); }
LLMR_EXPORT void llmr_slots_give(void* s, long long req) { static_cast<Slots*>(s)->give(req); }
LLMR_EXPORT int llmr_slots_slot(void* s, long long req) { return static_cast<Slots*>(s)->slot(req); }
LLMR_EXPORT int llmr_slots_num_free(void* s) { return (int)static_cast<Slots*>(s)->free_.size(); }

// --------------------------------------------------------------------------- C ABI: cache
LLMR_EXPORT void* llmr_cache_new(int n_groups, const int* kinds, const int* windows, const int* pages, int page_size,
                                 int n_slots) {
    if (page_size <= 0 || n_slots < 0) return nullptr;
    for (int i = 0; i < n_groups; ++i)
        if (pages[i] < 0 || (kinds[i] == KIND_WINDOW && windows[i] <= 0)) return nullptr;
    return new Cache(n_groups, kinds, windows, pages, page_size, n_slots);
}
LLMR_EXPORT void llmr_cache_delete(void* c) { delete static_cast<Cache*>(c); }
LLMR_EXPORT void* llmr_cache_group(void* c, int i) { return static_cast<Cache*>(c)->groups[i]; }
LLMR_EXPORT void* llmr_cache_slots(void* c) { return &static_cast<Cache*>(c)->slots; }
LLMR_EXPORT int llmr_cache_admit(void* c, long long req) { return static_cast<Cache*>(c)->admit(req); }
LLMR_EXPORT int llmr_cache_can_reserve(void* c, long long req, int start, int end) {
    return static_cast<Cache*>(c)->can_reserve(req, start, end) ? 1 : 0;
}
LLMR_EXPORT int llmr_cache_reserve(void* c, long long req, int start, int end) {
    return static_cast<Cache*>(c)->reserve(req, start, end) ? 1 : 0;
}
LLMR_EXPORT void llmr_cache_release(void* c, long long req) { static_cast<Cache*>(c)->release(req); }
LLMR_EXPORT void llmr_cache_release_pages(void* c, long long req) { static_cast<Cache*>(c)->release_pages(req); }
// Can a step compute positions [start, start + n) of `req`?  0 yes; 1 it holds no state slot (was not
// admitted); 2 a page that those positions write or still read is missing in some group.
LLMR_EXPORT int llmr_cache_check_step(void* c, long long req, int start, int n) {
    Cache* cache = static_cast<Cache*>(c);
    if (cache->slots.slot(req) < 0) return 1;
    const int ps = cache->page_size;
    for (Group* g : cache->groups) {
        const std::vector<int>* t = g->table(req);
        const int last_page = (start + n - 1) / ps;
        const int first_live = g->first_needed(start) / ps;
        if (!t || last_page >= (int)t->size()) return 2;
        for (int i = first_live; i <= last_page; ++i)
            if ((*t)[i] < 0) return 2;
    }
    return 0;
}
// slots handed out since the last call with clear != 0
LLMR_EXPORT int llmr_cache_fresh(void* c, int* out, int cap, int clear) {
    Cache* cache = static_cast<Cache*>(c);
    const int n = copy_out(cache->fresh, out, cap);
    if (clear) cache->fresh.clear();
    return n;
}

// ----------------------------------------------------------------------- C ABI: scheduler
LLMR_EXPORT void* llmr_sched_new(void* cache, int policy, int max_num_seqs, int max_batched, int chunk, const int* eos,
                                 int n_eos) {
    if (!cache || (policy != POLICY_PREFILL_FIRST && policy != POLICY_CHUNKED)) return nullptr;
    Sched* s = new Sched();
    s->cache = static_cast<Cache*>(cache);
    s->policy = policy;
    s->max_num_seqs = max_num_seqs;
    s->max_batched = max_batched;
    s->chunk = chunk;
    s->eos.assign(eos, eos + n_eos);
    return s;
}
LLMR_EXPORT void llmr_sched_delete(void* s) { delete static_cast<Sched*>(s); }
LLMR_EXPORT void llmr_sched_set_eos(void* s, const int* eos, int n_eos) { static_cast<Sched*>(s)->eos.assign(eos, eos + n_eos); }
LLMR_EXPORT void llmr_sched_add(void* sp, long long req, int prompt_len, int max_tokens, int ignore_eos) {
    Sched* s = static_cast<Sched*>(sp);
    s->reqs[req] = Req{req, prompt_len, prompt_len, 0, max_tokens, ignore_eos != 0, ST_WAITING, 0, 0, false};
    s->waiting.push_back(req);
}
LLMR_EXPORT int llmr_sched_is_finished(void* sp) {
    Sched* s = static_cast<Sched*>(sp);
    return (s->waiting.empty() && s->running.empty()) ? 1 : 0;
}
// One step's portions: (request, first position, length) triples; returns how many (at most `cap`
// are written).  `preempted` receives the requests that lost their place in this call.
// `emits[i]` is 1 when portion i reaches the last known token of its sequence, so that the step
// yields a new token for it.
LLMR_EXPORT int llmr_sched_schedule(void* sp, long long* reqs, int* q_start, int* q_len, int* emits, int cap,
                                    long long* preempted, int preempted_cap, int* n_preempted) {
    Sched* s = static_cast<Sched*>(sp);
    s->preempted_now.clear();
    std::vector<Item> out;
    if (s->policy == POLICY_PREFILL_FIRST) s->schedule_prefill_first(&out);
    else s->schedule_chunked(&out);
    const int n = std::min((int)out.size(), cap);
    for (int i = 0; i < n; ++i) {
        reqs[i] = out[i].req;
        q_start[i] = out[i].q_start;
        q_len[i] = out[i].q_len;
        emits[i] = out[i].q_start + out[i].q_len == s->reqs[out[i].req].length ? 1 : 0;
    }
    const int np = std::min((int)s->preempted_now.size(), preempted_cap);
    for (int i = 0; i < np; ++i) preempted[i] = s->preempted_now[i];
    *n_preempted = (int)s->preempted_now.size();
    return (int)out.size();
}
// After a step has been launched, what does not depend on the tokens it will sample: the portions
// count as computed, a sequence whose portion reached its end grows by one token (one more token
// of it is now pending), and a request that has its max_tokens with it leaves the queues and gives
// back what it holds.  The step may still be running: pages given back here are written again only
// by steps launched later on the same stream.  Returns how many requests left the queues.
LLMR_EXPORT int llmr_sched_advance(void* sp, int n, const long long* reqs, const int* q_start, const int* q_len) {
    Sched* s = static_cast<Sched*>(sp);
    int done = 0;
    for (int i = 0; i < n; ++i) {
        auto it = s->reqs.find(reqs[i]);
        if (it == s->reqs.end()) continue;
        Req& r = it->second;
        if (r.status == ST_FINISHED) continue;
        const bool emits = q_start[i] + q_len[i] == r.length;
        r.computed = q_start[i] + q_len[i];
        if (!emits) continue;
        r.length += 1;
        r.pending += 1;
        if (r.length - r.num_prompt >= r.max_tokens) {
            s->finish(r);
            ++done;
        }
    }
    return done;
}
// When the tokens of a step are known: `reqs[i]`, `tokens[i]` for every portion that yielded one, in
// the order of the step.  `last[i]` becomes 1 when that token is the request's last one: it ends the
// sequence (and the request does not ignore that), or it is the token that filled max_tokens.  A
// request that ended is released wherever it is (running, or waiting after a preemption); tokens
// that a later step, launched before this one was read, sampled for it are to be dropped
// (`last[i]` = -1 for those).  Returns how many requests ended here.
LLMR_EXPORT int llmr_sched_resolve(void* sp, int n, const long long* reqs, const int* tokens, int* last) {
    Sched* s = static_cast<Sched*>(sp);
    int done = 0;
    for (int i = 0; i < n; ++i) {
        last[i] = -1;
        auto it = s->reqs.find(reqs[i]);
        if (it == s->reqs.end()) continue;
        Req& r = it->second;
        r.pending -= 1;
        if (!r.reported) {
            last[i] = 0;
            const bool hit_eos = !r.ignore_eos && std::find(s->eos.begin(), s->eos.end(), tokens[i]) != s->eos.end();
            if (hit_eos || (r.status == ST_FINISHED && r.pending == 0)) {
                if (r.status != ST_FINISHED) s->finish(r);
                r.reported = true;
                last[i] = 1;
                ++done;
            }
        }
        if (r.reported && r.pending <= 0) s->reqs.erase(it);
    }
    return done;
}
LLMR_EXPORT int llmr_sched_num_preemptions(void* sp) { return static_cast<Sched*>(sp)->num_preemptions; }
LLMR_EXPORT int llmr_sched_queue(void* sp, int which, long long* out, int cap) {
    Sched* s = static_cast<Sched*>(sp);
    int n = 0;
    if (which == 0) {
        for (int64_t id : s->waiting) {
            if (n < cap) out[n] = id;
            ++n;
        }
    } else {
        for (int64_t id : s->running) {
            if (n < cap) out[n] = id;
            ++n;
        }
    }
    return n;
}
// (status, computed, preemptions, length) of a request the scheduler still knows; 0 if it does not
LLMR_EXPORT int llmr_sched_request(void* sp, long long req, int* out4) {
    Sched* s = static_cast<Sched*>(sp);
    auto it = s->reqs.find(req);
    if (it == s->reqs.end()) return 0;
    out4[0] = it->second.status;
    out4[1] = it->second.computed;
    out4[2] = it->second.preemptions;
    out4[3] = it->second.length;
    return 1;
}

// ------------------------------------------------------- C ABI: a decode step's metadata
// Rewrites, in a pinned host buffer that the same batch-size bucket filled last, what a step of
// single tokens changes: ids, positions, lengths, state slots, temperatures, and per group the slots
// and the block-table rows whose table changed (`row_stamps[g * bucket + s]` remembers request and
// stamp of what row s of group g holds; 0 = padding).  Offsets are in 4-byte words:
// offs = [ids, positions, ctx_len, state_slots, temps, ids_from, row_keys, then (slots_g, block_tables_g) per group].
// row_keys (two words a row) is the sampler's key of the row: (seed_base + stride * (position + 1)) ^ (request << 40),
// the reference's step_seed ^ (row << 40) (src/backend/cpu/sample.zig:28) with the position in the step's place
// and the request in the row's, so that a draw depends on neither the batch nor the number of steps so far.
// `from[s]` >= 0 names the row of the step before whose sampled token is row s's id (the host has
// not read it yet; tokens[s] is then ignored), -1 takes tokens[s].
// Returns 0, or 1 when a position has no page.
LLMR_EXPORT int llmr_fill_decode(void* c, int* host, const int* offs, int n, int bucket, int max_blocks,
                                 const long long* reqs, const int* tokens, const int* from, const int* starts,
                                 const float* temps, unsigned long long seed_base, long long* row_stamps) {
    Cache* cache = static_cast<Cache*>(c);
    const int ps = cache->page_size;
    int* ids = host + offs[0];
    int* pos = host + offs[1];
    int* ctx = host + offs[2];
    int* st = host + offs[3];
    float* tp = reinterpret_cast<float*>(host + offs[4]);
    int* fr = host + offs[5];
    int* keys = host + offs[6];
    for (int s = 0; s < bucket; ++s) {
        const bool live = s < n;
        const unsigned long long key =
            live ? (seed_base + 0x9E3779B97F4A7C15ull * (unsigned long long)(starts[s] + 1)) ^ ((unsigned long long)reqs[s] << 40) : 0ull;
        memcpy(keys + 2 * s, &key, sizeof(key));
        ids[s] = live && from[s] < 0 ? tokens[s] : 0;
        fr[s] = live ? from[s] : -1;
        pos[s] = live ? starts[s] : 0;
        ctx[s] = live ? starts[s] + 1 : 0;
        st[s] = live ? cache->slots.slot(reqs[s]) : -1;
        tp[s] = live ? temps[s] : 0.f;
    }
    const int n_groups = (int)cache->groups.size();
    for (int g = 0; g < n_groups; ++g) {
        Group* grp = cache->groups[g];
        int* slots = host + offs[7 + 2 * g];
        int* bt = host + offs[8 + 2 * g];
        long long* stamps = row_stamps + (size_t)g * bucket * 2;
        for (int s = 0; s < bucket; ++s) {
            int* row = bt + (size_t)s * max_blocks;
            if (s >= n) {
                slots[s] = -1;
                if (stamps[2 * s] != 0 || stamps[2 * s + 1] != 0) {
                    memset(row, 0, max_blocks * sizeof(int));
                    stamps[2 * s] = stamps[2 * s + 1] = 0;
                }
                continue;
            }
            const std::vector<int>* t = grp->table(reqs[s]);
            const int p = starts[s];
            if (!t || p / ps >= (int)t->size() || (*t)[p / ps] < 0) {
                snprintf(g_error, sizeof(g_error), "request %lld: no page reserved for position %d", reqs[s], p);
                return 1;
            }
            const long long stamp = grp->stamp(reqs[s]);
            // a row is rewritten unless it holds this very table at this very length (full-attention groups)
            if (stamp < 0 || stamps[2 * s] != reqs[s] + 1 || stamps[2 * s + 1] != stamp) {
                const int len = std::min((int)t->size(), max_blocks);
                memcpy(row, t->data(), len * sizeof(int));
                if (len < max_blocks) memset(row + len, 0, (max_blocks - len) * sizeof(int));
                stamps[2 * s] = reqs[s] + 1;
                stamps[2 * s + 1] = stamp;
            }
            slots[s] = (*t)[p / ps] * ps + p % ps;
        }
    }
    return 0;
}
