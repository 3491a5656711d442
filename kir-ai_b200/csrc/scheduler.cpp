// The scheduler's decisions in native code: which requests run which tokens in the next step.
// Same rules as engine/scheduler.py (which remains as the readable model and is checked against this in the
// tests): every step (1) each running request that is decoding gets its one token, evicting the most recently
// admitted other running request when its next page is missing; (2) what is left of the token budget goes to
// prompt portions of running requests, shrunk to the pages that are free; (3) waiting requests are admitted in
// arrival order while a state slot is free and the running set is below its limit (and no running request found
// the pages short in (2)); (4) if nothing at all could run, the most recently admitted running request is evicted
// until the oldest can go on.  An evicted request gives its
// pages and slot back and goes to the front of the waiting queue to be recomputed.  The reference keeps its policy
// in native code as well: the generation loop that never runs the last sampled token
// (crates/llm-native-runtime/src/native_text/driver.rs:439-477), admission by a concurrency limit
// (crates/llm-server/src/engine/scheduler.rs:642-668), eviction of the least recently used session
// (crates/llm-kv-cache/src/block_pool.rs:811-838).
//
// The scheduler knows requests by a key and by counts only (prompt length, generated tokens, tokens in the cache);
// token values, sampling options and stop conditions stay with the caller, which says in update() which requests
// finished.  It works on the page tables of page_tables.cpp through their C interface.
//
// C interface: functions return >= 0 on success; -2 unknown request, -6 bad argument, -7 no progress possible
// (no request fits the free pages), -8 the output arrays are too small (nothing has been decided then).
#include <algorithm>
#include <cstdint>
#include <deque>
#include <unordered_map>
#include <unordered_set>
#include <vector>

extern "C" {
int kirai_pages_open(void* handle, long key);
int kirai_pages_can_reserve(void* handle, long key, long new_tokens);
int kirai_pages_reserve(void* handle, long key, long new_tokens);
int kirai_pages_close(void* handle, long key);
long kirai_pages_length(void* handle, long key);
int kirai_pages_table(void* handle, long key, int group, int* out, int capacity);
int kirai_pages_stat(void* handle, int group, int what);
}

namespace {

enum State { WAITING = 0, RUNNING = 1, FINISHED = 2 };

struct Entry {
    long prompt_len = 0, output_len = 0, computed = 0;
    int state = WAITING;
    int slot = -1;  // while it holds pages
    long preemptions = 0;
    long pending() const { return prompt_len + output_len - computed; }
};

struct Scheduler {
    void* pages = nullptr;
    int groups = 0, page_size = 1;
    long max_batched_tokens = 1, max_running = 1, prefill_chunk = -1;
    std::deque<long> waiting;
    std::vector<long> running;  // in admission order
    std::unordered_map<long, Entry> entries;
    long steps = 0, preemptions = 0, scheduled_tokens = 0, finished = 0;
};

long portion(const Scheduler& s, const Entry& e, long budget) {
    long count = std::min(e.pending(), budget);
    if (s.prefill_chunk > 0 && e.pending() > 1) count = std::min(count, s.prefill_chunk);
    return count;
}

// The largest portion <= count whose pages are free (whole pages beyond what the request holds).
long fit_to_pages(const Scheduler& s, long key, long count) {
    if (kirai_pages_can_reserve(s.pages, key, count) == 1) return count;
    long free_pages = 0, held_pages = 0;
    for (int g = 0; g < s.groups; ++g) {
        const long f = kirai_pages_stat(s.pages, g, 1), h = kirai_pages_table(s.pages, key, g, nullptr, 0);
        free_pages = g == 0 ? f : std::min(free_pages, f);
        held_pages = g == 0 ? h : std::min(held_pages, h);
    }
    long room = held_pages * s.page_size - kirai_pages_length(s.pages, key) + free_pages * s.page_size;
    room = std::min(room, count);
    while (room > 0 && kirai_pages_can_reserve(s.pages, key, room) != 1) --room;
    return std::max(room, 0L);
}

void preempt(Scheduler& s, long key, std::vector<long>& preempted) {
    Entry& e = s.entries[key];
    kirai_pages_close(s.pages, key);
    e.slot = -1;
    e.computed = 0;
    e.state = WAITING;
    ++e.preemptions;
    s.running.erase(std::find(s.running.begin(), s.running.end(), key));
    s.waiting.push_front(key);
    ++s.preemptions;
    preempted.push_back(key);
}

void finish(Scheduler& s, long key) {
    Entry& e = s.entries[key];
    if (e.slot >= 0) {
        kirai_pages_close(s.pages, key);
        e.slot = -1;
    }
    e.state = FINISHED;
    auto it = std::find(s.running.begin(), s.running.end(), key);
    if (it != s.running.end()) s.running.erase(it);
    ++s.finished;
}

}  // namespace

#define KIRAI_HOST_EXPORT extern "C" __attribute__((visibility("default")))

KIRAI_HOST_EXPORT void* kirai_sched_create(void* pages, int groups, int page_size, long max_batched_tokens, long max_running,
                                           long prefill_chunk) {
    if (!pages || groups < 0 || page_size <= 0 || max_batched_tokens < 1 || max_running < 1) return nullptr;
    Scheduler* s = new Scheduler();
    s->pages = pages, s->groups = groups, s->page_size = page_size;
    s->max_batched_tokens = max_batched_tokens, s->max_running = max_running, s->prefill_chunk = prefill_chunk;
    return s;
}
KIRAI_HOST_EXPORT void kirai_sched_destroy(void* handle) { delete static_cast<Scheduler*>(handle); }

// A new request joins the end of the waiting queue (the caller has checked that it can ever run).
KIRAI_HOST_EXPORT int kirai_sched_add(void* handle, long key, long prompt_len) {
    Scheduler& s = *static_cast<Scheduler*>(handle);
    if (prompt_len < 1 || s.entries.count(key)) return -6;
    Entry e;
    e.prompt_len = prompt_len;
    s.entries.emplace(key, e);
    s.waiting.push_back(key);
    return 0;
}

// Chooses the next step's runs and reserves their pages.  Outputs: the chosen runs (key, first token index, count,
// whether the run reaches the end of the request's tokens), the requests evicted on the way (in order) and the
// requests admitted (key and state slot, in order).  Returns the number of runs.
KIRAI_HOST_EXPORT int kirai_sched_schedule(void* handle, long* keys, long* first, long* count, int* sample, int capacity,
                                           long* preempted_keys, int* num_preempted, long* admitted_keys,
                                           int* admitted_slots, int* num_admitted) {
    Scheduler& s = *static_cast<Scheduler*>(handle);
    // every request may be chosen, evicted or admitted once: arrays that could not hold them all are refused before
    // anything is reserved or evicted
    if (capacity < 0 || (size_t)capacity < s.running.size() + s.waiting.size()) return -8;
    long budget = s.max_batched_tokens;
    int chosen = 0;
    std::vector<long> preempted, admitted;
    std::unordered_set<long> taken;
    auto choose = [&](long key, long first_token, long tokens, bool samples) {
        if (chosen >= capacity) return false;
        keys[chosen] = key, first[chosen] = first_token, count[chosen] = tokens, sample[chosen] = samples ? 1 : 0;
        ++chosen;
        taken.insert(key);
        budget -= tokens;
        return true;
    };
    // (1) decoding requests, oldest first; evict the youngest others when a page is missing
    const std::vector<long> snapshot = s.running;
    for (long key : snapshot) {
        Entry& e = s.entries[key];
        if (e.state != RUNNING || e.pending() != 1 || budget < 1) continue;
        bool reserved = false;
        while (true) {
            if (kirai_pages_reserve(s.pages, key, 1) == 1) {
                reserved = true;
                break;
            }
            long victim = -1;
            for (auto it = s.running.rbegin(); it != s.running.rend(); ++it)
                if (*it != key && !taken.count(*it)) {
                    victim = *it;
                    break;
                }
            if (victim < 0) break;  // nothing left to evict: the request waits for pages
            preempt(s, victim, preempted);
        }
        if (reserved && !choose(key, e.computed, 1, true)) return -8;
    }
    // (2) prompt portions of running requests; starved: one of them found no page for even one token
    bool starved = false;
    int failure = 0;
    auto prompt_portions = [&]() {
        starved = false;
        for (long key : s.running) {
            Entry& e = s.entries[key];
            if (taken.count(key) || budget < 1 || e.pending() < 1) continue;
            const long tokens = fit_to_pages(s, key, portion(s, e, budget));
            if (tokens < 1) {
                starved = true;
                continue;
            }
            if (kirai_pages_reserve(s.pages, key, tokens) != 1) { failure = -6; return; }
            if (!choose(key, e.computed, tokens, tokens == e.pending())) { failure = -8; return; }
        }
    };
    prompt_portions();
    if (failure) return failure;
    // (3) admit waiting requests in order, unless a running request already found no page for its prompt
    while (!starved && !s.waiting.empty() && budget >= 1 && (long)s.running.size() < s.max_running) {
        const long key = s.waiting.front();
        Entry& e = s.entries[key];
        const int slot = kirai_pages_open(s.pages, key);
        if (slot < 0) break;  // no state slot
        const long tokens = fit_to_pages(s, key, portion(s, e, budget));
        if (tokens < 1) {
            kirai_pages_close(s.pages, key);
            break;
        }
        if (kirai_pages_reserve(s.pages, key, tokens) != 1) return -6;
        s.waiting.pop_front();
        e.state = RUNNING;
        e.slot = slot;
        s.running.push_back(key);
        admitted.push_back(key);
        if (!choose(key, 0, tokens, tokens == e.pending())) return -8;
    }
    // (4) nothing could run: every running request is in mid-prompt and the pages are all held (a decoding request
    // would have evicted the others in (1)).  The youngest gives its pages to the others until the oldest can go on.
    while (chosen == 0 && s.running.size() > 1) {
        preempt(s, s.running.back(), preempted);  // not admitted in this step: an admitted request was chosen
        prompt_portions();
        if (failure) return failure;
    }
    if (chosen == 0 && (!s.waiting.empty() || !s.running.empty())) return -7;
    if ((int)preempted.size() > capacity || (int)admitted.size() > capacity) return -8;
    for (size_t i = 0; i < preempted.size(); ++i) preempted_keys[i] = preempted[i];
    for (size_t i = 0; i < admitted.size(); ++i) admitted_keys[i] = admitted[i], admitted_slots[i] = s.entries[admitted[i]].slot;
    *num_preempted = (int)preempted.size();
    *num_admitted = (int)admitted.size();
    ++s.steps;
    for (int i = 0; i < chosen; ++i) s.scheduled_tokens += count[i];
    return chosen;
}

// Records what a step did: per run the tokens it put into the cache, whether it sampled a token, and whether the
// caller found the request finished by that token (its pages and slot are freed at once).
KIRAI_HOST_EXPORT int kirai_sched_update(void* handle, const long* keys, const long* count, const int* sampled,
                                         const int* finished, int runs) {
    Scheduler& s = *static_cast<Scheduler*>(handle);
    for (int i = 0; i < runs; ++i) {
        auto it = s.entries.find(keys[i]);
        if (it == s.entries.end()) return -2;
        Entry& e = it->second;
        e.computed += count[i];
        if (!sampled[i]) continue;
        ++e.output_len;
        if (finished[i]) finish(s, keys[i]);
    }
    return 0;
}

// Ends a request between steps; what it holds is given back.
KIRAI_HOST_EXPORT int kirai_sched_abort(void* handle, long key) {
    Scheduler& s = *static_cast<Scheduler*>(handle);
    auto it = s.entries.find(key);
    if (it == s.entries.end()) return -2;
    if (it->second.state == FINISHED) return 0;
    auto waiting = std::find(s.waiting.begin(), s.waiting.end(), key);
    if (waiting != s.waiting.end()) s.waiting.erase(waiting);
    finish(s, key);
    return 0;
}

// Forgets a finished request (its key may then be used again).
KIRAI_HOST_EXPORT int kirai_sched_forget(void* handle, long key) {
    Scheduler& s = *static_cast<Scheduler*>(handle);
    auto it = s.entries.find(key);
    if (it == s.entries.end()) return -2;
    if (it->second.state != FINISHED) return -6;
    s.entries.erase(it);
    return 0;
}

// what: 0 steps, 1 preemptions, 2 scheduled tokens, 3 finished, 4 waiting now, 5 running now.
KIRAI_HOST_EXPORT long kirai_sched_stat(void* handle, int what) {
    const Scheduler& s = *static_cast<Scheduler*>(handle);
    switch (what) {
        case 0: return s.steps;
        case 1: return s.preemptions;
        case 2: return s.scheduled_tokens;
        case 3: return s.finished;
        case 4: return (long)s.waiting.size();
        case 5: return (long)s.running.size();
    }
    return -6;
}
