// The scheduler's decisions in C++: whether a request may be submitted and admitted, what a step
// holds, how long a prompt portion may be, and whether a request ends after a token.  The
// functions are pure: the Python class in engine/scheduler.py keeps the request objects and the
// queues and hands their numbers over; nothing here allocates beyond a call's own scratch.
//
// The rules and where the reference has them:
//  * refusals at submission: a prompt that leaves no room for one output token, a full queue;
//    the output limit is clamped to what the cache has left after the prompt
//    (crates/mrun/src/runtime/generate.rs:522-532, 600-636; crates/mrun/src/runtime/queue.rs:80-91);
//  * admission: a free place among the running requests, a free state slot and, with
//    reservations, pages for prompt + clamped output beside what is reserved already
//    (crates/mrun/src/runtime/handle.rs:497-559); side requests first, then the next member's
//    turn (crates/mrun/src/runtime/handle.rs:563-587);
//  * a step: one token of every request that has finished its prompt, then prompt portions while
//    the token budget lasts, fewest tokens left first, ties by admission order
//    (crates/mrun/src/runtime/lanes.rs:187-196); a portion is at most chunk_len(depth)
//    (crates/mrun-engine/src/engine.rs:481-486);
//  * ends: an end token, the output limit, or the last 512 output tokens repeating with a period
//    of at most 256, looked at every 16 tokens (crates/mrun/src/runtime/generate.rs:27-33, 420-426, 866-919);
//  * stop sequences of token ids: the output ends where one of them is complete, without it
//    (crates/mrun/src/chat/stop.rs:24-85).
#include <algorithm>
#include <cstdint>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int LOOP_WINDOW = 512, LOOP_MAX_PERIOD = 256, LOOP_CHECK_EVERY = 16;

inline int64_t blocks_for(int64_t tokens, int page_size) { return (tokens + page_size - 1) / page_size; }

}  // namespace

// Longest prompt portion at `depth` tokens already in the cache: the whole budget up to 16,384
// tokens of depth, then shrinking with the depth, never below 128 (or the budget, if smaller).
HOST_API int mrun_sched_chunk_len(int64_t depth, int budget) {
    const int64_t scaled = (int64_t)budget * 16384 / std::max<int64_t>(depth, 1);
    return (int)std::max<int64_t>(std::min(128, budget), std::min<int64_t>(budget, scaled));
}

// 1 if the last LOOP_WINDOW of the n tokens repeat with some period of 1 .. LOOP_MAX_PERIOD.
HOST_API int mrun_sched_looping(const int* tokens, int64_t n) {
    if (n < LOOP_WINDOW) return 0;
    const int* window = tokens + (n - LOOP_WINDOW);
    for (int period = 1; period <= LOOP_MAX_PERIOD; ++period) {
        bool repeats = true;
        for (int i = period; i < LOOP_WINDOW; ++i)
            if (window[i] != window[i - period]) {
                repeats = false;
                break;
            }
        if (repeats) return 1;
    }
    return 0;
}

// How many output tokens lie between two looks at the loop guard.
HOST_API int mrun_sched_loop_check_every() { return LOOP_CHECK_EVERY; }

// Refusal of a request whose prompt and sampling settings are valid: 0 none, 1 too long (the
// prompt leaves no room for one output token), 2 the queue is full (max_queue < 0: no bound).
// *limit gets the output limit clamped to the room the cache has after the prompt.
HOST_API int mrun_sched_submit_check(int64_t prompt_len, int64_t max_tokens, int64_t capacity_tokens, int64_t waiting,
                                     int64_t max_queue, int64_t* limit) {
    const int64_t room = capacity_tokens - prompt_len;
    *limit = 0;
    if (room < 1) return 1;
    *limit = std::min(max_tokens, room);
    if (max_queue >= 0 && waiting >= max_queue) return 2;
    return 0;
}

// Whether the request at the head of the queue starts now.  With reservations: its prompt plus its
// output limit (need_tokens) fit, in pages, beside what the running requests have reserved.
// On demand: the pages free now, less what the n running requests (sequence_len[i] tokens in all,
// fed[i] of them in the cache) still have to bring in, hold its sequence and one page more; a
// request that would run alone always starts.
HOST_API int mrun_sched_can_admit(int running, int max_running, int free_slots, int reserve, int64_t reserved_pages,
                                  int64_t num_pages, int page_size, int64_t free_pages, int64_t need_tokens,
                                  int64_t own_sequence_len, int n, const int64_t* sequence_len, const int64_t* fed) {
    if (running >= max_running || free_slots < 1) return 0;
    if (reserve) return reserved_pages + blocks_for(need_tokens, page_size) <= num_pages ? 1 : 0;
    if (running == 0) return 1;
    int64_t outstanding = 0;
    for (int i = 0; i < n; ++i) outstanding += blocks_for(sequence_len[i], page_size) - blocks_for(fed[i], page_size);
    return free_pages - outstanding >= blocks_for(own_sequence_len, page_size) + 1 ? 1 : 0;
}

// The step over the n running requests, given in the order they were admitted to the running
// list.  Request i has sequence_len[i] tokens (prompt + output read so far), fed[i] of them in
// the cache, inflight[i] tokens sampled on the device but not read yet, output_len[i] tokens of
// output read, the output limit limit[i], retiring[i] != 0 when it has ended already, and
// admission order order[i].  Entry e of the step: request entry_request[e] feeds entry_tokens[e]
// tokens, entry_wants[e] != 0 if the logits of the last one are wanted, entry_from_device[e] != 0
// if its one token is still on the device.  The arrays hold n entries.  Returns the entries made.
HOST_API int mrun_sched_plan(int n, const int64_t* sequence_len, const int64_t* fed, const int* inflight,
                             const int64_t* output_len, const int64_t* limit, const int* retiring,
                             const int64_t* order, int max_batch_tokens, int* entry_request, int* entry_tokens,
                             int* entry_wants, int* entry_from_device) {
    int64_t budget = max_batch_tokens;
    int made = 0;
    std::vector<int> readers;
    readers.reserve((size_t)n);
    // a request whose unread token will be its last, or that ended while a step was in flight,
    // takes no part any more
    for (int i = 0; i < n; ++i) {
        if (retiring[i] || output_len[i] + inflight[i] >= limit[i]) continue;
        const int64_t remaining = sequence_len[i] + inflight[i] - fed[i];
        const bool decoding = remaining == 1 && fed[i] > 0;
        if (decoding) {
            if (made < max_batch_tokens) {
                entry_request[made] = i;
                entry_tokens[made] = 1;
                entry_wants[made] = 1;
                entry_from_device[made] = inflight[i] ? 1 : 0;
                ++made;
            }
        } else if (!inflight[i]) {
            readers.push_back(i);
        }
    }
    budget -= made;
    std::stable_sort(readers.begin(), readers.end(), [&](int a, int b) {
        const int64_t ra = sequence_len[a] - fed[a], rb = sequence_len[b] - fed[b];
        return ra != rb ? ra < rb : order[a] < order[b];
    });
    for (int i : readers) {
        if (budget < 1) break;
        const int64_t remaining = sequence_len[i] - fed[i];
        const int64_t take = std::min<int64_t>({remaining, budget, (int64_t)mrun_sched_chunk_len(fed[i], max_batch_tokens)});
        entry_request[made] = i;
        entry_tokens[made] = (int)take;
        entry_wants[made] = take == remaining ? 1 : 0;
        entry_from_device[made] = 0;
        ++made;
        budget -= take;
    }
    return made;
}

// Why a request ends at a sampled token: 0 it goes on, 1 an end token (the token is not part of
// the output: output_len is the output's length without it), 2 the output limit, 3 repetition
// (output_len counts the token).  The loop guard is off with ignore_eos: runs of a forced length
// go to their limit on purpose (crates/mrun/src/runtime/generate.rs:908-913).  `recent` holds the last recent_len tokens of
// the output (the loop guard wants the last 512); it is looked at only when output_len is a
// multiple of the loop guard's interval and may be null otherwise.
HOST_API int mrun_sched_end_reason(int is_end_token, int ignore_eos, int64_t output_len, int64_t limit,
                                   const int* recent, int64_t recent_len) {
    if (is_end_token && !ignore_eos) return 1;
    if (output_len >= limit) return 2;
    if (!ignore_eos && recent != nullptr && output_len % LOOP_CHECK_EVERY == 0 && mrun_sched_looping(recent, recent_len)) return 3;
    return 0;
}

// The waiting request to start next (crates/mrun/src/runtime/handle.rs:563-587): the oldest side
// ("auxiliary") request, else the oldest request of another member's turn than the one served
// last (has_last = 0: nobody was served yet), else the oldest.  Before all of them, a request
// that gave its pages back and waits to go on (resumed[i] != 0): it was admitted once already.
// The arrays are in queue order, oldest first; turn < 0 = no member named.  -1 for an empty queue.
HOST_API int mrun_sched_next_turn(int n, const int* auxiliary, const int* turn, const int* resumed, int has_last,
                                  int last_turn) {
    for (int i = 0; i < n; ++i)
        if (resumed[i]) return i;
    for (int i = 0; i < n; ++i)
        if (auxiliary[i]) return i;
    if (has_last)
        for (int i = 0; i < n; ++i)
            if (turn[i] != last_turn) return i;
    return n > 0 ? 0 : -1;
}

// Stop sequences, on token ids (the reference matches stop strings on the streamed text, earliest
// match first, and holds back what may still begin one: crates/mrun/src/chat/stop.rs:24-85; at
// most 4 of them, crates/mrun/src/chat/limits.rs:6).  `stops` holds the n_stops sequences one after
// the other, `lens` their lengths; `tail` the last tail_len tokens of the output.
// The sequence that the output ends with, the longest if several do (it began earliest): its
// index, or -1.
HOST_API int mrun_sched_stop_match(const int* tail, int tail_len, const int* stops, const int* lens, int n_stops) {
    int best = -1, best_len = 0, at = 0;
    for (int s = 0; s < n_stops; at += lens[s], ++s) {
        const int len = lens[s];
        if (len < 1 || len > tail_len || len <= best_len) continue;
        if (std::equal(stops + at, stops + at + len, tail + tail_len - len)) {
            best = s;
            best_len = len;
        }
    }
    return best;
}

// How many tokens at the end of the output may still begin a stop sequence (a proper prefix of
// one): they are not streamed yet.
HOST_API int mrun_sched_stop_held(const int* tail, int tail_len, const int* stops, const int* lens, int n_stops) {
    int held = 0, at = 0;
    for (int s = 0; s < n_stops; at += lens[s], ++s)
        for (int n = std::min(lens[s] - 1, tail_len); n > held; --n)
            if (std::equal(stops + at, stops + at + n, tail + tail_len - n)) {
                held = n;
                break;
            }
    return held;
}

// The running request that gives its pages back when they run out: the one admitted last among
// those that have not ended (retiring[i] == 0); -1 when at most one such request runs.
HOST_API int mrun_sched_preemption_victim(int n, const int* retiring, const int64_t* order) {
    int candidates = 0, victim = -1;
    for (int i = 0; i < n; ++i) {
        if (retiring[i]) continue;
        ++candidates;
        if (victim < 0 || order[i] > order[victim]) victim = i;
    }
    return candidates <= 1 ? -1 : victim;
}
