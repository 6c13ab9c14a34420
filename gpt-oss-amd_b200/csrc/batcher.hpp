// Token grouping of the serving loop: which (sequence, position) rows go into
// the next forward() call.
//
// The reference cuts the requests into static batches of batch_size, hands a
// batch to a DP rank from an atomic counter (src/getp/run.cpp:661-736) and steps
// it one position per sequence per call until EVERY sequence of the batch has
// finished, re-compacting the rows that are still active each step
// (src/getp/run.cpp:573-617): the rows per call -- the T of the MoE block --
// decay as sequences finish, and the expert GEMMs run at a fraction of the batch
// they were sized for.  This scheduler keeps a pool of n_slots sequence slots per
// rank; in continuous mode a slot whose sequence finished is refilled at once
// from the shared request queue (the same atomic hand-out, one request at a
// time), so T stays at n_slots until the queue drains.  A slot is what the
// engine calls batch index (its KV-cache row, the batch_indices argument of
// forward(), src/forward.cpp:202-204); a refilled slot starts again at position 0.
// Static mode reproduces the reference's loop row for row (tests compare the two).
//
// Per-sequence rules are the reference's (src/getp/run.cpp:547-571,573-617): a
// prompt is fed one token per step; once the position passes the prompt the
// sampled token is appended to the request's output; tokens 199999 and 200002 or
// position + 1 >= max_seq_len end the sequence and a -1 closes its output.
//
// Host code only; one batcher per rank (thread), one queue shared by all.
#pragma once
#include <atomic>
#include <vector>

namespace moe {
namespace sched {

constexpr int EOS_A = 199999, EOS_B = 200002;  // src/getp/run.cpp:558

struct RequestQueue {
    int n_requests = 0, max_seq_len = 0;
    const int* const* prompt_tokens = nullptr;  // [n_requests] -> [prompt_lens[r]]
    const int* prompt_lens = nullptr;
    int* const* output_tokens = nullptr;        // [n_requests] -> [max_seq_len + 1], may be null
    std::atomic<int> next{0};                   // next request (continuous) / next batch start (static)
};

struct Slot {
    int request = -1;
    int pos = 0, current = 0;
    bool finished = true;
};

struct Batcher {
    RequestQueue* q = nullptr;
    int n_slots = 0;
    bool continuous = true;
    std::vector<Slot> slots;
    std::vector<int> row_slot;  // rows of the step in flight
    int active = 0;             // sequences not finished
    bool step_open = false;
    long long steps = 0, rows = 0, tokens_out = 0;
};

inline void start_sequence(Batcher& b, int slot, int request) {
    Slot& s = b.slots[slot];
    s.request = request;
    s.pos = 0;
    s.current = b.q->prompt_tokens[request][0];
    s.finished = false;
    b.active++;
}

// Fills free slots from the queue.  Continuous: every free slot, one request each.
// Static: only when no sequence is active, a whole batch of consecutive requests
// (the reference's batch_starts hand-out, src/getp/run.cpp:668-676,716-722).
inline void refill(Batcher& b) {
    RequestQueue& q = *b.q;
    if (b.continuous) {
        for (int s = 0; s < b.n_slots; s++) {
            if (!b.slots[s].finished)
                continue;
            const int r = q.next.fetch_add(1, std::memory_order_relaxed);
            if (r >= q.n_requests) {
                q.next.store(q.n_requests, std::memory_order_relaxed);  // keep the counter from wrapping
                break;
            }
            start_sequence(b, s, r);
        }
    } else if (b.active == 0) {
        const int start = q.next.fetch_add(b.n_slots, std::memory_order_relaxed);
        if (start >= q.n_requests) {
            q.next.store(q.n_requests, std::memory_order_relaxed);
            return;
        }
        const int n = q.n_requests - start < b.n_slots ? q.n_requests - start : b.n_slots;
        for (int s = 0; s < b.n_slots; s++)
            b.slots[s] = Slot();
        for (int s = 0; s < n; s++)
            start_sequence(b, s, start + s);
    }
}

// The rows of the next forward(): token, position and slot of every active sequence,
// in slot order (src/getp/run.cpp:576-583).  needs_sample[i] (optional) tells whether
// row i's next token comes from the sampler (its position has reached the end of the
// prompt) or from the prompt.  Returns the number of rows; 0 = everything is done.
inline int begin_step(Batcher& b, int* tokens, int* positions, int* slot_ids, int* needs_sample) {
    for (;;) {
        refill(b);
        b.row_slot.clear();
        const int steps = b.q->max_seq_len;
        for (int s = 0; s < b.n_slots; s++) {
            const Slot& sl = b.slots[s];
            if (!sl.finished && sl.pos + 1 < steps) {
                const int i = (int)b.row_slot.size();
                tokens[i] = sl.current;
                positions[i] = sl.pos;
                slot_ids[i] = s;
                if (needs_sample)
                    needs_sample[i] = (sl.pos + 1 >= b.q->prompt_lens[sl.request]) ? 1 : 0;
                b.row_slot.push_back(s);
            }
        }
        if (!b.row_slot.empty())
            break;
        // nothing to run: sequences that cannot advance (max_seq_len reached before they
        // finished) are dropped as the reference's loop drops them (its `break`)
        bool dropped = false;
        for (int s = 0; s < b.n_slots; s++)
            if (!b.slots[s].finished) {
                b.slots[s].finished = true;
                b.active--;
                dropped = true;
            }
        if (!dropped && b.q->next.load(std::memory_order_relaxed) >= b.q->n_requests)
            return 0;  // every slot is free and the queue is empty
    }
    b.step_open = true;
    b.steps++;
    b.rows += (long long)b.row_slot.size();
    return (int)b.row_slot.size();
}

// After forward(): sampled[i] is the sampler's token for row i (read only where the
// row has left its prompt).  Applies src/getp/run.cpp:547-571,596-611.
inline void end_step(Batcher& b, const int* sampled) {
    const int steps = b.q->max_seq_len;
    for (size_t i = 0; i < b.row_slot.size(); i++) {
        Slot& s = b.slots[b.row_slot[i]];
        const int r = s.request;
        const int n_prompt = b.q->prompt_lens[r];
        int* out = b.q->output_tokens ? b.q->output_tokens[r] : nullptr;
        s.pos++;
        int next;
        bool counted;
        if (s.pos < n_prompt) {
            next = b.q->prompt_tokens[r][s.pos];
            counted = false;
        } else {
            next = sampled[i];
            counted = true;
        }
        if (counted) {
            const int oi = s.pos - n_prompt;
            if (out && oi >= 0)
                out[oi] = next;
            b.tokens_out++;
        }
        if ((next == EOS_A || next == EOS_B || s.pos + 1 >= steps) && !s.finished) {
            s.finished = true;
            b.active--;
            const int end = s.pos - n_prompt + 1;
            if (out && end >= 0)
                out[end] = -1;
        }
        s.current = next;
    }
    b.step_open = false;
}

}  // namespace sched
}  // namespace moe
