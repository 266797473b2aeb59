// C-ABI implementation, part 4: continuous batching over the rows of one decoder.
//
// The reference's BatchScheduler (crates/autodiff/src/generate/scheduler.rs:395-) keeps a FIFO queue of requests
// and a bounded set of requests in progress, admits from the queue into free places at the start of every step,
// advances every request in progress by one token, finishes a request when it reaches its max_length, and
// processes requests in the order of their ids so that runs are reproducible.  Here a place is a row of the
// decoder's batch: a request is admitted by restarting a free row (b200_decoder_row_restart); all but the last token
// of its prompt go through one multi-token prefill pass of that row (b200_decoder_prefill), the last prompt token and
// then the sampled tokens are fed through the batched decode step; rows without a request sit the step out
// (b200_decoder_step_rows).  With prefill switched off the prompt is fed one token per step instead.
//
// A request that cannot be served - a token id outside the vocabulary, no cache blocks for its row - is set apart
// with its error and never reaches the device (take_failed, scheduler.rs:568-589, 718); the other requests go on.
//
// The host logic is split from the device calls so that it can be tested without a GPU: plan_step decides
// admissions and the token every row feeds, commit_step takes the sampled tokens.  Sampling is greedy (first
// maximum), the only mode of the decode driver.
#include <cstring>
#include <deque>
#include <new>
#include <string>
#include <vector>

#include "backend.h"

using namespace b200;

namespace {

struct Request {
    uint64_t id = 0;
    std::vector<int32_t> tokens;   // prompt, then generated tokens
    int32_t prompt_len = 0;
    int32_t max_length = 0;
    int32_t fed = 0;               // tokens given to the decoder so far
};

}  // namespace

struct b200_scheduler {
    b200_decoder* dec = nullptr;   // null: host logic only
    int32_t max_active = 0, max_queued = 0, max_length = 0;
    uint64_t next_id = 1;
    std::deque<Request> queue;
    std::vector<Request> rows;     // one slot per decoder row
    std::vector<uint8_t> busy;
    std::deque<Request> finished;
    bool step_planned = false;
    std::vector<int32_t> ids, sampled, restart_rows, restart_lens;
    std::vector<uint8_t> active;
    struct Failure { uint64_t id; int32_t status; std::string message; };
    std::deque<Failure> failed;
    bool prefill = false;          // admitted prompts go through a multi-token prefill pass (all but the last token)
    int32_t vocab = 0;             // 0: token ids are not checked on admission
};

namespace {

int32_t sched_invalid(const std::string& m) { return fail(B200_INVALID_ARGUMENT, "scheduler: " + m); }

}  // namespace

extern "C" {

int32_t b200_scheduler_create(b200_decoder* dec, int32_t max_active, int32_t max_queued, int32_t max_length,
                              b200_scheduler** out) {
    if (!out) return sched_invalid("out is null");
    *out = nullptr;
    // SchedulerLimits::new (scheduler.rs:90-107): every limit must be positive
    if (max_active <= 0 || max_queued <= 0 || max_length <= 0) return sched_invalid("limits must be positive");
    b200_scheduler* s = new (std::nothrow) b200_scheduler();
    if (!s) return fail(B200_DEVICE_ALLOCATION_FAILED, "scheduler: host allocation failed");
    s->dec = dec;
    s->max_active = max_active;
    s->max_queued = max_queued;
    s->max_length = max_length;
    s->rows.resize(max_active);
    s->busy.assign(max_active, 0);
    s->ids.assign(max_active, 0);
    s->sampled.assign(max_active, 0);
    s->active.assign(max_active, 0);
    s->restart_rows.assign(max_active, 0);
    s->restart_lens.assign(max_active, 0);
    if (dec) {
        s->prefill = true;
        s->vocab = b200_decoder_vocab(dec);
        std::vector<int32_t> lens(max_active, max_length);
        if (int32_t st = b200_decoder_begin(dec, max_active, nullptr, lens.data())) {
            delete s;
            return st;
        }
    }
    *out = s;
    return B200_OK;
}

void b200_scheduler_destroy(b200_scheduler* s) { delete s; }

int32_t b200_scheduler_queued_len(const b200_scheduler* s) { return s ? static_cast<int32_t>(s->queue.size()) : 0; }

int32_t b200_scheduler_active_len(const b200_scheduler* s) {
    if (!s) return 0;
    int32_t n = 0;
    for (uint8_t b : s->busy) n += b ? 1 : 0;
    return n;
}

int32_t b200_scheduler_finished_len(const b200_scheduler* s) { return s ? static_cast<int32_t>(s->finished.size()) : 0; }

// BatchScheduler::submit (scheduler.rs:445-504): queues a copy of the prompt; no forward; state unchanged on error.
int32_t b200_scheduler_submit(b200_scheduler* s, const int32_t* prompt, int32_t prompt_len, int32_t max_length,
                              uint64_t* request_id) {
    if (!s) return sched_invalid("scheduler is null");
    if (max_length <= 0) return sched_invalid("max_length must be positive");
    if (!prompt || prompt_len <= 0) return sched_invalid("the prompt is empty");
    if (prompt_len > max_length) return sched_invalid("the prompt is longer than max_length");
    if (max_length > s->max_length) return sched_invalid("max_length exceeds the scheduler's limit");
    if (static_cast<int32_t>(s->queue.size()) >= s->max_queued) return sched_invalid("the queue is full");
    Request r;
    r.id = s->next_id++;
    r.tokens.assign(prompt, prompt + prompt_len);
    r.prompt_len = prompt_len;
    r.max_length = max_length;
    s->queue.push_back(std::move(r));
    if (request_id) *request_id = s->queue.back().id;
    return B200_OK;
}

// First half of a step: admits queued requests into free rows (ascending row, FIFO queue; a request whose prompt
// already has max_length tokens finishes without a forward) and fills, per row, the token to feed and whether the
// row takes part.  restart_rows / restart_lens list the rows that were just given a new request.
int32_t b200_scheduler_plan_step(b200_scheduler* s, int32_t* ids, uint8_t* active, int32_t* restart_rows,
                                 int32_t* restart_lens, int32_t* n_restart, int32_t* completed_without_forward) {
    if (!s) return sched_invalid("scheduler is null");
    if (s->step_planned) return sched_invalid("the planned step has not been committed");
    int32_t nr = 0, done = 0;
    for (int32_t row = 0; row < s->max_active; ++row) {
        while (!s->busy[row] && !s->queue.empty()) {
            Request r = std::move(s->queue.front());
            s->queue.pop_front();
            if (s->vocab > 0) {                     // a request the model cannot embed is set apart, the others go on
                bool bad = false;
                for (int32_t t : r.tokens) bad = bad || t < 0 || t >= s->vocab;
                if (bad) {
                    s->failed.push_back({r.id, B200_INVALID_ARGUMENT, "the prompt holds a token id outside the vocabulary"});
                    continue;
                }
            }
            if (r.prompt_len == r.max_length) {     // nothing to generate (scheduler.rs:506-515)
                s->finished.push_back(std::move(r));
                ++done;
                continue;
            }
            if (s->prefill) r.fed = r.prompt_len - 1;   // the step function prefills tokens [0, prompt_len - 1)
            s->restart_rows[nr] = row;
            s->restart_lens[nr] = r.max_length;
            ++nr;
            s->rows[row] = std::move(r);
            s->busy[row] = 1;
        }
    }
    for (int32_t row = 0; row < s->max_active; ++row) {
        s->active[row] = s->busy[row];
        s->ids[row] = s->busy[row] ? s->rows[row].tokens[s->rows[row].fed] : 0;
    }
    if (ids) std::memcpy(ids, s->ids.data(), size_t(s->max_active) * sizeof(int32_t));
    if (active) std::memcpy(active, s->active.data(), size_t(s->max_active));
    if (restart_rows) std::memcpy(restart_rows, s->restart_rows.data(), size_t(nr) * sizeof(int32_t));
    if (restart_lens) std::memcpy(restart_lens, s->restart_lens.data(), size_t(nr) * sizeof(int32_t));
    if (n_restart) *n_restart = nr;
    if (completed_without_forward) *completed_without_forward = done;
    s->step_planned = true;
    return B200_OK;
}

// Second half: `sampled[row]` is the greedy token of the step for every row that took part.  A row whose fed token
// was the last prompt token or a generated one appends its sample; a request that reaches max_length finishes and
// frees its row.  *completed counts the requests finished by this call.
int32_t b200_scheduler_commit_step(b200_scheduler* s, const int32_t* sampled, int32_t* completed) {
    if (!s) return sched_invalid("scheduler is null");
    if (!s->step_planned) return sched_invalid("no step has been planned");
    if (!sampled) return sched_invalid("sampled is null");
    int32_t done = 0;
    for (int32_t row = 0; row < s->max_active; ++row) {
        if (!s->busy[row]) continue;
        Request& r = s->rows[row];
        r.fed += 1;
        if (r.fed >= r.prompt_len) r.tokens.push_back(sampled[row]);
        if (static_cast<int32_t>(r.tokens.size()) >= r.max_length) {
            s->finished.push_back(std::move(r));
            s->rows[row] = Request();
            s->busy[row] = 0;
            ++done;
        }
    }
    s->step_planned = false;
    if (completed) *completed = done;
    return B200_OK;
}

// BatchScheduler::step (scheduler.rs:571-589): admit, advance every request in progress by one token; returns the
// number of requests that completed in this call.  A device failure poisons the decoder and is returned.
int32_t b200_scheduler_step(b200_scheduler* s, int32_t* completed) {
    if (!s) return sched_invalid("scheduler is null");
    if (!s->dec) return sched_invalid("created without a decoder: use plan_step / commit_step");
    if (completed) *completed = 0;
    int32_t nr = 0, done0 = 0;
    std::vector<int32_t> rr(s->max_active), rl(s->max_active);
    if (int32_t st = b200_scheduler_plan_step(s, nullptr, nullptr, rr.data(), rl.data(), &nr, &done0)) return st;
    bool any = false;
    for (uint8_t b : s->active) any = any || b != 0;
    if (!any) {                      // nothing in progress: no forward
        s->step_planned = false;
        if (completed) *completed = done0;
        return B200_OK;
    }
    for (int32_t i = 0; i < nr; ++i) {
        const int32_t row = rr[i];
        Request& r = s->rows[row];
        int32_t st = b200_decoder_row_restart(s->dec, row, rl[i]);
        if (st == B200_OK && s->prefill && r.prompt_len > 1) st = b200_decoder_prefill(s->dec, row, 1, r.tokens.data(), r.prompt_len - 1);
        if (st == B200_INVALID_ARGUMENT || st == B200_UNSUPPORTED) {
            // this request cannot be served (no blocks for its row, ...): set it apart and free the row
            s->failed.push_back({r.id, st, b200_last_error()});
            s->rows[row] = Request();
            s->busy[row] = 0;
            s->active[row] = 0;
            s->ids[row] = 0;
        } else if (st != B200_OK) {
            s->step_planned = false;
            return st;
        }
    }
    any = false;
    for (uint8_t b : s->active) any = any || b != 0;
    if (!any) {
        s->step_planned = false;
        if (completed) *completed = done0;
        return B200_OK;
    }
    if (int32_t st = b200_decoder_step_rows(s->dec, s->ids.data(), s->active.data(), s->sampled.data())) {
        s->step_planned = false;
        return st;
    }
    int32_t done1 = 0;
    if (int32_t st = b200_scheduler_commit_step(s, s->sampled.data(), &done1)) return st;
    if (completed) *completed = done0 + done1;
    return B200_OK;
}

int32_t b200_scheduler_failed_len(const b200_scheduler* s) { return s ? static_cast<int32_t>(s->failed.size()) : 0; }

// take_failed (scheduler.rs:718): pops the oldest request that was set apart: its id, the status code and the message.
// *have = 0 when there is none.
int32_t b200_scheduler_take_failed(b200_scheduler* s, uint64_t* request_id, int32_t* status, char* message, int32_t capacity,
                                   int32_t* have) {
    if (!s || !have) return sched_invalid("null argument");
    *have = 0;
    if (s->failed.empty()) return B200_OK;
    const b200_scheduler::Failure& f = s->failed.front();
    if (request_id) *request_id = f.id;
    if (status) *status = f.status;
    if (message && capacity > 0) {
        std::strncpy(message, f.message.c_str(), size_t(capacity) - 1);
        message[capacity - 1] = 0;
    }
    *have = 1;
    s->failed.pop_front();
    return B200_OK;
}

// Host-logic switches for a scheduler without a decoder: whether admitted prompts are prefilled (all but the last
// token count as fed on admission) and the vocabulary size token ids are checked against (0: no check).
int32_t b200_scheduler_configure(b200_scheduler* s, int32_t prefill, int32_t vocab) {
    if (!s || vocab < 0) return sched_invalid("bad argument");
    s->prefill = prefill != 0;
    s->vocab = vocab;
    return B200_OK;
}

// Pops the oldest finished request: its id and tokens (prompt + generated).  *len = -1 when there is none; when
// `capacity` is too small nothing is popped, *len holds the needed size and the call fails.
int32_t b200_scheduler_take_finished(b200_scheduler* s, uint64_t* request_id, int32_t* tokens, int32_t capacity,
                                     int32_t* len) {
    if (!s || !len) return sched_invalid("null argument");
    if (s->finished.empty()) {
        *len = -1;
        return B200_OK;
    }
    const Request& r = s->finished.front();
    *len = static_cast<int32_t>(r.tokens.size());
    if (capacity < *len || !tokens) return sched_invalid("token buffer too small");
    std::memcpy(tokens, r.tokens.data(), r.tokens.size() * sizeof(int32_t));
    if (request_id) *request_id = r.id;
    s->finished.pop_front();
    return B200_OK;
}

}  // extern "C"
