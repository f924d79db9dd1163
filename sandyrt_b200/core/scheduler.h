// The scheduler: which requests run in the next step, with how many tokens each.
//
// It works on the host-side BlockAllocator only, so all of its decisions can be tested without a
// GPU.
//
// The reference lets exactly one request generate at a time (a FIFO ticket gate,
// src/server/GenerationGate.cpp:13-37) and runs it to the end: the prompt in chunks of
// `prefillChunkTokens` (default 2048, src/server/Session.h:23, loop :423-448), then token by token
// (:477-514); finish reasons "stop" (the stop token is part of the output, :481-497) and "length"
// (:498-501; max_tokens == 0 finishes at once with no forward, :407-417).  Those meanings are
// kept.  What is new here is that many requests are live at once:
//
//   * admission: first come first served, while a state slot is free, fewer than `max_live` are
//     running and the pool can hold the request's first portion;
//   * a token budget per step: every running request that is decoding gets its one token first;
//     what is left of the budget goes to prompts, oldest first, in portions of at most
//     `prefill_chunk` tokens, cut wherever the budget or the free pages end;
//   * pages run out: a decoding request that cannot get its next page preempts the most recently
//     admitted running request (possibly itself): that request gives back all its pages and goes
//     back to the head of the waiting queue with prompt + output so far, to be recomputed later.
//     A request that could never fit in the whole pool is refused when it is added.
#pragma once

#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <unordered_set>
#include <vector>

#include "cache.h"
#include "sampling.h"

namespace sandy {

enum class RequestState { Waiting, Running, Finished };

struct Request {
    RequestId rid = 0;
    std::vector<int> prompt;
    int max_tokens = 0;
    std::unordered_set<int> stop_ids;
    SamplingParams sampling;
    uint64_t seed = 0;                 // the seed the request's uniform numbers come from
    std::vector<int> output;
    RequestState state = RequestState::Waiting;
    int computed = 0;                  // tokens of prompt+output whose keys/values are cached
    std::string finish_reason;
    int preemptions = 0;
    int64_t admitted_at = -1;          // admission counter value (larger = admitted later)
    // timing, filled by the caller of the scheduler (seconds on a steady clock)
    double t_added = 0, t_first_scheduled = 0, t_first_token = 0, t_finished = 0;

    int n_tokens() const { return (int)(prompt.size() + output.size()); }
    int pending() const { return n_tokens() - computed; }       // tokens not yet run through the model
    int token(int i) const { return i < (int)prompt.size() ? prompt[(size_t)i] : output[(size_t)i - prompt.size()]; }
    int last_token() const { return output.empty() ? prompt.back() : output.back(); }
};
using RequestPtr = std::shared_ptr<Request>;

// One request's share of a planned step.
struct Portion {
    RequestPtr request;
    int start = 0;             // index into the request's tokens of the first token run
    int count = 0;
    bool samples = false;      // the portion reaches the request's last token: sample after it
};

struct StepPlan {
    std::vector<Portion> portions;
    std::vector<RequestPtr> preempted;
    int n_tokens() const {
        int n = 0;
        for (const auto& p : portions) n += p.count;
        return n;
    }
};

class Scheduler {
public:
    struct Options {
        int max_step_tokens = 2048;
        int prefill_chunk = 2048;
        int max_live = 64;
        std::optional<int> max_positions;
    };
    // admit: how a request takes its state slot (default: the allocator's own `admit`).  The entry
    // point passes the cache manager's, which also zeroes the slot's fixed-size state on the
    // device, so that a request never starts from the state of the slot's last holder.
    Scheduler(BlockAllocator& alloc, Options options, std::function<int(RequestId)> admit = {});

    void add(RequestPtr req);                        // RequestRefused if it can never be served
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    StepPlan plan();                                 // decide the next step and reserve its pages; may preempt
    // The planned step ran.  `sampled[i]` is the token drawn for portion i (ignored unless it
    // samples).  Returns the requests that finished.
    std::vector<RequestPtr> complete(const StepPlan& plan, const std::vector<int>& sampled);
    RequestPtr abort(RequestId rid, const std::string& reason = "cancelled");
    void forget(RequestId rid);                      // drop a finished request from the scheduler's records

    const std::deque<RequestPtr>& waiting() const { return waiting_; }
    const std::vector<RequestPtr>& running() const { return running_; }
    const std::vector<RequestPtr>& finished() const { return finished_; }
    const std::map<std::string, int64_t>& stats() const { return stats_; }
    const Options& options() const { return opt_; }

private:
    int pages_for(int group, int n_tokens) const;
    void preempt(const RequestPtr& req, StepPlan& plan);
    int fit(const Request& req, int want) const;
    void finish(const RequestPtr& req, const std::string& reason);
    BlockAllocator& alloc_;
    Options opt_;
    std::function<int(RequestId)> admit_;
    std::deque<RequestPtr> waiting_;
    std::vector<RequestPtr> running_, finished_;
    int64_t admissions_ = 0;
    std::map<std::string, int64_t> stats_;
};

}  // namespace sandy
