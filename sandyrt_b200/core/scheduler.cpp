#include "scheduler.h"

#include <algorithm>
#include <fstream>
#include <random>

namespace sandy {

uint64_t fresh_seed() {
    uint64_t v = 0;
    std::ifstream f("/dev/urandom", std::ios::binary);
    if (f && f.read(reinterpret_cast<char*>(&v), sizeof v)) return v;
    std::random_device rd;
    return ((uint64_t)rd() << 32) ^ rd();
}

Scheduler::Scheduler(BlockAllocator& alloc, Options options, std::function<int(RequestId)> admit)
    : alloc_(alloc), opt_(options), admit_(std::move(admit)) {
    if (opt_.max_step_tokens <= 0 || opt_.prefill_chunk <= 0 || opt_.max_live <= 0)
        throw ValueError("token budget, chunk size and request limit must be positive");
    if (!admit_) admit_ = [this](RequestId rid) { return alloc_.admit(rid); };
    stats_ = {{"admissions", 0}, {"preemptions", 0}, {"steps", 0}, {"tokens", 0}};
}

// Most pages of `group` a request of n_tokens holds at one time.
int Scheduler::pages_for(int group, int n_tokens) const {
    const int ps = alloc_.page_size();
    const int window = alloc_.layout().groups[(size_t)group].spec.window;
    const int all = (n_tokens + ps - 1) / ps;
    if (window) {
        // pages covering the window plus the portion being appended
        const int span = std::min(n_tokens, window + opt_.prefill_chunk);
        return std::min(all, (span + ps - 1) / ps + 1);
    }
    return all;
}

void Scheduler::add(RequestPtr req) {
    if (req->prompt.empty()) throw RequestRefused("the prompt must not be empty");          // Session.cpp:389-390
    if (req->max_tokens < 0) throw RequestRefused("max_tokens must be >= 0");               // Session.cpp:391-392
    if (opt_.max_positions && (int)req->prompt.size() > *opt_.max_positions)
        throw RequestRefused("the prompt has " + std::to_string(req->prompt.size()) + " tokens, the model has " +
                             std::to_string(*opt_.max_positions) + " positions");
    int longest = (int)req->prompt.size() + std::max(req->max_tokens - 1, 0);
    if (opt_.max_positions) longest = std::min(longest, *opt_.max_positions);
    for (int g = 0; g < alloc_.n_groups(); g++) {
        const int need = pages_for(g, longest);
        if (need > alloc_.pool(g).num_pages())
            throw RequestRefused("the request may grow to " + std::to_string(longest) + " tokens, which needs " +
                                 std::to_string(need) + " pages of cache group " + std::to_string(g) + "; the pool has " +
                                 std::to_string(alloc_.pool(g).num_pages()));
    }
    if (req->max_tokens == 0) {
        req->state = RequestState::Finished;
        req->finish_reason = "length";
        finished_.push_back(std::move(req));
        return;
    }
    req->state = RequestState::Waiting;
    waiting_.push_back(std::move(req));
}

void Scheduler::preempt(const RequestPtr& req, StepPlan& plan) {
    alloc_.release(req->rid);
    running_.erase(std::remove(running_.begin(), running_.end(), req), running_.end());
    req->state = RequestState::Waiting;
    req->computed = 0;
    req->preemptions++;
    waiting_.push_front(req);
    plan.preempted.push_back(req);
    plan.portions.erase(std::remove_if(plan.portions.begin(), plan.portions.end(),
                                       [&](const Portion& p) { return p.request == req; }),
                        plan.portions.end());
    stats_["preemptions"]++;
}

// Largest n <= want such that pages for req.computed + n tokens can be reserved.
int Scheduler::fit(const Request& req, int want) const {
    const int lo = req.computed;
    if (alloc_.can_reserve(req.rid, lo + want)) return want;
    const int ps = alloc_.page_size();
    int best = want;
    for (int g = 0; g < alloc_.n_groups(); g++) {
        const int have = (int)alloc_.block_list(req.rid, g).size();
        const int room = (have + alloc_.pool(g).free_pages()) * ps - lo;
        best = std::min(best, room);
    }
    return std::max(best, 0);
}

StepPlan Scheduler::plan() {
    StepPlan plan;
    int budget = opt_.max_step_tokens;
    std::vector<RequestPtr> by_age = running_;
    std::sort(by_age.begin(), by_age.end(), [](const RequestPtr& a, const RequestPtr& b) { return a->admitted_at < b->admitted_at; });
    auto newest = [this]() {
        return *std::max_element(running_.begin(), running_.end(),
                                 [](const RequestPtr& a, const RequestPtr& b) { return a->admitted_at < b->admitted_at; });
    };

    // 1. running requests that are decoding: one token each, oldest first
    for (const RequestPtr& req : by_age) {
        if (req->state != RequestState::Running || req->pending() != 1 || req->output.empty()) continue;
        if (budget <= 0) break;
        while (req->state == RequestState::Running && !alloc_.can_reserve(req->rid, req->computed + 1)) preempt(newest(), plan);
        if (req->state != RequestState::Running) continue;          // it preempted itself
        alloc_.reserve(req->rid, req->computed + 1);
        plan.portions.push_back(Portion{req, req->computed, 1, true});
        budget--;
    }

    // 2. running requests still working through their prompt (or a recomputation)
    for (const RequestPtr& req : by_age) {
        if (budget <= 0) break;
        if (req->state != RequestState::Running) continue;
        bool scheduled = false;
        for (const auto& p : plan.portions) scheduled = scheduled || p.request == req;
        if (scheduled) continue;
        const int n = fit(*req, std::min({req->pending(), opt_.prefill_chunk, budget}));
        if (n <= 0) continue;
        alloc_.reserve(req->rid, req->computed + n);
        plan.portions.push_back(Portion{req, req->computed, n, n == req->pending()});
        budget -= n;
    }

    // 3. admit waiting requests, first come first served
    while (!waiting_.empty() && budget > 0 && (int)running_.size() < opt_.max_live) {
        RequestPtr req = waiting_.front();
        if (std::find(plan.preempted.begin(), plan.preempted.end(), req) != plan.preempted.end())
            break;                                                  // never re-admit in the step that preempted it
        if (alloc_.free_slots() == 0) break;
        const int first = std::min({req->pending(), opt_.prefill_chunk, budget});
        const std::vector<int> needed = alloc_.pages_for_new_request(first);
        bool room = true;
        for (size_t g = 0; g < needed.size(); g++) room = room && needed[g] <= alloc_.free_pages((int)g);
        if (!room) break;
        waiting_.pop_front();
        admit_(req->rid);
        alloc_.reserve(req->rid, first);
        req->state = RequestState::Running;
        req->admitted_at = admissions_++;
        running_.push_back(req);
        plan.portions.push_back(Portion{req, 0, first, first == req->pending()});
        budget -= first;
        stats_["admissions"]++;
    }

    // 4. nothing could move although requests are live: every running request is in the middle of
    //    its prompt and the pool is full.  Give the newest one's pages to the rest.
    if (plan.portions.empty() && !running_.empty()) {
        preempt(newest(), plan);
        if (!running_.empty() || !waiting_.empty()) {
            StepPlan again = this->plan();
            again.preempted.insert(again.preempted.begin(), plan.preempted.begin(), plan.preempted.end());
            return again;
        }
    }
    stats_["steps"]++;
    stats_["tokens"] += plan.n_tokens();
    return plan;
}

std::vector<RequestPtr> Scheduler::complete(const StepPlan& plan, const std::vector<int>& sampled) {
    std::vector<RequestPtr> done;
    for (size_t i = 0; i < plan.portions.size(); i++) {
        const Portion& p = plan.portions[i];
        const RequestPtr& req = p.request;
        req->computed = p.start + p.count;
        alloc_.commit(req->rid, req->computed);
        if (!p.samples) continue;
        const int token = sampled.at(i);
        req->output.push_back(token);
        std::string reason;
        if (req->stop_ids.count(token)) reason = "stop";
        else if ((int)req->output.size() >= req->max_tokens) reason = "length";
        else if (opt_.max_positions && req->n_tokens() > *opt_.max_positions)
            reason = "length";                                     // the new token has no position left to run at
        if (!reason.empty()) {
            finish(req, reason);
            done.push_back(req);
        }
    }
    return done;
}

void Scheduler::finish(const RequestPtr& req, const std::string& reason) {
    req->state = RequestState::Finished;
    req->finish_reason = reason;
    auto it = std::find(running_.begin(), running_.end(), req);
    if (it != running_.end()) {
        running_.erase(it);
        alloc_.release(req->rid);
    }
    finished_.push_back(req);
}

void Scheduler::forget(RequestId rid) {
    finished_.erase(std::remove_if(finished_.begin(), finished_.end(), [rid](const RequestPtr& r) { return r->rid == rid; }),
                    finished_.end());
}

RequestPtr Scheduler::abort(RequestId rid, const std::string& reason) {
    for (const RequestPtr& req : running_)
        if (req->rid == rid) {
            RequestPtr keep = req;
            finish(keep, reason);
            return keep;
        }
    for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
        if ((*it)->rid == rid) {
            RequestPtr req = *it;
            waiting_.erase(it);
            req->state = RequestState::Finished;
            req->finish_reason = reason;
            finished_.push_back(req);
            return req;
        }
    return nullptr;
}

}  // namespace sandy
