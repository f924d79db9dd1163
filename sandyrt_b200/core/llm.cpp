#include "llm.h"

#include <algorithm>
#include <chrono>
#include <cstdio>

namespace sandy {

namespace {
double now_seconds() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
double rate(int tokens, double ms) { return ms > 0 ? tokens / (ms / 1000.0) : 0.0; }
}  // namespace

std::unique_ptr<LLM> LLM::load(const std::string& model_dir, const LLMOptions& options) {
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0)
        throw StepError("sandyrt_b200 needs a CUDA device; there is no CPU path");
    cuda_check(cudaSetDevice(options.device), "selecting the device");
    return std::unique_ptr<LLM>(new LLM(load_model(model_dir, options.dtype), options));
}

LLM::LLM(std::unique_ptr<Model> model, const LLMOptions& options) : opt_(options), model_(std::move(model)) {
    std::optional<int64_t> limit = model_->max_positions();
    if (opt_.max_context_tokens > 0) limit = limit ? std::min<int64_t>(*limit, opt_.max_context_tokens) : opt_.max_context_tokens;
    if (limit) max_positions_ = (int)*limit;
    int64_t cache_tokens = opt_.cache_tokens;
    if (cache_tokens <= 0) cache_tokens = std::min<int64_t>((int64_t)opt_.max_live * (limit ? *limit : 4096), 1 << 20);
    Engine::Options eo;
    eo.max_tokens = cache_tokens;
    eo.page_size = opt_.page_size;
    eo.max_requests = opt_.max_live;
    eo.max_step_tokens = opt_.max_step_tokens;
    eo.use_cuda_graphs = opt_.use_cuda_graphs;
    engine_.reset(new Engine(*model_, eo));
    Scheduler::Options so;
    so.max_step_tokens = opt_.max_step_tokens;
    so.prefill_chunk = opt_.prefill_chunk_tokens;
    so.max_live = opt_.max_live;
    so.max_positions = max_positions_;
    Engine* eng = engine_.get();
    scheduler_.reset(new Scheduler(engine_->cache().alloc(), so, [eng](RequestId rid) { return eng->admit(rid); }));
    max_burst_ = engine_->use_cuda_graphs() ? std::max(1, std::min(opt_.max_burst, kMaxBurst)) : 1;
}

RequestPtr LLM::find(RequestId rid) const {
    auto it = requests_.find(rid);
    if (it == requests_.end()) throw ValueError("unknown request id " + std::to_string(rid));
    return it->second;
}

RequestId LLM::add_request(const std::vector<int>& prompt_ids, int max_tokens, const SamplingParams& sampling,
                           const std::vector<int>& stop_token_ids) {
    sampling.validate();
    const int64_t vocab = model_->spec().vocab_size;
    for (int t : prompt_ids)
        if (t < 0 || t >= vocab)
            throw RequestRefused("token id " + std::to_string(t) + " is outside the vocabulary of " + std::to_string(vocab));
    auto req = std::make_shared<Request>();
    req->rid = next_id_++;
    req->prompt = prompt_ids;
    req->max_tokens = max_tokens;
    req->stop_ids.insert(stop_token_ids.begin(), stop_token_ids.end());
    req->stop_ids.insert(opt_.eos_token_ids.begin(), opt_.eos_token_ids.end());
    req->sampling = sampling;
    req->seed = sampling.seed ? *sampling.seed : fresh_seed();
    req->t_added = now_seconds();
    scheduler_->add(req);
    requests_[req->rid] = req;
    return req->rid;
}

// How many decode steps may run on the device before the host looks again: more than one only when
// every request of the step is decoding and nobody waits to be admitted, and never past a request's
// token limit, the model's positions or the free pages.
int LLM::burst_length(const StepPlan& plan) const {
    if (max_burst_ <= 1 || !scheduler_->waiting().empty() || plan.portions.empty()) return 1;
    std::vector<RequestPtr> reqs;
    for (const Portion& p : plan.portions) {
        if (p.count != 1 || !p.samples || p.request->output.empty()) return 1;
        reqs.push_back(p.request);
    }
    return steps_possible(reqs, 0);
}

// Steps (at most max_burst, possibly 0) that all of `reqs` can still take when they are already
// `in_flight` steps ahead of what the host has seen: no request past its token limit or the model's
// positions, and pages for all of them.
int LLM::steps_possible(const std::vector<RequestPtr>& reqs, int in_flight) const {
    int n = max_burst_;
    for (const RequestPtr& r : reqs) {
        n = std::min(n, r->max_tokens - (int)r->output.size() - in_flight);
        if (max_positions_) n = std::min(n, *max_positions_ - r->computed - in_flight);
    }
    const BlockAllocator& alloc = engine_->cache().alloc();
    while (n > 1) {
        std::vector<int> need((size_t)alloc.n_groups(), 0);
        for (const RequestPtr& r : reqs) {
            const std::vector<int> k = alloc.pages_needed(r->rid, r->computed + in_flight + n);
            for (size_t g = 0; g < k.size(); g++) need[g] += k[g];
        }
        bool ok = true;
        for (size_t g = 0; g < need.size(); g++) ok = ok && need[g] <= alloc.free_pages((int)g);
        if (ok) break;
        n /= 2;
    }
    return std::max(n, in_flight == 0 ? 1 : 0);
}

// Queue n decode steps of `reqs` on the device (behind `in_flight` steps already queued).
BurstHandle LLM::queue_burst(const std::vector<RequestPtr>& reqs, int n, int in_flight) {
    std::vector<StepEntry> entries;
    std::vector<SampleRow> rows;
    std::vector<float> uniforms((size_t)n * reqs.size(), 0.0f);
    for (size_t i = 0; i < reqs.size(); i++) {
        const Request& r = *reqs[i];
        StepEntry e;
        e.rid = r.rid;
        e.tokens = {in_flight ? 0 : r.last_token()};
        e.want = {0};
        entries.push_back(std::move(e));
        const SamplingParams& sp = r.sampling;
        rows.push_back(SampleRow{sp.greedy() ? 0.0f : sp.temperature, sp.top_k, sp.top_p, 0.0f});
        if (!sp.greedy())
            for (int j = 0; j < n; j++) uniforms[(size_t)j * reqs.size() + i] = uniform_for(r.seed, r.output.size() + (size_t)in_flight + (size_t)j);
    }
    return engine_->decode_burst_async(entries, rows, uniforms, n, in_flight);
}

// Read a queued burst's tokens and do the scheduler's bookkeeping for each of its steps in order.  A
// request that finishes part of the way (or was finished or aborted while the burst ran) keeps only
// the tokens up to its finish; what the device computed for it after that is dropped.
std::vector<std::pair<RequestId, int>> LLM::collect_burst(const BurstHandle& handle, const std::vector<RequestPtr>& reqs) {
    const std::vector<int> tokens = engine_->burst_tokens(handle);      // throws if a kernel of the burst reported a fault
    const int n = handle.n, S = handle.S;
    decode_steps_run += n;
    const double now = now_seconds();
    std::vector<std::pair<RequestId, int>> got;
    std::vector<int> alive;
    for (int i = 0; i < S; i++)
        if (reqs[(size_t)i]->state == RequestState::Running) alive.push_back(i);
    for (int j = 0; j < n; j++)
        for (int i : alive)
            if (tokens[(size_t)j * S + i] < 0) throw ValueError("sampling logits must not contain NaN");      // Sampler.cpp:64-67
    for (int j = 0; j < n && !alive.empty(); j++) {
        StepPlan sub;
        std::vector<int> sampled;
        for (int i : alive) {
            sub.portions.push_back(Portion{reqs[(size_t)i], reqs[(size_t)i]->computed, 1, true});
            sampled.push_back(tokens[(size_t)j * S + i]);
            got.emplace_back(reqs[(size_t)i]->rid, tokens[(size_t)j * S + i]);
        }
        for (const RequestPtr& r : scheduler_->complete(sub, sampled)) r->t_finished = now;
        std::vector<int> still;
        for (int i : alive)
            if (reqs[(size_t)i]->state == RequestState::Running) still.push_back(i);
        alive.swap(still);
    }
    return got;
}

// A burst is in flight.  If its requests can all go on (nobody is waiting to be admitted, nobody is
// known to have finished, tokens, positions and pages allow it), queue the next burst behind it
// BEFORE reading its tokens; then read them.  A request that turns out to have stopped inside the
// burst just read has wasted rows in the one queued behind it, nothing more: its pages are given back
// at once, but anything that could reuse them is queued on the same stream behind that burst.
std::vector<std::pair<RequestId, int>> LLM::advance() {
    std::unique_ptr<Inflight> cur = std::move(inflight_);
    std::unique_ptr<Inflight> next;
    bool all_running = true;
    for (const RequestPtr& r : cur->reqs) all_running = all_running && r->state == RequestState::Running;
    if (opt_.pipeline_bursts && scheduler_->waiting().empty() && all_running) {
        const int n = steps_possible(cur->reqs, cur->handle.n);
        if (n >= 1) {
            try {
                BurstHandle h = queue_burst(cur->reqs, n, cur->handle.n);
                next.reset(new Inflight{h, cur->reqs});
                bursts_queued_ahead++;
            } catch (const OutOfPages&) {
            }
        }
    }
    std::vector<std::pair<RequestId, int>> got = collect_burst(cur->handle, cur->reqs);
    inflight_ = std::move(next);
    return got;
}

std::vector<std::pair<RequestId, int>> LLM::step() {
    if (inflight_) return advance();
    StepPlan plan = scheduler_->plan();
    if (plan.portions.empty()) return {};
    const int n_burst = burst_length(plan);
    if (n_burst > 1) {
        std::vector<RequestPtr> reqs;
        for (const Portion& p : plan.portions) reqs.push_back(p.request);
        BurstHandle h = queue_burst(reqs, n_burst, 0);
        inflight_.reset(new Inflight{h, reqs});
        return advance();
    }
    double now = now_seconds();
    std::vector<StepEntry> entries;
    std::vector<SampleRow> rows;
    std::vector<size_t> sampled_portions;
    for (size_t i = 0; i < plan.portions.size(); i++) {
        const Portion& p = plan.portions[i];
        Request& req = *p.request;
        if (req.t_first_scheduled == 0.0) req.t_first_scheduled = now;
        StepEntry e;
        e.rid = req.rid;
        e.tokens.reserve((size_t)p.count);
        for (int t = p.start; t < p.start + p.count; t++) e.tokens.push_back(req.token(t));
        if (p.samples) {
            e.want = {p.count - 1};
            const SamplingParams& sp = req.sampling;
            rows.push_back(SampleRow{sp.greedy() ? 0.0f : sp.temperature, sp.top_k, sp.top_p,
                                     sp.greedy() ? 0.0f : uniform_for(req.seed, req.output.size())});
            sampled_portions.push_back(i);
        }
        entries.push_back(std::move(e));
    }
    engine_->step(entries, &rows);
    std::vector<int> sampled(plan.portions.size(), 0);
    std::vector<std::pair<RequestId, int>> got;
    if (!sampled_portions.empty()) {
        const std::vector<int> host = engine_->read_sampled((int)sampled_portions.size());    // throws on a kernel fault
        for (size_t k = 0; k < sampled_portions.size(); k++) {
            if (host[k] < 0) throw ValueError("sampling logits must not contain NaN");       // Sampler.cpp:64-67
            sampled[sampled_portions[k]] = host[k];
            got.emplace_back(plan.portions[sampled_portions[k]].request->rid, host[k]);
        }
    }
    now = now_seconds();
    for (size_t k : sampled_portions) {
        Request& r = *plan.portions[k].request;
        if (r.t_first_token == 0.0) r.t_first_token = now;
    }
    for (const RequestPtr& r : scheduler_->complete(plan, sampled)) r->t_finished = now;
    decode_steps_run++;
    return got;
}

std::vector<std::pair<RequestId, int>> LLM::drain() {
    std::vector<std::pair<RequestId, int>> got;
    while (inflight_) {
        std::unique_ptr<Inflight> cur = std::move(inflight_);
        auto more = collect_burst(cur->handle, cur->reqs);
        got.insert(got.end(), more.begin(), more.end());
    }
    return got;
}

bool LLM::finished(RequestId rid) const { return find(rid)->state == RequestState::Finished; }
const Request& LLM::request(RequestId rid) const { return *find(rid); }

GenerateResult LLM::result(RequestId rid) const {
    const Request& r = *find(rid);
    const double t_end = r.t_finished != 0.0 ? r.t_finished : now_seconds();
    const double first = r.t_first_token != 0.0 ? r.t_first_token : t_end;
    const double start = r.t_first_scheduled != 0.0 ? r.t_first_scheduled : r.t_added;
    GenerateResult g;
    g.output_ids = r.output;
    g.finish_reason = r.finish_reason;
    g.prompt_tokens = (int)r.prompt.size();
    g.completion_tokens = (int)r.output.size();
    g.prefill_ms = std::max(0.0, (first - start) * 1e3);
    g.decode_ms = std::max(0.0, (t_end - first) * 1e3);
    g.prefill_tokens_per_second = rate(g.prompt_tokens, g.prefill_ms);
    g.decode_tokens_per_second = rate(std::max(g.completion_tokens - 1, 0), g.decode_ms);
    g.preemptions = r.preemptions;
    return g;
}

void LLM::forget(RequestId rid) {
    requests_.erase(rid);
    scheduler_->forget(rid);
}
void LLM::abort(RequestId rid) { scheduler_->abort(rid, "cancelled"); }

std::vector<GenerateResult> LLM::generate(const std::vector<std::vector<int>>& prompts, const GenerateParams& params) {
    std::vector<RequestId> rids;
    std::unordered_map<RequestId, int> index;
    try {
        for (size_t i = 0; i < prompts.size(); i++) {
            SamplingParams s;
            s.temperature = params.temperature;
            s.top_k = params.top_k;
            s.top_p = params.top_p;
            if (params.seed) s.seed = *params.seed + i;
            rids.push_back(add_request(prompts[i], params.max_tokens, s, params.stop_token_ids));
            index[rids.back()] = (int)i;
        }
    } catch (...) {
        for (RequestId r : rids) { abort(r); forget(r); }
        throw;
    }
    std::unordered_map<RequestId, int> delivered;
    std::unordered_map<RequestId, bool> cancelled;
    auto pending = [&]() {
        for (RequestId r : rids)
            if (!finished(r)) return true;
        return false;
    };
    while (pending()) {
        const auto got = step();
        if (!params.on_token) continue;
        for (const auto& rt : got) {
            auto it = index.find(rt.first);
            if (it == index.end() || cancelled[rt.first]) continue;
            delivered[rt.first]++;
            if (!params.on_token(it->second, rt.second)) {
                // the request ends with the token just delivered; what a burst had already drawn
                // beyond it is dropped
                cancelled[rt.first] = true;
                RequestPtr r = find(rt.first);
                if (r->state != RequestState::Finished) abort(rt.first);
                r->output.resize((size_t)delivered[rt.first]);
                r->finish_reason = "cancelled";
            }
        }
    }
    std::vector<GenerateResult> results;
    for (RequestId r : rids) results.push_back(result(r));
    for (RequestId r : rids) forget(r);
    if (params.report)
        for (const GenerateResult& res : results)
            // the reference prints the same line to stderr (src/server/Session.cpp:539-548)
            std::fprintf(stderr,
                         "sandy throughput: prefill_tokens=%d prefill_ms=%.3f prefill_toks_per_s=%.3f decode_tokens=%d "
                         "decode_ms=%.3f decode_toks_per_s=%.3f\n",
                         res.prompt_tokens, res.prefill_ms, res.prefill_tokens_per_second, res.completion_tokens, res.decode_ms,
                         res.decode_tokens_per_second);
    return results;
}

}  // namespace sandy
