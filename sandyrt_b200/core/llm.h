// LLM: the C++ entry point.  Model folder in, generated token ids out.
//
//     auto llm = sandy::LLM::load("path/to/model", options);
//     auto results = llm->generate({{15496, 11, 616, 1438, 318}}, params);
//     results[0].output_ids, results[0].finish_reason
//
// The calls mirror the reference's Model::load(ModelConfig) and Model::generate(requestId, inputIds,
// maxTokens, stopTokenIds, samplingOverrides, control, onToken) -> GenerateResult
// (src/server/Model.h:34-48) and its GenerateResult fields (src/server/Session.h:25-34): output ids,
// finish reason, prompt and completion token counts, prefill and decode times and rates.  Unlike the
// reference, which serves one request at a time behind a gate, all requests given to `generate` (or
// added with `add_request`) run together under the scheduler:
//
//     id = add_request(prompt, ...);  while (has_work()) for (auto& [rid, token] : step()) ...;  result(id)
//
// Tokens go in and come out as host integers; every step copies its inputs to the device and reads
// the drawn tokens back.
//
// Decode bursts: when every running request is decoding, up to `max_burst` decode steps run back to
// back on the device per look of the host (Engine::decode_burst_async).  Bursts are queued ahead:
// while burst k runs, burst k+1 of the same requests is queued behind it and only then are burst k's
// tokens read, so scheduling, packing and read-back do not leave the device idle.  A request that
// stopped inside burst k has wasted rows in burst k+1, nothing more.
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "engine.h"
#include "scheduler.h"

namespace sandy {

// Fields of the reference's GenerateResult (src/server/Session.h:25-34).
struct GenerateResult {
    std::vector<int> output_ids;
    std::string finish_reason;
    int prompt_tokens = 0;
    int completion_tokens = 0;
    double prefill_ms = 0.0, decode_ms = 0.0;
    double prefill_tokens_per_second = 0.0, decode_tokens_per_second = 0.0;
    int preemptions = 0;
};

struct LLMOptions {
    DType dtype = DType::BF16;
    int device = 0;
    int64_t cache_tokens = 0;            // tokens the cache pool holds (0: room for `max_live` requests of full length, capped at 1M)
    int page_size = 16;
    int max_live = 64;                   // most requests live at once
    int max_step_tokens = 2048;          // token budget of one step
    int prefill_chunk_tokens = 2048;
    std::vector<int> eos_token_ids;      // stop tokens added to every request (the config's eos_token_id is NOT added by itself)
    int max_context_tokens = 0;          // if > 0, a lower limit on a request's length than the model's
    bool use_cuda_graphs = true;
    int max_burst = 8;                   // most decode steps run on the device between two looks of the host
    bool pipeline_bursts = true;         // queue the next burst before the tokens of the last one have been read
};

struct GenerateParams {
    int max_tokens = 16;
    float temperature = 0.0f;
    float top_p = 1.0f;
    int top_k = 0;
    std::optional<uint64_t> seed;        // request i draws with seed + i
    std::vector<int> stop_token_ids;
    // called with (request index, token) for every new token; returning false cancels that request
    // (finish reason "cancelled"; the reference fails the request with "request cancelled",
    // src/server/Session.cpp:491-492)
    std::function<bool(int, int)> on_token;
    bool report = false;                 // print the reference's throughput line per request to stderr
};

class LLM {
public:
    static std::unique_ptr<LLM> load(const std::string& model_dir, const LLMOptions& options = {});
    LLM(std::unique_ptr<Model> model, const LLMOptions& options);

    RequestId add_request(const std::vector<int>& prompt_ids, int max_tokens = 16, const SamplingParams& sampling = {},
                          const std::vector<int>& stop_token_ids = {});
    bool has_work() const { return scheduler_->has_work() || inflight_; }
    // Plan and run one step (or, when every request is decoding, a burst of steps on the device).
    // Returns (request, token) for every token drawn, in order.
    std::vector<std::pair<RequestId, int>> step();
    std::vector<std::pair<RequestId, int>> drain();       // read the bursts still queued, queue nothing new
    bool finished(RequestId rid) const;
    GenerateResult result(RequestId rid) const;
    const Request& request(RequestId rid) const;
    void forget(RequestId rid);
    void abort(RequestId rid);
    std::vector<GenerateResult> generate(const std::vector<std::vector<int>>& prompts, const GenerateParams& params = {});

    Engine& engine() { return *engine_; }
    Scheduler& scheduler() { return *scheduler_; }
    Model& model() { return *model_; }
    int max_burst() const { return max_burst_; }
    bool pipeline_bursts() const { return opt_.pipeline_bursts; }
    long long decode_steps_run = 0, bursts_queued_ahead = 0;

private:
    struct Inflight { BurstHandle handle; std::vector<RequestPtr> reqs; };
    int burst_length(const StepPlan& plan) const;
    int steps_possible(const std::vector<RequestPtr>& reqs, int in_flight) const;
    BurstHandle queue_burst(const std::vector<RequestPtr>& reqs, int n, int in_flight);
    std::vector<std::pair<RequestId, int>> collect_burst(const BurstHandle& handle, const std::vector<RequestPtr>& reqs);
    std::vector<std::pair<RequestId, int>> advance();
    RequestPtr find(RequestId rid) const;

    LLMOptions opt_;
    std::unique_ptr<Model> model_;
    std::unique_ptr<Engine> engine_;
    std::unique_ptr<Scheduler> scheduler_;
    std::optional<int> max_positions_;
    int max_burst_ = 1;
    std::unique_ptr<Inflight> inflight_;
    std::unordered_map<RequestId, RequestPtr> requests_;
    RequestId next_id_ = 1;
};

}  // namespace sandy
