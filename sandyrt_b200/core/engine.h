// The step function: one batch of (request, its next tokens) through the model.
//
// `Engine::step(entries)` takes, for each request of the step, the tokens that follow what the
// request already has in the cache (a portion of a prompt of any length, or one decoded token) and
// the places among them whose logits are wanted.  It runs exactly those tokens as one batch, reading
// everything earlier from the cache, appends their keys and values to the cache, and returns float32
// logits [wanted, vocab] in the order of the entries and of their wanted places.  With `sampling` it
// also draws one token per wanted row on the device.
//
// The reference's counterpart, Engine::runValues on one of two compiled graphs (decode with input_id
// [1,1], prefill with input_id [1,n]; src/engine/Engine.h:100-104, src/server/Model.cpp:216-255,
// inputs built in src/server/Session.cpp:167-206), serves one request per call, returns logits for
// every row and samples on the host.  Here there is one code path for every mix of requests, and
// rows nobody asked for are never computed past the last layer.
//
// All the step's index arrays (token ids, positions, request of each token, block tables, wanted
// rows, sampling options) are packed on the host into one pinned buffer (a ring of four) and reach
// the device with one copy into ONE device buffer with a fixed address.  Every step shape that comes
// by a second time (tokens, requests, wanted rows, longest portion, block-table width, sampling,
// burst) is recorded as a CUDA graph and replayed from then on, prompt steps included (portion
// starts and lengths are device data); a graph is dropped when a workspace buffer has moved since it
// was recorded, at most 64 are kept.
//
// `decode_burst_async` runs several decode steps of the same requests with no trip to the host in
// between: the sampler writes each drawn token over the step's input token and moves the position
// on, so the same recorded graph is simply replayed n times (or the whole burst is one graph);
// pages for all n steps are reserved beforehand and the drawn tokens of all steps come back in one
// copy, with the two status words behind them.
//
// Everything runs on the engine's own stream.
#pragma once

#include <array>
#include <deque>
#include <map>
#include <memory>
#include <vector>

#include "cache.h"
#include "device.h"
#include "model.h"

namespace sandy {

constexpr int kMaxBurst = 32;      // most decode steps one burst may run
constexpr int kMaxGraphs = 64;     // most recorded step shapes kept at a time

// One request's share of a step.
struct StepEntry {
    RequestId rid = 0;
    std::vector<int> tokens;
    std::vector<int> want;         // indices into `tokens` whose logits are returned
};

// How the token of one wanted row is drawn (see SamplingParams).
struct SampleRow {
    float temperature = 0.0f;
    int top_k = 0;
    float top_p = 1.0f;
    float uniform = 0.0f;
};

// A burst of decode steps queued on the device.
struct BurstHandle {
    int n = 0;                     // steps
    int S = 0;                     // requests
    const int* host = nullptr;     // pinned buffer the tokens are copied to; the two status words follow them
    cudaEvent_t done = nullptr;    // recorded behind that copy (owned by the engine)
};

class Engine {
public:
    struct Options {
        int64_t max_tokens = 0;          // tokens the cache pool holds
        int page_size = 16;
        int max_requests = 64;
        int max_step_tokens = 2048;
        bool use_cuda_graphs = true;
    };
    Engine(Model& model, const Options& options);
    ~Engine();
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    // ---- request lifetime
    int admit(RequestId rid) { return cache_->admit(rid); }
    void release(RequestId rid) { cache_->release(rid); }
    int length(RequestId rid) const { return cache_->alloc().length(rid); }
    void commit(RequestId rid, int new_len) { cache_->alloc().commit(rid, new_len); }   // after a burst

    // ---- running
    // Runs one step; the logits are workspace memory on the device: the next step overwrites them.
    // They are complete once the engine's stream has passed (synchronize()).  With `sampling` (one
    // SampleRow per wanted place) the drawn tokens are read with read_sampled().
    Tensor step(const std::vector<StepEntry>& entries, const std::vector<SampleRow>* sampling = nullptr);
    // The tokens drawn by the last step with `sampling`, on the host.  The step's status words come
    // back in the same wait; a non-zero one throws (the tokens are not valid then).
    std::vector<int> read_sampled(int n);
    // Queue n = uniforms.size() / requests decode steps of the same requests back to back.  Every
    // entry brings one token and wants its logits; step j of request r is drawn with sampling[r] and
    // uniforms[j * S + r]; the token drawn in step j is the input of step j + 1.  Pages for all n steps
    // are reserved before anything runs (OutOfPages otherwise, with nothing taken).  The requests'
    // lengths are NOT advanced: the caller commits as many of each request's steps as it keeps.
    // With `in_flight` > 0 the burst continues one of the same requests, in the same order, that was
    // queued before and is `in_flight` steps long: the token ids are not sent (they are where the
    // sampler left them), so the host can queue the next burst before it has seen the tokens of the last.
    BurstHandle decode_burst_async(const std::vector<StepEntry>& entries, const std::vector<SampleRow>& sampling,
                                   const std::vector<float>& uniforms, int n_steps, int in_flight = 0);
    // Wait for a queued burst; its tokens, [n][requests].  Throws if a kernel of the burst reported a fault.
    std::vector<int> burst_tokens(const BurstHandle& handle);
    void check_status();               // throws if a kernel reported bad input or an expired wait since the last check
    void synchronize();
    cudaStream_t stream() const { return stream_; }

    Model& model() { return model_; }
    CacheManager& cache() { return *cache_; }
    bool use_cuda_graphs() const { return use_graphs_; }
    DType dtype() const { return dtype_; }
    const Options& options() const { return opt_; }

    // counters
    long long steps_run = 0, graph_replays = 0, stale_graphs = 0, burst_graphs_recorded = 0;
    long long h2d_bytes_total = 0, d2h_bytes_total = 0;
    int last_h2d_bytes = 0, last_launches = 0;
    size_t recorded_graphs() const { return graphs_.size(); }

private:
    using Key = std::array<long long, 9>;
    struct Prepared {
        StepContext ctx;
        int* sample = nullptr;             // device: [temperature R | top_k R | top_p R | uniform R]
        float* burst_uniform = nullptr;    // device: [n, R]
        int* row_step = nullptr;           // device: [R]
        int n_burst = 0;
        Key key{};
    };
    struct Graph {
        cudaGraphExec_t exec = nullptr;
        Tensor logits;
        int launches = 0;
        uint64_t ws_version = 0;
    };
    struct Staging;
    Prepared prepare(const std::vector<StepEntry>& entries, const std::vector<SampleRow>* sampling,
                     const float* burst_uniform, int n_burst, int in_flight);
    Tensor run(Prepared& p);
    Tensor execute(Prepared& p, int times);
    Graph* graph_for(const Key& key, int record_at, bool& record);
    Graph* record(const Key& key, Prepared& p, int times);
    void drop_graph(const Key& key);
    void copy_status(int* host_at);

    Model& model_;
    Options opt_;
    DType dtype_;
    int64_t vocab_;
    cudaStream_t stream_ = nullptr;
    std::unique_ptr<CacheManager> cache_;
    Workspace workspace_;
    std::unique_ptr<Staging> staging_;
    DeviceBuffer status_;                  // [0] bad input, [1] kernel faults
    DeviceBuffer sampled_;
    DeviceBuffer burst_tokens_;
    PinnedBuffer burst_hosts_[2];
    cudaEvent_t burst_done_[2] = {nullptr, nullptr};
    PinnedBuffer token_host_;
    int burst_turn_ = 0, burst_flip_ = 0;
    bool use_graphs_ = true;
    std::map<Key, Graph> graphs_;
    std::deque<Key> graph_order_;
    std::map<Key, int> seen_;
};

}  // namespace sandy
