#include "engine.h"

#include <algorithm>
#include <cstring>
#include <set>

#include "kernels.h"

namespace sandy {

namespace {
size_t next_pow2(size_t n) {
    size_t p = 1;
    while (p < n) p <<= 1;
    return p;
}
}  // namespace

// A ring of pinned host buffers and ONE device buffer for the step's index arrays.  The device
// buffer keeps its address for the engine's lifetime unless a step outgrows it.
struct Engine::Staging {
    static constexpr int kDepth = 4;
    size_t capacity = 0;            // in ints
    PinnedBuffer host[kDepth];
    cudaEvent_t events[kDepth] = {nullptr, nullptr, nullptr, nullptr};
    bool used[kDepth] = {false, false, false, false};
    DeviceBuffer dev;
    int turn = 0;
    long long generation = 0;

    explicit Staging(size_t cap) {
        for (auto& e : events) cuda_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "creating an event");
        allocate(cap);
    }
    ~Staging() {
        for (auto& e : events)
            if (e) cudaEventDestroy(e);
    }
    void allocate(size_t cap) {
        capacity = cap;
        for (int i = 0; i < kDepth; i++) {
            if (used[i]) cudaEventSynchronize(events[i]);
            host[i] = PinnedBuffer(cap * sizeof(int));
            used[i] = false;
        }
        dev = DeviceBuffer(cap * sizeof(int));
        generation++;
    }
    int acquire(size_t n) {
        if (n > capacity) allocate(next_pow2(n));
        const int i = turn;
        turn = (turn + 1) % kDepth;
        if (used[i]) cuda_check(cudaEventSynchronize(events[i]), "waiting for a staging copy");    // the copy that last used this buffer is done
        return i;
    }
    // Copy elements [start, n) of host buffer i to the same place of the device buffer.
    void send(int i, size_t n, size_t start, cudaStream_t stream) {
        if (n > start)
            cuda_check(cudaMemcpyAsync((int*)dev.get() + start, (int*)host[i].get() + start, (n - start) * sizeof(int),
                                       cudaMemcpyHostToDevice, stream),
                       "copying the step's arrays");
        cuda_check(cudaEventRecord(events[i], stream), "recording an event");
        used[i] = true;
    }
};

Engine::Engine(Model& model, const Options& options) : model_(model), opt_(options) {
    if (!model.bound()) throw StepError("the model has no weights bound");
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0)
        throw StepError("the engine runs on a CUDA device only; there is no CPU path");
    dtype_ = model.compute_dtype();
    vocab_ = model.spec().vocab_size;
    cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "creating the engine's stream");
    cache_.reset(new CacheManager(model.cache_specs(), opt_.page_size, opt_.max_tokens, opt_.max_requests, dtype_, stream_));
    const long long positions = model.max_positions() ? *model.max_positions() : opt_.max_tokens;
    const long long blocks_cap = (((positions + opt_.page_size - 1) / opt_.page_size + 8) + 31) / 32 * 32;
    const size_t cap = 4 * (size_t)opt_.max_step_tokens + 3 * (size_t)opt_.max_requests + 1 +
                       (5 + kMaxBurst) * (size_t)opt_.max_requests +
                       cache_->layout().groups.size() * (size_t)opt_.max_requests * (size_t)blocks_cap;
    staging_.reset(new Staging(next_pow2(cap)));
    const size_t reqs = (size_t)std::max(opt_.max_requests, 1);
    status_ = DeviceBuffer(2 * sizeof(int));
    cuda_check(cudaMemset(status_.get(), 0, 2 * sizeof(int)), "clearing the status words");
    sampled_ = DeviceBuffer(reqs * sizeof(int));
    burst_tokens_ = DeviceBuffer(kMaxBurst * reqs * sizeof(int));
    // two pinned buffers: the tokens of one burst are read while the next one runs
    for (int i = 0; i < 2; i++) {
        burst_hosts_[i] = PinnedBuffer((kMaxBurst * reqs + 2) * sizeof(int));
        cuda_check(cudaEventCreateWithFlags(&burst_done_[i], cudaEventDisableTiming), "creating an event");
    }
    token_host_ = PinnedBuffer((reqs + 2) * sizeof(int));
    use_graphs_ = opt_.use_cuda_graphs && model.graph_safe();
}

Engine::~Engine() {
    if (stream_) cudaStreamSynchronize(stream_);
    for (auto& kv : graphs_)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    for (auto& e : burst_done_)
        if (e) cudaEventDestroy(e);
    staging_.reset();
    cache_.reset();
    if (stream_) cudaStreamDestroy(stream_);
}

void Engine::synchronize() { cuda_check(cudaStreamSynchronize(stream_), "waiting for the engine's stream"); }

// ---- packing a step ------------------------------------------------------------------------------------
Engine::Prepared Engine::prepare(const std::vector<StepEntry>& entries, const std::vector<SampleRow>* sampling,
                                 const float* burst_uniform, int n_burst, int in_flight) {
    BlockAllocator& alloc = cache_->alloc();
    if (entries.empty()) throw StepError("a step needs at least one token");
    const int extra = std::max(n_burst - 1, 0);          // positions a burst adds beyond this step's
    const int S = (int)entries.size();
    std::set<RequestId> seen;
    std::vector<int> q_lens, kv_before, slots;
    const std::optional<int64_t> limit = model_.max_positions();
    for (const StepEntry& e : entries) {
        if (!seen.insert(e.rid).second) throw StepError("request " + std::to_string(e.rid) + " appears twice in one step");
        if (!alloc.contains(e.rid)) admit(e.rid);
        const int before = alloc.length(e.rid) + in_flight;
        const int n = (int)e.tokens.size();
        if (limit && before + n + extra > *limit)
            throw StepError("request " + std::to_string(e.rid) + ": " + std::to_string(before + n + extra) +
                            " tokens exceed the model's " + std::to_string(*limit) + " positions");
        q_lens.push_back(n);
        kv_before.push_back(before);
        slots.push_back(alloc.slot(e.rid));
    }
    // all-or-nothing page reservation for the whole step (or burst)
    std::vector<int> need((size_t)alloc.n_groups(), 0);
    for (int s = 0; s < S; s++) {
        const std::vector<int> k = alloc.pages_needed(entries[(size_t)s].rid, kv_before[(size_t)s] + q_lens[(size_t)s] + extra);
        for (size_t g = 0; g < k.size(); g++) need[g] += k[g];
    }
    for (size_t g = 0; g < need.size(); g++)
        if (need[g] > alloc.free_pages((int)g))
            throw OutOfPages("step needs " + std::to_string(need[g]) + " new pages in cache group " + std::to_string(g) + ", " +
                             std::to_string(alloc.free_pages((int)g)) + " of " + std::to_string(alloc.pool((int)g).num_pages()) + " are free");
    for (int s = 0; s < S; s++) alloc.reserve(entries[(size_t)s].rid, kv_before[(size_t)s] + q_lens[(size_t)s] + extra);

    int T = 0, R = 0, max_q = 0, max_kv = 0;
    for (int s = 0; s < S; s++) {
        T += q_lens[(size_t)s];
        R += (int)entries[(size_t)s].want.size();
        max_q = std::max(max_q, q_lens[(size_t)s]);
        max_kv = std::max(max_kv, kv_before[(size_t)s] + q_lens[(size_t)s]);
    }
    if (sampling && (int)sampling->size() != R)
        throw StepError(std::to_string(sampling->size()) + " sampling rows for " + std::to_string(R) + " wanted places");
    const auto& groups = cache_->layout().groups;
    const bool decode_only = max_q == 1;
    if (n_burst && (!decode_only || R != S || !sampling))
        throw StepError("a burst takes single tokens only, each with its logits wanted and sampled");
    if (in_flight && !n_burst) throw StepError("only a burst can continue a burst");
    const long long generation = staging_->generation;
    const int page = cache_->page_size();
    int max_blocks = 0;
    for (int s = 0; s < S; s++) max_blocks = std::max(max_blocks, (kv_before[(size_t)s] + q_lens[(size_t)s] + extra + page - 1) / page);
    // widths in steps of 8 pages (32 for bursts, whose recordings are dearer): few distinct graphs
    const int grain = n_burst ? 32 : 8;
    max_blocks = std::max(8, (max_blocks + grain - 1) / grain * grain);
    const size_t n_sample = (sampling ? 4 * (size_t)R : 0) + (n_burst ? (size_t)R + (size_t)n_burst * R : 0);
    const size_t total = 3 * (size_t)T + S + (S + 1) + S + R + n_sample + groups.size() * (size_t)S * max_blocks;
    const int bi = staging_->acquire(total);
    int* h = (int*)staging_->host[bi].get();
    int* dev = (int*)staging_->dev.get();
    size_t off = 0;
    auto take = [&](size_t n) { const size_t at = off; off += n; return at; };
    const size_t ids_at = take(T), pos_at = take(T), seq_at = take(T), slot_at = take(S), qs_at = take(S + 1), kvb_at = take(S),
                 rows_at = take(R);
    int t0 = 0, r0 = 0;
    for (int s = 0; s < S; s++) {
        const StepEntry& e = entries[(size_t)s];
        const int n = q_lens[(size_t)s], before = kv_before[(size_t)s];
        for (int i = 0; i < n; i++) {
            const int tok = e.tokens[(size_t)i];
            if (!in_flight && (tok < 0 || tok >= vocab_))
                throw StepError("request " + std::to_string(e.rid) + ": a token id is outside the vocabulary of " + std::to_string(vocab_));
            h[ids_at + t0 + i] = tok;
            h[pos_at + t0 + i] = before + i;
            h[seq_at + t0 + i] = s;
        }
        h[qs_at + s] = t0;
        for (int w : e.want) {
            if (w < 0 || w >= n)
                throw StepError("request " + std::to_string(e.rid) + ": wanted place " + std::to_string(w) + " is outside its " +
                                std::to_string(n) + " tokens");
            h[rows_at + r0++] = t0 + w;
        }
        h[slot_at + s] = slots[(size_t)s];
        h[kvb_at + s] = before;
        t0 += n;
    }
    h[qs_at + S] = T;
    size_t sample_at = 0, step_at = 0, uni_at = 0;
    if (sampling) {
        sample_at = take(4 * (size_t)R);
        float* f = reinterpret_cast<float*>(h + sample_at);
        for (int r = 0; r < R; r++) {
            const SampleRow& row = (*sampling)[(size_t)r];
            f[r] = row.temperature;
            h[sample_at + R + r] = row.top_k;
            f[2 * R + r] = row.top_p;
            f[3 * R + r] = row.uniform;
        }
    }
    if (n_burst) {
        step_at = take(R);
        for (int r = 0; r < R; r++) h[step_at + r] = 0;
    }
    std::vector<size_t> table_at;
    for (const auto& g : groups) {
        const size_t at = take((size_t)S * max_blocks);
        table_at.push_back(at);
        for (int s = 0; s < S; s++) {
            const std::vector<int>& row = alloc.block_list(entries[(size_t)s].rid, g.index);
            const int m = std::min((int)row.size(), max_blocks);
            int* dst = h + at + (size_t)s * max_blocks;
            std::memcpy(dst, row.data(), (size_t)m * sizeof(int));
            for (int b = m; b < max_blocks; b++) dst[b] = kFreed;
        }
    }
    if (n_burst) {
        // last in the buffer: its length changes with the burst, nothing else may move with it
        uni_at = take((size_t)n_burst * R);
        std::memcpy(h + uni_at, burst_uniform, (size_t)n_burst * R * sizeof(float));
    }
    if (in_flight && staging_->generation != generation) throw StepError("the step buffer moved under a running burst");
    staging_->send(bi, total, in_flight ? (size_t)T : 0, stream_);
    last_h2d_bytes = (int)(4 * (total - (in_flight ? (size_t)T : 0)));
    h2d_bytes_total += last_h2d_bytes;

    Prepared p;
    StepContext& c = p.ctx;
    c.n_tokens = T;
    c.n_seqs = S;
    c.n_rows = R;
    c.token_ids = dev + ids_at;
    c.positions = dev + pos_at;
    c.token_seq = dev + seq_at;
    c.seq_slots = dev + slot_at;
    c.q_start = dev + qs_at;
    c.kv_before = dev + kvb_at;
    c.logit_rows = dev + rows_at;
    for (size_t at : table_at) c.block_tables.push_back(dev + at);
    c.max_blocks = max_blocks;
    c.compute_dtype = dtype_;
    c.workspace = &workspace_;
    c.caches = &cache_->device();
    c.host_q_lens = q_lens;
    c.host_kv_before = kv_before;
    c.host_slots = slots;
    c.max_q_len = max_q;
    c.max_kv_len = max_kv + extra;
    c.launch.stream = stream_;
    c.launch.status = (int*)status_.get();
    c.launch.kernel_status = (int*)status_.get() + 1;
    p.sample = sampling ? dev + sample_at : nullptr;
    p.n_burst = n_burst;
    if (n_burst) {
        p.burst_uniform = reinterpret_cast<float*>(dev + uni_at);
        p.row_step = dev + step_at;
        burst_flip_ ^= 1;
    }
    // Everything a launch's shape depends on.  The portions' own lengths and starts are device data
    // (q_start, kv_before, positions), so steps that agree on these counts share a graph: decode
    // steps always do, prompt steps do when the token budget is filled the same way.  A burst is
    // recorded whole (all its steps in one graph), in two copies used in turn: a graph that is
    // launched again while it still runs makes the host wait for it.
    p.key = Key{T, S, R, max_q, max_blocks, sampling ? 1 : 0, n_burst, n_burst ? burst_flip_ : 0, staging_->generation};
    return p;
}

// ---- running it ---------------------------------------------------------------------------------------------
Tensor Engine::run(Prepared& p) {
    StepContext& ctx = p.ctx;
    Tensor logits = model_.forward(ctx);
    const int R = ctx.n_rows;
    if (p.sample && R) {
        const float* f = reinterpret_cast<const float*>(p.sample);
        if (p.n_burst) {
            ops::SampleFeedback fb;
            fb.token_ids = ctx.token_ids;
            fb.logit_rows = ctx.logit_rows;
            fb.positions = ctx.positions;
            fb.burst_tokens = (int*)burst_tokens_.get();
            fb.row_step = p.row_step;
            ops::sample(ctx.launch, logits, (int*)sampled_.get(), f, p.sample + R, f + 2 * R, p.burst_uniform, &fb);
        } else {
            ops::sample(ctx.launch, logits, (int*)sampled_.get(), f, p.sample + R, f + 2 * R, f + 3 * R, nullptr);
        }
    }
    return logits;
}

void Engine::drop_graph(const Key& key) {
    auto it = graphs_.find(key);
    if (it == graphs_.end()) return;
    if (it->second.exec) cudaGraphExecDestroy(it->second.exec);
    graphs_.erase(it);
    graph_order_.erase(std::remove(graph_order_.begin(), graph_order_.end(), key), graph_order_.end());
}

// The valid recorded graph of `key`, or null; counts how often the key came by and says whether this
// is the time to record it.
Engine::Graph* Engine::graph_for(const Key& key, int record_at, bool& record) {
    record = false;
    auto it = graphs_.find(key);
    if (it != graphs_.end() && it->second.ws_version != workspace_.version()) {
        // a workspace buffer has moved since this graph was recorded: its pointers are stale
        drop_graph(key);
        seen_.erase(key);
        stale_graphs++;
        it = graphs_.end();
    }
    if (it != graphs_.end()) return &it->second;
    int& seen = seen_[key];
    record = seen >= record_at;
    seen++;
    return nullptr;
}

Engine::Graph* Engine::record(const Key& key, Prepared& p, int times) {
    const long long before = g_launches;
    const uint64_t ws_before = workspace_.version();
    cuda_check(cudaStreamSynchronize(stream_), "waiting before a recording");
    cuda_check(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "beginning a graph capture");
    Tensor logits;
    cudaGraph_t graph = nullptr;
    try {
        for (int i = 0; i < times; i++) logits = run(p);
    } catch (...) {
        cudaStreamEndCapture(stream_, &graph);
        if (graph) cudaGraphDestroy(graph);
        throw;
    }
    cuda_check(cudaStreamEndCapture(stream_, &graph), "ending a graph capture");
    if (workspace_.version() != ws_before) {
        // a buffer was (re)allocated while recording: what was recorded is not to be trusted
        cudaGraphDestroy(graph);
        return nullptr;
    }
    Graph g;
    const cudaError_t e = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    cuda_check(e, "instantiating a graph");
    g.logits = logits;
    g.launches = (int)((g_launches - before) / times);
    g.ws_version = workspace_.version();
    while ((int)graphs_.size() >= kMaxGraphs) {          // the oldest recording makes room
        drop_graph(graph_order_.front());
        seen_.clear();
    }
    graphs_[key] = g;
    graph_order_.push_back(key);
    if (times > 1) burst_graphs_recorded++;
    return &graphs_[key];
}

// Run the prepared step `times` times (more than once only for a burst, whose sampler moves the
// step's inputs on), through recorded graphs where there are any.
//
// Two kinds of recordings.  One step: recorded the second time its shape comes by, replayed `times`
// times for a burst.  A whole burst (all its steps in one graph, one launch): recorded once the same
// burst shape has come by three times, so that only workloads that stay in one shape pay for it;
// kept in two copies used in turn (the key carries the turn), because a graph launched again while
// it still runs makes the host wait for it, and the host has the next burst to prepare.
Tensor Engine::execute(Prepared& p, int times) {
    const long long before = g_launches;
    auto eager = [&]() {
        Tensor logits;
        for (int i = 0; i < times; i++) logits = run(p);
        last_launches = (int)((g_launches - before) / times);
        return logits;
    };
    if (!use_graphs_) return eager();
    Key step_key = p.key;
    bool rec = false;
    if (p.n_burst) {
        step_key[6] = 1;                    // any burst length, either turn
        step_key[7] = 0;
        Graph* hit = graph_for(p.key, 2, rec);
        if (!hit && rec) hit = record(p.key, p, times);
        if (hit) {
            cuda_check(cudaGraphLaunch(hit->exec, stream_), "launching a recorded burst");
            graph_replays += times;
            last_launches = hit->launches;
            return hit->logits;
        }
    }
    Graph* hit = graph_for(step_key, 1, rec);
    if (!hit && rec) hit = record(step_key, p, 1);
    if (hit) {
        for (int i = 0; i < times; i++) cuda_check(cudaGraphLaunch(hit->exec, stream_), "launching a recorded step");
        graph_replays += times;
        last_launches = hit->launches;
        return hit->logits;
    }
    return eager();
}

Tensor Engine::step(const std::vector<StepEntry>& all, const std::vector<SampleRow>* sampling) {
    std::vector<StepEntry> entries;
    for (const StepEntry& e : all)
        if (!e.tokens.empty()) entries.push_back(e);
    Prepared p = prepare(entries, sampling, nullptr, 0, 0);
    const size_t R = (size_t)p.ctx.n_rows;
    if (sampled_.bytes() < R * sizeof(int)) {
        synchronize();
        sampled_ = DeviceBuffer(next_pow2(R) * sizeof(int));
        for (auto& kv : graphs_)
            if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);    // recorded graphs hold the old address
        graphs_.clear();
        graph_order_.clear();
        seen_.clear();
    }
    Tensor logits = execute(p, 1);
    for (size_t s = 0; s < entries.size(); s++)
        cache_->alloc().commit(entries[s].rid, p.ctx.host_kv_before[s] + p.ctx.host_q_lens[s]);
    steps_run++;
    return logits;
}

BurstHandle Engine::decode_burst_async(const std::vector<StepEntry>& entries, const std::vector<SampleRow>& sampling,
                                       const std::vector<float>& uniforms, int n, int in_flight) {
    const int S = (int)entries.size();
    if (n < 1 || n > kMaxBurst) throw StepError("a burst runs 1 to " + std::to_string(kMaxBurst) + " steps, got " + std::to_string(n));
    if ((size_t)n * S * sizeof(int) > burst_tokens_.bytes()) throw StepError("more requests in a burst than the engine was built for");
    if (uniforms.size() != (size_t)n * S) throw StepError("a burst needs one uniform number per step and request");
    Prepared p = prepare(entries, &sampling, uniforms.data(), n, in_flight);
    execute(p, n);
    const int turn = burst_turn_;
    burst_turn_ ^= 1;
    int* host = (int*)burst_hosts_[turn].get();
    cuda_check(cudaMemcpyAsync(host, burst_tokens_.get(), (size_t)n * S * sizeof(int), cudaMemcpyDeviceToHost, stream_),
               "copying a burst's tokens to the host");
    copy_status(host + (size_t)n * S);
    d2h_bytes_total += 4LL * n * S + 8;
    cuda_check(cudaEventRecord(burst_done_[turn], stream_), "recording an event");
    steps_run += n;
    BurstHandle hnd;
    hnd.n = n;
    hnd.S = S;
    hnd.host = host;
    hnd.done = burst_done_[turn];
    return hnd;
}

// Queue a copy of the two status words (bad input, kernel faults) behind whatever the stream holds:
// they travel with the drawn tokens, at no extra wait.
void Engine::copy_status(int* host_at) {
    cuda_check(cudaMemcpyAsync(host_at, status_.get(), 2 * sizeof(int), cudaMemcpyDeviceToHost, stream_), "copying the status words");
}

std::vector<int> Engine::burst_tokens(const BurstHandle& handle) {
    cuda_check(cudaEventSynchronize(handle.done), "waiting for a burst");
    const size_t n = (size_t)handle.n * handle.S;
    if (handle.host[n] || handle.host[n + 1]) check_status();
    return std::vector<int>(handle.host, handle.host + n);
}

std::vector<int> Engine::read_sampled(int n) {
    if (token_host_.bytes() < ((size_t)n + 2) * sizeof(int)) token_host_ = PinnedBuffer(((size_t)n + 2) * sizeof(int));
    int* host = (int*)token_host_.get();
    if (n) cuda_check(cudaMemcpyAsync(host, sampled_.get(), (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, stream_), "copying drawn tokens");
    copy_status(host + n);
    d2h_bytes_total += 4LL * n + 8;
    synchronize();
    if (host[n] || host[n + 1]) check_status();
    return std::vector<int>(host, host + n);
}

void Engine::check_status() {
    int host[2] = {0, 0};
    cuda_check(cudaMemcpyAsync(host, status_.get(), sizeof host, cudaMemcpyDeviceToHost, stream_), "reading the status words");
    synchronize();
    if (host[0] || host[1]) {
        cuda_check(cudaMemsetAsync(status_.get(), 0, sizeof host, stream_), "clearing the status words");
        synchronize();
    }
    if (host[0])
        throw StepError("a kernel reported bad input (status " + std::to_string(host[0]) +
                        ": bit 0 token id or NaN logits, bit 1 position)");
    if (host[1])
        throw KernelError("a kernel reported a fault (status " + std::to_string(host[1]) + ": " + ops::kernel_status_text() +
                          "); the step's output is not valid");
}

}  // namespace sandy
