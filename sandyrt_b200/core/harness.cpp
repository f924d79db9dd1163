#include "harness.h"

#include <algorithm>
#include <cstring>

namespace sandy {

namespace {
Json tensor_table(const TensorMap& t) {
    Json out = Json::object();
    for (const auto& kv : t) {
        Json e = Json::object();
        Json shape = Json::array();
        for (int64_t d : kv.second.shape) shape.push((long long)d);
        e["shape"] = shape;
        e["address"] = (long long)(uintptr_t)kv.second.data;
        out[kv.first] = e;
    }
    return out;
}
}  // namespace

PartHarness::PartHarness(const Json& args) {
    family_ = args.at("family").as_string();
    const std::string dt = args.find("dtype") ? args.at("dtype").as_string() : "float32";
    dtype_ = dt == "bfloat16" ? DType::BF16 : DType::F32;
    const uint64_t seed = args.find("seed") ? (uint64_t)args.at("seed").as_int() : 0;
    const PartSpec spec = part_spec_from_json(args.at("part"));
    part_ = get_part(family_, spec.kind).make(spec);
    part_tensors_ = random_tensors(part_->requests(), seed, StoreDType::F32);
    cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "creating a stream");
    if (family_ == "head") {
        auto* head = dynamic_cast<Head*>(part_.get());
        head->bind_head(part_tensors_, dtype_, nullptr);
    } else {
        part_->bind(part_tensors_, dtype_);
    }
    if (const Json* p = args.find("position")) {
        if (p->is_object()) {
            position_ = make_part<PositionEncoding>("position", part_spec_from_json(*p));
            position_tensors_ = random_tensors(position_->requests(), seed + 1, StoreDType::F32);
            position_->bind(position_tensors_, dtype_);
        }
    }
    std::vector<CacheSpec> specs;
    if (auto* m = dynamic_cast<Mixer*>(part_.get())) specs.push_back(m->cache_spec());
    const int page_size = args.find("page_size") ? (int)args.at("page_size").as_int() : 8;
    const int64_t max_tokens = args.find("max_tokens") ? args.at("max_tokens").as_int() : 512;
    const int max_requests = args.find("max_requests") ? (int)args.at("max_requests").as_int() : 8;
    cache_.reset(new CacheManager(specs, page_size, max_tokens, max_requests, dtype_, stream_));
    cache_->device().poison(stream_);
    status_ = DeviceBuffer(2 * sizeof(int));
    cuda_check(cudaMemset(status_.get(), 0, 2 * sizeof(int)), "clearing the status words");
    if (spec.params.find("width") && spec.params.at("width").is_int()) width_ = spec.params.at("width").as_int();
}

PartHarness::~PartHarness() {
    if (stream_) {
        cudaStreamSynchronize(stream_);
        cudaStreamDestroy(stream_);
    }
}

Json PartHarness::tensors() const {
    Json out = Json::object();
    out["part"] = tensor_table(part_tensors_);
    out["position"] = tensor_table(position_tensors_);
    return out;
}

Json PartHarness::info() const {
    Json out = Json::object();
    out["max_positions"] = (position_ && position_->max_positions()) ? Json((long long)*position_->max_positions()) : Json();
    out["weight_bytes"] = (long long)part_->weight_bytes();
    out["graph_safe"] = part_->graph_safe();
    return out;
}

void PartHarness::set_step(const std::vector<std::pair<int, int>>& seqs, const int* ids) {
    BlockAllocator& alloc = cache_->alloc();
    const int S = (int)seqs.size();
    std::vector<int> pos, seq, qs{0}, slots, before;
    for (int s = 0; s < S; s++) {
        if (!alloc.contains(s)) cache_->admit(s);
        else alloc.commit(s, seqs[(size_t)s].first);
        alloc.reserve(s, seqs[(size_t)s].first + seqs[(size_t)s].second);
        for (int i = 0; i < seqs[(size_t)s].second; i++) {
            pos.push_back(seqs[(size_t)s].first + i);
            seq.push_back(s);
        }
        qs.push_back(qs.back() + seqs[(size_t)s].second);
        slots.push_back(alloc.slot(s));
        before.push_back(seqs[(size_t)s].first);
    }
    const int T = (int)pos.size();
    int max_blocks = 1;
    const int G = alloc.n_groups();
    for (int g = 0; g < G; g++)
        for (int s = 0; s < S; s++) max_blocks = std::max(max_blocks, (int)alloc.block_list(s, g).size());
    std::vector<int> host;
    auto put = [&](const std::vector<int>& v) { const size_t at = host.size(); host.insert(host.end(), v.begin(), v.end()); return at; };
    std::vector<int> id_vec((size_t)T, 0);
    if (ids) std::copy(ids, ids + T, id_vec.begin());
    const size_t ids_at = put(id_vec), pos_at = put(pos), seq_at = put(seq), slot_at = put(slots), qs_at = put(qs), kvb_at = put(before);
    std::vector<size_t> table_at;
    for (int g = 0; g < G; g++) {
        std::vector<int> table((size_t)S * max_blocks, kFreed);
        for (int s = 0; s < S; s++) {
            const auto& bl = alloc.block_list(s, g);
            std::copy(bl.begin(), bl.end(), table.begin() + (size_t)s * max_blocks);
        }
        table_at.push_back(put(table));
    }
    cuda_check(cudaStreamSynchronize(stream_), "waiting for the last step");
    arrays_ = DeviceBuffer(host.size() * sizeof(int));
    cuda_check(cudaMemcpy(arrays_.get(), host.data(), host.size() * sizeof(int), cudaMemcpyHostToDevice), "copying the step's arrays");
    int* dev = (int*)arrays_.get();
    ctx_ = StepContext();
    ctx_.n_tokens = T;
    ctx_.n_seqs = S;
    ctx_.n_rows = 0;
    ctx_.token_ids = dev + ids_at;
    ctx_.positions = dev + pos_at;
    ctx_.token_seq = dev + seq_at;
    ctx_.seq_slots = dev + slot_at;
    ctx_.q_start = dev + qs_at;
    ctx_.kv_before = dev + kvb_at;
    ctx_.logit_rows = nullptr;
    for (size_t at : table_at) ctx_.block_tables.push_back(dev + at);
    ctx_.max_blocks = max_blocks;
    ctx_.compute_dtype = dtype_;
    ctx_.workspace = &workspace_;
    ctx_.caches = &cache_->device();
    ctx_.position = position_.get();
    for (int s = 0; s < S; s++) {
        ctx_.host_q_lens.push_back(seqs[(size_t)s].second);
        ctx_.host_kv_before.push_back(seqs[(size_t)s].first);
        ctx_.max_q_len = std::max(ctx_.max_q_len, seqs[(size_t)s].second);
        ctx_.max_kv_len = std::max(ctx_.max_kv_len, seqs[(size_t)s].first + seqs[(size_t)s].second);
    }
    ctx_.host_slots = slots;
    ctx_.launch.stream = stream_;
    ctx_.launch.status = (int*)status_.get();
    ctx_.launch.kernel_status = (int*)status_.get() + 1;
    have_step_ = true;
}

Tensor PartHarness::view(const void* p, int64_t rows, int64_t cols, DType dt) const {
    Tensor t;
    t.data = const_cast<void*>(p);
    t.dtype = dt;
    t.rows = rows;
    t.cols = cols;
    t.ld = cols;
    return t;
}

void PartHarness::run_norm(const void* x, int x_rows, void* out, int n_rows, const int* rows_host) {
    auto* norm = dynamic_cast<Norm*>(part_.get());
    if (!norm) throw ValueError("this part is not a norm");
    if (!have_step_) set_step({{0, std::max(x_rows, 1)}}, nullptr);
    DeviceBuffer rows_dev;
    const int* rows = nullptr;
    if (rows_host) {
        rows_dev = DeviceBuffer((size_t)n_rows * sizeof(int));
        cuda_check(cudaMemcpy(rows_dev.get(), rows_host, (size_t)n_rows * sizeof(int), cudaMemcpyHostToDevice), "copying rows");
        rows = (const int*)rows_dev.get();
    }
    Tensor xin = view(x, x_rows, width_, DType::F32), o = view(out, n_rows, width_, dtype_);
    norm->forward(ctx_, xin, o, rows, n_rows);
    cuda_check(cudaStreamSynchronize(stream_), "running a norm");
}

void PartHarness::run_feed_forward(const void* h, void* x) {
    auto* ff = dynamic_cast<FeedForward*>(part_.get());
    if (!ff) throw ValueError("this part is not a feed-forward");
    if (!have_step_) throw ValueError("set a step first");
    // the normed input is given: a norm that hands it over unchanged
    struct Given : Norm {
        Tensor t;
        Given(const PartSpec& s, Tensor t_) : Norm(s), t(t_) {}
        void forward(StepContext& ctx, const Tensor&, Tensor& out, const int*, int) override {
            cuda_check(cudaMemcpyAsync(out.data, t.data, (size_t)t.numel() * t.elem_size(), cudaMemcpyDeviceToDevice, ctx.launch.stream),
                       "copying the given input");
        }
    } given(part_->spec(), view(h, ctx_.n_tokens, width_, dtype_));
    Tensor xs = view(x, ctx_.n_tokens, width_, DType::F32);
    NormedInput in(ctx_, given, xs);
    ff->forward(ctx_, in, xs);
    cuda_check(cudaStreamSynchronize(stream_), "running a feed-forward");
}

void PartHarness::run_mixer(const void* h, void* x, bool write_cache) {
    auto* mixer = dynamic_cast<Mixer*>(part_.get());
    if (!mixer) throw ValueError("this part is not a mixer");
    if (!have_step_) throw ValueError("set a step first");
    struct Given : Norm {
        Tensor t;
        Given(const PartSpec& s, Tensor t_) : Norm(s), t(t_) {}
        void forward(StepContext& ctx, const Tensor&, Tensor& out, const int*, int) override {
            cuda_check(cudaMemcpyAsync(out.data, t.data, (size_t)t.numel() * t.elem_size(), cudaMemcpyDeviceToDevice, ctx.launch.stream),
                       "copying the given input");
        }
    } given(part_->spec(), view(h, ctx_.n_tokens, width_, dtype_));
    Tensor xs = view(x, ctx_.n_tokens, width_, DType::F32);
    NormedInput in(ctx_, given, xs);
    LayerCall call{0, 0, write_cache};
    mixer->forward(ctx_, in, xs, call);
    cuda_check(cudaStreamSynchronize(stream_), "running a mixer");
    int st[2] = {0, 0};
    cuda_check(cudaMemcpy(st, status_.get(), sizeof st, cudaMemcpyDeviceToHost), "reading the status words");
    if (st[0] || st[1]) throw KernelError("a kernel reported a fault (status " + std::to_string(st[0]) + ", " + std::to_string(st[1]) + ")");
}

void PartHarness::run_embedding(void* x) {
    auto* emb = dynamic_cast<Embedding*>(part_.get());
    if (!emb) throw ValueError("this part is not an embedding");
    if (!have_step_) throw ValueError("set a step first");
    Tensor xs = view(x, ctx_.n_tokens, width_, DType::F32);
    emb->forward(ctx_, xs);
    cuda_check(cudaStreamSynchronize(stream_), "running an embedding");
}

}  // namespace sandy
