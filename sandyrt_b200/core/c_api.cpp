#include "c_api.h"

#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <string>

#include "config.h"
#include "engine.h"
#include "errors.h"
#include "foreign.h"
#include "harness.h"
#include "json.h"
#include "kernels.h"
#include "llm.h"
#include "model.h"
#include "scheduler.h"
#include "weights.h"

using namespace sandy;

namespace {

thread_local std::string t_kind, t_message, t_details, t_result;

void set_error(const std::string& kind, const std::string& message, const std::string& details = "") {
    t_kind = kind;
    t_message = message;
    t_details = details;
}

template <typename F>
auto guarded(F&& f, decltype(f()) failure) -> decltype(f()) {
    try {
        return f();
    } catch (const Error& e) {
        set_error(e.kind(), e.what(), e.details());
    } catch (const std::bad_alloc&) {
        set_error("MemoryError", "out of host memory");
    } catch (const std::exception& e) {
        set_error("RuntimeError", e.what());
    } catch (...) {
        set_error("RuntimeError", "unknown error");
    }
    return failure;
}

// ---- objects behind handles ---------------------------------------------------------------------------
struct AllocatorBox {
    std::unique_ptr<BlockAllocator> owned;
    BlockAllocator* alloc = nullptr;          // owned, or borrowed from an engine
};
struct PoolBox {
    std::unique_ptr<PagePool> pool;
};
struct SchedulerBox {
    std::unique_ptr<Scheduler> sched;
    std::map<RequestId, RequestPtr> requests;
    std::map<long long, StepPlan> plans;
    long long next_plan = 1;
};
struct ModelBox {
    std::unique_ptr<Model> model;
};
struct EngineBox {
    std::unique_ptr<Model> model;             // set when the engine owns its model
    std::unique_ptr<Engine> owned;
    Engine* engine = nullptr;                 // owned, or borrowed from an LLM
    std::map<int, BurstHandle> bursts;
    int next_burst = 0;
    cudaEvent_t marks[2] = {nullptr, nullptr};
};
struct LLMBox {
    std::unique_ptr<LLM> llm;
    EngineBox engine_box;                     // a borrowed view of the LLM's engine
};
struct WeightsBox {
    std::unique_ptr<SafetensorsFile> file;
    TensorMap loaded;                         // after "load": the bound tensors
};

DType dtype_from(const Json& args, const char* key = "dtype", DType fallback = DType::BF16) {
    const Json* v = args.find(key);
    if (!v || v->is_null()) return fallback;
    const std::string s = v->as_string();
    if (s == "bfloat16" || s == "bf16") return DType::BF16;
    if (s == "float32" || s == "fp32") return DType::F32;
    throw ValueError("dtype must be 'bfloat16' or 'float32', got '" + s + "'");
}

StoreDType store_from(const Json& args, const char* key = "dtype") {
    const Json* v = args.find(key);
    if (!v || v->is_null()) return StoreDType::BF16;
    return store_dtype_from_name(v->as_string());
}

long long geti(const Json& a, const char* key, long long fallback) {
    const Json* v = a.find(key);
    return (v && !v->is_null()) ? v->as_int() : fallback;
}
bool getb(const Json& a, const char* key, bool fallback) {
    const Json* v = a.find(key);
    return (v && !v->is_null()) ? v->as_bool() : fallback;
}

Json ints(const std::vector<int>& v) {
    Json a = Json::array();
    for (int x : v) a.push(x);
    return a;
}

Json requests_json(const TensorRequests& reqs) {
    Json out = Json::object();
    for (const auto& kv : reqs) {
        Json e = Json::object();
        Json shape = Json::array();
        for (int64_t d : kv.second.shape) shape.push((long long)d);
        e["shape"] = shape;
        e["integer"] = kv.second.integer;
        e["keep_32bit"] = kv.second.keep_32bit;
        e["init"] = kv.second.init;
        out[kv.first] = e;
    }
    return out;
}

TensorRequests requests_from(const Json& j) {
    TensorRequests out;
    for (const auto& m : j.members()) {
        TensorRequest r;
        for (const Json& d : m.second.at("shape").items()) r.shape.push_back(d.as_int());
        if (const Json* v = m.second.find("integer")) r.integer = v->as_bool();
        if (const Json* v = m.second.find("keep_32bit")) r.keep_32bit = v->as_bool();
        if (const Json* v = m.second.find("init")) r.init = v->as_string();
        out[m.first] = r;
    }
    return out;
}

Json tensors_json(const TensorMap& t) {
    Json out = Json::object();
    for (const auto& kv : t) {
        Json e = Json::object();
        Json shape = Json::array();
        for (int64_t d : kv.second.shape) shape.push((long long)d);
        e["shape"] = shape;
        e["dtype"] = store_dtype_name(kv.second.dtype);
        e["address"] = (long long)(uintptr_t)kv.second.data;
        e["bytes"] = (long long)kv.second.bytes();
        out[kv.first] = e;
    }
    return out;
}

std::vector<CacheSpec> cache_specs_from(const Json& j) {
    std::vector<CacheSpec> out;
    for (const Json& s : j.items()) {
        if (s.is_null()) { out.push_back(CacheSpec::none()); continue; }
        const std::string kind = s.at("kind").as_string();
        if (kind == "paged") out.push_back(CacheSpec::paged((int)s.at("n_kv_heads").as_int(), (int)s.at("head_dim").as_int(), (int)geti(s, "window", 0)));
        else if (kind == "state") {
            std::vector<int64_t> shape;
            for (const Json& d : s.at("shape").items()) shape.push_back(d.as_int());
            out.push_back(CacheSpec::state(shape));
        } else throw CacheError("unknown cache spec kind '" + kind + "'");
    }
    return out;
}

Json layout_json(const CacheLayout& l) {
    Json out = Json::object();
    out["page_size"] = l.page_size;
    Json groups = Json::array();
    for (const auto& g : l.groups) {
        Json e = Json::object();
        e["index"] = g.index;
        e["caches"] = ints(g.caches);
        e["n_kv_heads"] = g.spec.n_kv_heads;
        e["head_dim"] = g.spec.head_dim;
        e["window"] = g.spec.window;
        groups.push(e);
    }
    out["groups"] = groups;
    Json goc = Json::object();
    for (const auto& kv : l.group_of_cache) {
        Json pair = Json::array();
        pair.push(kv.second.first);
        pair.push(kv.second.second);
        goc[std::to_string(kv.first)] = pair;
    }
    out["group_of_cache"] = goc;
    Json states = Json::array();
    for (const auto& kv : l.state_of_cache) states.push(kv.first);
    out["state_caches"] = states;
    return out;
}

Json request_json(const Request& r) {
    Json o = Json::object();
    o["rid"] = (long long)r.rid;
    o["state"] = r.state == RequestState::Waiting ? "waiting" : (r.state == RequestState::Running ? "running" : "finished");
    o["output"] = ints(r.output);
    o["computed"] = r.computed;
    o["finish_reason"] = r.finish_reason.empty() ? Json() : Json(r.finish_reason);
    o["preemptions"] = r.preemptions;
    o["admitted_at"] = (long long)r.admitted_at;
    o["n_prompt"] = (long long)r.prompt.size();
    return o;
}

Json result_json(const GenerateResult& g) {
    Json o = Json::object();
    o["output_ids"] = ints(g.output_ids);
    o["finish_reason"] = g.finish_reason;
    o["prompt_tokens"] = g.prompt_tokens;
    o["completion_tokens"] = g.completion_tokens;
    o["prefill_ms"] = g.prefill_ms;
    o["decode_ms"] = g.decode_ms;
    o["prefill_tokens_per_second"] = g.prefill_tokens_per_second;
    o["decode_tokens_per_second"] = g.decode_tokens_per_second;
    o["preemptions"] = g.preemptions;
    return o;
}

Json handle_json(void* p) {
    Json o = Json::object();
    o["handle"] = (long long)(uintptr_t)p;
    return o;
}

LLMOptions llm_options_from(const Json& a) {
    LLMOptions o;
    o.dtype = dtype_from(a);
    o.device = (int)geti(a, "device", 0);
    o.cache_tokens = geti(a, "cache_tokens", 0);
    o.page_size = (int)geti(a, "page_size", 16);
    o.max_live = (int)geti(a, "max_live", 64);
    o.max_step_tokens = (int)geti(a, "max_step_tokens", 2048);
    o.prefill_chunk_tokens = (int)geti(a, "prefill_chunk_tokens", 2048);
    if (const Json* e = a.find("eos_token_ids"))
        if (e->is_array())
            for (const Json& t : e->items()) o.eos_token_ids.push_back((int)t.as_int());
    o.max_context_tokens = (int)geti(a, "max_context_tokens", 0);
    o.use_cuda_graphs = getb(a, "use_cuda_graphs", true);
    o.max_burst = (int)geti(a, "max_burst", 8);
    o.pipeline_bursts = getb(a, "pipeline_bursts", true);
    return o;
}

// ---- method tables ----------------------------------------------------------------------------------------
Json call_global(const std::string& m, const Json& a) {
    if (m == "architectures") {
        Json out = Json::array();
        for (const auto& n : architectures()) out.push(n);
        return out;
    }
    if (m == "part_kinds") {
        Json out = Json::array();
        for (const auto& n : part_kinds(a.at("family").as_string())) out.push(n);
        return out;
    }
    if (m == "check_part_kind") {
        get_part(a.at("family").as_string(), a.at("kind").as_string());
        return Json(true);
    }
    if (m == "get_architecture") {
        get_architecture(a.at("name").as_string());
        return Json(true);
    }
    if (m == "parse_config") {                       // raw config.json -> typed, optionally validated
        const Json& raw = a.at("config");
        const Architecture& arch = get_architecture(a.find("architecture") ? a.at("architecture").as_string() : architecture_name(raw));
        std::unique_ptr<ModelConfig> cfg = arch.parse(raw);
        if (getb(a, "validate", true)) cfg->validate();
        return cfg->to_json();
    }
    if (m == "load_config") return load_config(a.at("model_dir").as_string())->to_json();
    if (m == "save_config") return Json(save_config(*parse_config(a.at("config")), a.at("model_dir").as_string()));
    if (m == "describe") return to_json(describe(*parse_config(a.at("config"))));
    if (m == "write_random_model")
        return Json(write_random_model(*parse_config(a.at("config")), a.at("out_dir").as_string(), (uint64_t)geti(a, "seed", 0), store_from(a)));
    if (m == "uniform_for") return Json((double)uniform_for((uint64_t)a.at("seed").as_int(), (uint64_t)a.at("index").as_int()));
    if (m == "validate_sampling") {
        SamplingParams s;
        s.temperature = (float)a.at("temperature").as_double();
        s.top_k = (int)a.at("top_k").as_int();
        s.top_p = (float)a.at("top_p").as_double();
        s.validate();
        return Json(true);
    }
    if (m == "decode_splits")
        return Json(ops::decode_splits((int)a.at("n_tokens").as_int(), (int)a.at("n_heads").as_int(), (int)a.at("max_kv").as_int(), (int)geti(a, "sms", 0)));
    if (m == "small_gemm_kernel")                     // {"M", "N", "K"} -> "split_k" | "streaming": the rule for products of up to 64 rows
        return Json(ops::small_gemm_kernel(a.at("M").as_int(), a.at("N").as_int(), a.at("K").as_int()) == ops::SmallGemm::SplitK
                        ? std::string("split_k") : std::string("streaming"));
    if (m == "leave_out") {                           // {"families": [...]}: launches to skip (timing only); [] restores
        std::vector<std::string> families;
        if (a.has("families"))
            for (const Json& f : a.at("families").items()) families.push_back(f.as_string());
        ops::leave_out(families);
        return Json();
    }
    if (m == "force_tile") {                          // {"N", "K", "tile"}: the tcgen05 variant of one weight shape; 0 restores
        ops::force_tile(a.at("N").as_int(), a.at("K").as_int(), (int)a.at("tile").as_int());
        return Json();
    }
    if (m == "profile_kernels") {                     // {"enable": bool} -> what was gathered since it was switched on
        Json out = Json::array();
        for (const ops::ProfileRow& r : ops::profile_report()) {
            Json e = Json::object();
            e["class"] = r.op_class;
            e["calls"] = r.calls;
            e["us"] = r.us;
            e["bytes"] = r.bytes;
            e["flops"] = r.flops;
            out.push(e);
        }
        ops::profile_enable(getb(a, "enable", false));
        return out;
    }
    if (m == "random_tensors") {                      // {"requests": {...}, "seed", "dtype"} -> a weights handle holding them
        auto* box = new WeightsBox();
        box->loaded = random_tensors(requests_from(a.at("requests")), (uint64_t)geti(a, "seed", 0), store_from(a));
        Json out = handle_json(box);
        out["tensors"] = tensors_json(box->loaded);
        return out;
    }
    if (m == "new_allocator") {
        CacheLayout layout = CacheLayout::from_specs(cache_specs_from(a.at("specs")), (int)geti(a, "page_size", 16));
        std::vector<int> pages;
        if (a.at("pages").is_array()) for (const Json& p : a.at("pages").items()) pages.push_back((int)p.as_int());
        else pages.assign(layout.groups.size(), (int)a.at("pages").as_int());
        auto* box = new AllocatorBox();
        box->owned.reset(new BlockAllocator(std::move(layout), pages, (int)geti(a, "max_requests", 4)));
        box->alloc = box->owned.get();
        return handle_json(box);
    }
    if (m == "new_pool") {
        auto* box = new PoolBox();
        std::unique_ptr<PoolBox> guard(box);
        box->pool.reset(new PagePool((int)a.at("num_pages").as_int()));
        guard.release();
        return handle_json(box);
    }
    if (m == "new_scheduler") {
        auto* ab = (AllocatorBox*)(uintptr_t)a.at("allocator").as_int();
        Scheduler::Options o;
        o.max_step_tokens = (int)geti(a, "max_step_tokens", 2048);
        o.prefill_chunk = (int)geti(a, "prefill_chunk", 2048);
        o.max_live = (int)geti(a, "max_live", 64);
        if (const Json* p = a.find("max_positions"))
            if (!p->is_null()) o.max_positions = (int)p->as_int();
        auto* box = new SchedulerBox();
        box->sched.reset(new Scheduler(*ab->alloc, o));
        return handle_json(box);
    }
    if (m == "build_model") {                         // from a configuration, no weights
        auto* box = new ModelBox();
        std::shared_ptr<ModelConfig> cfg = parse_config(a.at("config"));
        box->model.reset(new Model(describe(*cfg)));
        box->model->set_config(cfg);
        return handle_json(box);
    }
    if (m == "build_model_from_spec") {
        auto* box = new ModelBox();
        box->model.reset(new Model(model_spec_from_json(a.at("spec"))));
        return handle_json(box);
    }
    if (m == "load_model") {
        cuda_check(cudaSetDevice((int)geti(a, "device", 0)), "selecting the device");
        auto* box = new ModelBox();
        box->model = load_model(a.at("model_dir").as_string(), dtype_from(a));
        return handle_json(box);
    }
    if (m == "new_engine") {
        auto* mb = (ModelBox*)(uintptr_t)a.at("model").as_int();
        Engine::Options o;
        o.max_tokens = a.at("max_tokens").as_int();
        o.page_size = (int)geti(a, "page_size", 16);
        o.max_requests = (int)geti(a, "max_requests", 64);
        o.max_step_tokens = (int)geti(a, "max_step_tokens", 2048);
        o.use_cuda_graphs = getb(a, "use_cuda_graphs", true);
        auto* box = new EngineBox();
        box->owned.reset(new Engine(*mb->model, o));
        box->engine = box->owned.get();
        return handle_json(box);
    }
    if (m == "open_weights") {
        auto* box = new WeightsBox();
        box->file.reset(new SafetensorsFile(a.at("path").as_string()));
        return handle_json(box);
    }
    if (m == "load_weights") {                        // check a folder's file against requests; the tensors stay mapped
        auto* box = new WeightsBox();
        std::vector<std::string> prefixes, ignored;
        if (const Json* p = a.find("prefixes")) for (const Json& v : p->items()) prefixes.push_back(v.as_string());
        if (const Json* p = a.find("ignored")) for (const Json& v : p->items()) ignored.push_back(v.as_string());
        std::unique_ptr<WeightsBox> guard(box);
        box->loaded = load_weights(a.at("model_dir").as_string(), requests_from(a.at("requests")), prefixes, ignored);
        guard.release();
        Json out = handle_json(box);
        out["tensors"] = tensors_json(box->loaded);
        return out;
    }
    if (m == "write_safetensors") {                   // {"path", "tensors": {name: {"dtype","shape","address"}}}
        std::map<std::string, HostTensor> tensors;
        for (const auto& kv : a.at("tensors").members()) {
            HostTensor t;
            t.dtype = store_dtype_from_name(kv.second.at("dtype").as_string());
            for (const Json& d : kv.second.at("shape").items()) t.shape.push_back(d.as_int());
            t.data = (const void*)(uintptr_t)kv.second.at("address").as_int();
            tensors[kv.first] = t;
        }
        write_safetensors(a.at("path").as_string(), tensors);
        return Json(true);
    }
    if (m == "new_harness") return handle_json(new PartHarness(a));
    throw ValueError("no global method '" + m + "'");
}

Json call_allocator(BlockAllocator& al, const std::string& m, const Json& a) {
    auto rid = [&]() { return (RequestId)a.at("rid").as_int(); };
    if (m == "admit") return Json(al.admit(rid()));
    if (m == "reserve") { al.reserve(rid(), (int)a.at("new_len").as_int()); return Json(); }
    if (m == "commit") { al.commit(rid(), (int)a.at("new_len").as_int()); return Json(); }
    if (m == "release") { al.release(rid()); return Json(); }
    if (m == "check") { al.check(); return Json(); }
    if (m == "contains") return Json(al.contains(rid()));
    if (m == "slot") return Json(al.slot(rid()));
    if (m == "length") return Json(al.length(rid()));
    if (m == "block_version") return Json((long long)al.block_version(rid()));
    if (m == "block_list") return ints(al.block_list(rid(), (int)geti(a, "group", 0)));
    if (m == "free_slots") return Json(al.free_slots());
    if (m == "free_pages") return Json(al.free_pages((int)geti(a, "group", 0)));
    if (m == "pages_needed") return ints(al.pages_needed(rid(), (int)a.at("new_len").as_int()));
    if (m == "can_reserve") return Json(al.can_reserve(rid(), (int)a.at("new_len").as_int()));
    if (m == "live") {
        Json out = Json::array();
        for (RequestId r : al.live()) out.push((long long)r);
        return out;
    }
    if (m == "layout") return layout_json(al.layout());
    if (m == "pools") {
        Json out = Json::array();
        for (int g = 0; g < al.n_groups(); g++) {
            Json p = Json::object();
            p["num_pages"] = al.pool(g).num_pages();
            p["free_pages"] = al.pool(g).free_pages();
            p["used_pages"] = al.pool(g).used_pages();
            p["high_water"] = al.pool(g).high_water();
            out.push(p);
        }
        return out;
    }
    if (m == "info") {
        Json o = Json::object();
        o["page_size"] = al.page_size();
        o["max_requests"] = al.max_requests();
        o["n_groups"] = al.n_groups();
        return o;
    }
    throw ValueError("no allocator method '" + m + "'");
}

Json call_pool(PagePool& p, const std::string& m, const Json& a) {
    if (m == "allocate") return ints(p.allocate((int)a.at("n").as_int()));
    if (m == "release") {
        std::vector<int> pages;
        for (const Json& v : a.at("pages").items()) pages.push_back((int)v.as_int());
        p.release(pages);
        return Json();
    }
    if (m == "info") {
        Json o = Json::object();
        o["num_pages"] = p.num_pages();
        o["free_pages"] = p.free_pages();
        o["used_pages"] = p.used_pages();
        o["high_water"] = p.high_water();
        return o;
    }
    throw ValueError("no pool method '" + m + "'");
}

Json plan_json(SchedulerBox& sb, StepPlan plan) {
    Json o = Json::object();
    Json portions = Json::array();
    for (const Portion& p : plan.portions) {
        Json e = Json::object();
        e["rid"] = (long long)p.request->rid;
        e["start"] = p.start;
        e["count"] = p.count;
        e["samples"] = p.samples;
        portions.push(e);
    }
    o["portions"] = portions;
    Json pre = Json::array();
    for (const RequestPtr& r : plan.preempted) pre.push((long long)r->rid);
    o["preempted"] = pre;
    const long long id = sb.next_plan++;
    o["plan"] = id;
    sb.plans[id] = std::move(plan);
    while (sb.plans.size() > 64) sb.plans.erase(sb.plans.begin());
    return o;
}

Json call_scheduler(SchedulerBox& sb, const std::string& m, const Json& a) {
    Scheduler& s = *sb.sched;
    if (m == "add") {
        auto r = std::make_shared<Request>();
        r->rid = (RequestId)a.at("rid").as_int();
        for (const Json& t : a.at("prompt").items()) r->prompt.push_back((int)t.as_int());
        r->max_tokens = (int)a.at("max_tokens").as_int();
        if (const Json* st = a.find("stop_ids")) for (const Json& t : st->items()) r->stop_ids.insert((int)t.as_int());
        sb.requests[r->rid] = r;
        try {
            s.add(r);
        } catch (...) {
            sb.requests.erase(r->rid);
            throw;
        }
        return request_json(*r);
    }
    if (m == "plan") return plan_json(sb, s.plan());
    if (m == "complete") {
        auto it = sb.plans.find(a.at("plan").as_int());
        if (it == sb.plans.end()) throw ValueError("unknown plan");
        std::vector<int> sampled(it->second.portions.size(), 0);
        const Json& given = a.at("sampled");           // {rid: token}
        for (size_t i = 0; i < it->second.portions.size(); i++) {
            const Portion& p = it->second.portions[i];
            if (!p.samples) continue;
            const Json* t = given.find(std::to_string(p.request->rid));
            if (!t) throw ValueError("no sampled token for request " + std::to_string(p.request->rid));
            sampled[i] = (int)t->as_int();
        }
        Json done = Json::array();
        for (const RequestPtr& r : s.complete(it->second, sampled)) done.push((long long)r->rid);
        sb.plans.erase(it);
        return done;
    }
    if (m == "abort") {
        RequestPtr r = s.abort((RequestId)a.at("rid").as_int(), a.find("reason") ? a.at("reason").as_string() : "cancelled");
        return r ? Json((long long)r->rid) : Json();
    }
    if (m == "has_work") return Json(s.has_work());
    if (m == "request") {
        auto it = sb.requests.find((RequestId)a.at("rid").as_int());
        if (it == sb.requests.end()) throw ValueError("unknown request");
        return request_json(*it->second);
    }
    if (m == "queues") {
        Json o = Json::object();
        Json w = Json::array(), r = Json::array(), f = Json::array();
        for (const auto& q : s.waiting()) w.push((long long)q->rid);
        for (const auto& q : s.running()) r.push((long long)q->rid);
        for (const auto& q : s.finished()) f.push((long long)q->rid);
        o["waiting"] = w; o["running"] = r; o["finished"] = f;
        return o;
    }
    if (m == "stats") {
        Json o = Json::object();
        for (const auto& kv : s.stats()) o[kv.first] = (long long)kv.second;
        return o;
    }
    throw ValueError("no scheduler method '" + m + "'");
}

Json call_model(Model& model, const std::string& m, const Json& a) {
    (void)a;
    if (m == "tensor_requests") return requests_json(model.tensor_requests());
    if (m == "spec") return to_json(model.spec());
    if (m == "config") return model.config() ? model.config()->to_json() : Json();
    if (m == "info") {
        Json o = Json::object();
        o["graph_safe"] = model.graph_safe();
        o["max_positions"] = model.max_positions() ? Json((long long)*model.max_positions()) : Json();
        o["bound"] = model.bound();
        o["weight_bytes"] = model.bound() ? Json((long long)model.weight_bytes()) : Json();
        o["dtype"] = dtype_name(model.compute_dtype());
        o["vocab_size"] = (long long)model.spec().vocab_size;
        o["width"] = (long long)model.spec().width;
        return o;
    }
    if (m == "bind_random") {                         // seeded random weights straight onto the device
        cuda_check(cudaSetDevice((int)geti(a, "device", 0)), "selecting the device");
        const DType dt = dtype_from(a);
        model.bind(random_tensors(model.tensor_requests(), (uint64_t)geti(a, "seed", 0), dt == DType::BF16 ? StoreDType::BF16 : StoreDType::F32), dt);
        return Json();
    }
    throw ValueError("no model method '" + m + "'");
}

Json call_engine(EngineBox& eb, const std::string& m, const Json& a) {
    Engine& e = *eb.engine;
    if (m == "allocator") {                            // a borrowed allocator handle
        auto* box = new AllocatorBox();
        box->alloc = &e.cache().alloc();
        return handle_json(box);
    }
    if (m == "admit") return Json(e.admit((RequestId)a.at("rid").as_int()));
    if (m == "release") { e.release((RequestId)a.at("rid").as_int()); return Json(); }
    if (m == "length") return Json(e.length((RequestId)a.at("rid").as_int()));
    if (m == "commit") { e.commit((RequestId)a.at("rid").as_int(), (int)a.at("new_len").as_int()); return Json(); }
    if (m == "poison") { e.cache().device().poison(e.stream()); e.synchronize(); return Json(); }
    if (m == "check_status") { e.check_status(); return Json(); }
    if (m == "counters") {
        Json o = Json::object();
        o["steps_run"] = e.steps_run;
        o["graph_replays"] = e.graph_replays;
        o["stale_graphs"] = e.stale_graphs;
        o["burst_graphs_recorded"] = e.burst_graphs_recorded;
        o["recorded_graphs"] = (long long)e.recorded_graphs();
        o["h2d_bytes_total"] = e.h2d_bytes_total;
        o["d2h_bytes_total"] = e.d2h_bytes_total;
        o["last_h2d_bytes"] = e.last_h2d_bytes;
        o["last_launches"] = e.last_launches;
        o["use_cuda_graphs"] = e.use_cuda_graphs();
        o["kv_bytes_per_token"] = (long long)e.cache().kv_bytes_per_token();
        o["cache_bytes"] = (long long)e.cache().device().bytes();
        o["page_size"] = e.cache().page_size();
        o["max_requests"] = e.cache().max_requests();
        o["dtype"] = dtype_name(e.dtype());
        return o;
    }
    if (m == "state") {                                // a fixed-size state's device view
        const StateView v = e.cache().device().state((int)a.at("cache").as_int());
        Json o = Json::object();
        o["address"] = (long long)(uintptr_t)v.data;
        o["row_elems"] = (long long)v.row_elems;
        o["rows"] = v.rows;
        o["dtype"] = dtype_name(v.dtype);
        return o;
    }
    throw ValueError("no engine method '" + m + "'");
}

Json call_llm(LLMBox& lb, const std::string& m, const Json& a) {
    LLM& l = *lb.llm;
    if (m == "result") return result_json(l.result((RequestId)a.at("rid").as_int()));
    if (m == "request") return request_json(l.request((RequestId)a.at("rid").as_int()));
    if (m == "forget") { l.forget((RequestId)a.at("rid").as_int()); return Json(); }
    if (m == "abort") { l.abort((RequestId)a.at("rid").as_int()); return Json(); }
    if (m == "info") {
        Json o = Json::object();
        o["max_burst"] = l.max_burst();
        o["pipeline_bursts"] = l.pipeline_bursts();
        o["decode_steps_run"] = l.decode_steps_run;
        o["bursts_queued_ahead"] = l.bursts_queued_ahead;
        o["n_waiting"] = (long long)l.scheduler().waiting().size();
        o["n_running"] = (long long)l.scheduler().running().size();
        return o;
    }
    if (m == "scheduler_stats") {
        Json o = Json::object();
        for (const auto& kv : l.scheduler().stats()) o[kv.first] = (long long)kv.second;
        return o;
    }
    if (m == "model_info") return call_model(l.model(), "info", a);
    if (m == "model_config") return call_model(l.model(), "config", a);
    if (m == "tensor_requests" || m == "spec") return call_model(l.model(), m, a);
    throw ValueError("no llm method '" + m + "'");
}

Json call_weights(WeightsBox& wb, const std::string& m, const Json& a) {
    if (m == "tensors") {
        if (wb.file) {
            TensorMap all;
            for (const auto& n : wb.file->names()) all[n] = wb.file->tensor(n);
            return tensors_json(all);
        }
        return tensors_json(wb.loaded);
    }
    (void)a;
    throw ValueError("no weights method '" + m + "'");
}

Json call_harness(PartHarness& h, const std::string& m, const Json& a) {
    auto ptr = [&](const char* key) -> void* {
        const Json* v = a.find(key);
        return (v && !v->is_null()) ? (void*)(uintptr_t)v->as_int() : nullptr;
    };
    if (m == "tensors") return h.tensors();
    if (m == "info") return h.info();
    if (m == "set_step") {
        std::vector<std::pair<int, int>> seqs;
        for (const Json& s : a.at("seqs").items()) seqs.emplace_back((int)s.items()[0].as_int(), (int)s.items()[1].as_int());
        std::vector<int> ids;
        if (const Json* v = a.find("ids"))
            if (v->is_array()) for (const Json& t : v->items()) ids.push_back((int)t.as_int());
        h.set_step(seqs, ids.empty() ? nullptr : ids.data());
        return Json();
    }
    if (m == "run_norm") {
        std::vector<int> rows;
        if (const Json* v = a.find("rows"))
            if (v->is_array()) for (const Json& t : v->items()) rows.push_back((int)t.as_int());
        h.run_norm(ptr("x"), (int)a.at("x_rows").as_int(), ptr("out"), (int)a.at("n_rows").as_int(), rows.empty() ? nullptr : rows.data());
        return Json();
    }
    if (m == "run_feed_forward") { h.run_feed_forward(ptr("h"), ptr("x")); return Json(); }
    if (m == "run_mixer") { h.run_mixer(ptr("h"), ptr("x"), getb(a, "write_cache", true)); return Json(); }
    if (m == "run_embedding") { h.run_embedding(ptr("x")); return Json(); }
    throw ValueError("no harness method '" + m + "'");
}

}  // namespace

// ---- exported functions ---------------------------------------------------------------------------------------
extern "C" {

#define SANDY_EXPORT __attribute__((visibility("default")))

SANDY_EXPORT const char* sandy_last_error_kind(void) { return t_kind.c_str(); }
SANDY_EXPORT const char* sandy_last_error_message(void) { return t_message.c_str(); }
SANDY_EXPORT const char* sandy_last_error_details(void) { return t_details.c_str(); }

SANDY_EXPORT void sandy_set_kernel_dir(const char* dir) { set_kernel_dir(dir ? dir : ""); }
SANDY_EXPORT void sandy_set_kernel_provider(sandy_kernel_provider provider) { set_kernel_provider(provider); }
SANDY_EXPORT long long sandy_kernel_launches(void) { return g_launches; }

SANDY_EXPORT const char* sandy_call(const char* object, void* handle, const char* method, const char* args_json) {
    return guarded(
        [&]() -> const char* {
            const std::string obj = object ? object : "", m = method ? method : "";
            const Json a = (args_json && *args_json) ? Json::parse(args_json) : Json::object();
            Json out;
            if (obj == "global") out = call_global(m, a);
            else if (!handle) throw ValueError("a null handle was given for a '" + obj + "'");
            else if (obj == "allocator") out = call_allocator(*((AllocatorBox*)handle)->alloc, m, a);
            else if (obj == "pool") out = call_pool(*((PoolBox*)handle)->pool, m, a);
            else if (obj == "scheduler") out = call_scheduler(*(SchedulerBox*)handle, m, a);
            else if (obj == "model") {
                auto* mb = (ModelBox*)handle;
                if (!mb->model) throw ValueError("this model was handed over to an engine; ask the engine");
                out = call_model(*mb->model, m, a);
            }
            else if (obj == "engine") out = call_engine(*(EngineBox*)handle, m, a);
            else if (obj == "llm") out = call_llm(*(LLMBox*)handle, m, a);
            else if (obj == "weights") out = call_weights(*(WeightsBox*)handle, m, a);
            else if (obj == "harness") out = call_harness(*(PartHarness*)handle, m, a);
            else throw ValueError("no object kind '" + obj + "'");
            t_result = out.dump();
            return t_result.c_str();
        },
        (const char*)nullptr);
}

SANDY_EXPORT void sandy_release(const char* object, void* handle) {
    if (!handle || !object) return;
    const std::string obj = object;
    try {
        if (obj == "allocator") delete (AllocatorBox*)handle;
        else if (obj == "pool") delete (PoolBox*)handle;
        else if (obj == "scheduler") delete (SchedulerBox*)handle;
        else if (obj == "model") delete (ModelBox*)handle;
        else if (obj == "engine") {
            auto* eb = (EngineBox*)handle;
            for (auto& e : eb->marks) if (e) cudaEventDestroy(e);
            delete eb;
        } else if (obj == "llm") {
            auto* lb = (LLMBox*)handle;
            for (auto& e : lb->engine_box.marks) if (e) cudaEventDestroy(e);
            delete lb;
        } else if (obj == "weights") delete (WeightsBox*)handle;
        else if (obj == "harness") delete (PartHarness*)handle;
    } catch (...) {
    }
}

SANDY_EXPORT int sandy_register_architecture(const char* name, sandy_json_fn parse, sandy_json_fn describe_fn, void* user) {
    return guarded([&]() { register_foreign_architecture(name, parse, describe_fn, user); return 0; }, 1);
}
SANDY_EXPORT void sandy_set_callback_error(const char* kind, const char* message) {
    set_callback_error(kind ? kind : "ForeignError", message ? message : "");
}
SANDY_EXPORT int sandy_register_part(const char* family, const char* kind, const SandyForeignPart* vtable, void* user) {
    return guarded([&]() { register_foreign_part(family, kind, *vtable, user); return 0; }, 1);
}
SANDY_EXPORT int sandy_step_state(const SandyStepView* step, int cache, SandyTensorView* out) {
    return guarded(
        [&]() {
            auto* ctx = (StepContext*)step->context;
            const StateView v = ctx->caches->state(cache);
            out->data = v.data;
            out->dtype = (int)v.dtype;
            out->cols = v.row_elems;
            out->ld = v.row_elems;
            out->rows = v.rows;
            return 0;
        },
        1);
}
SANDY_EXPORT int sandy_step_kv(const SandyStepView* step, int cache, SandyTensorView* k, SandyTensorView* v, int* group,
                               int* n_kv_heads, int* page_size, int* head_dim) {
    return guarded(
        [&]() {
            auto* ctx = (StepContext*)step->context;
            const KVView c = ctx->caches->kv(cache);
            *k = SandyTensorView{c.k, (int)c.dtype, c.num_pages, (long long)c.n_kv_heads * c.page_size * c.head_dim, c.page_stride};
            *v = SandyTensorView{c.v, (int)c.dtype, c.num_pages, (long long)c.n_kv_heads * c.page_size * c.head_dim, c.page_stride};
            *group = c.group;
            *n_kv_heads = c.n_kv_heads;
            *page_size = c.page_size;
            *head_dim = c.head_dim;
            return 0;
        },
        1);
}

// ---- LLM ----
static LLMBox* finish_llm(std::unique_ptr<LLM> llm) {
    auto* box = new LLMBox();
    box->llm = std::move(llm);
    box->engine_box.engine = &box->llm->engine();
    return box;
}
SANDY_EXPORT void* sandy_llm_load(const char* model_dir, const char* options_json) {
    return guarded(
        [&]() -> void* {
            const Json a = (options_json && *options_json) ? Json::parse(options_json) : Json::object();
            return finish_llm(LLM::load(model_dir, llm_options_from(a)));
        },
        (void*)nullptr);
}
SANDY_EXPORT void* sandy_llm_from_model(void* model, const char* options_json) {
    return guarded(
        [&]() -> void* {
            const Json a = (options_json && *options_json) ? Json::parse(options_json) : Json::object();
            auto* mb = (ModelBox*)model;
            if (!mb->model) throw ValueError("the model handle is empty (it was given to another engine)");
            return finish_llm(std::unique_ptr<LLM>(new LLM(std::move(mb->model), llm_options_from(a))));
        },
        (void*)nullptr);
}
SANDY_EXPORT long long sandy_llm_add_request(void* llm, const int* prompt_ids, int n_prompt, int max_tokens, float temperature,
                                             int top_k, float top_p, int has_seed, unsigned long long seed, const int* stop_ids,
                                             int n_stop) {
    return guarded(
        [&]() -> long long {
            SamplingParams s;
            s.temperature = temperature;
            s.top_k = top_k;
            s.top_p = top_p;
            if (has_seed) s.seed = seed;
            return ((LLMBox*)llm)->llm->add_request(std::vector<int>(prompt_ids, prompt_ids + n_prompt), max_tokens, s,
                                                    std::vector<int>(stop_ids, stop_ids + n_stop));
        },
        -1LL);
}
static int write_pairs(const std::vector<std::pair<RequestId, int>>& got, long long* rids, int* tokens, int capacity) {
    for (size_t i = 0; i < got.size() && (int)i < capacity; i++) {
        rids[i] = got[i].first;
        tokens[i] = got[i].second;
    }
    return (int)got.size();
}
SANDY_EXPORT int sandy_llm_step(void* llm, long long* rids, int* tokens, int capacity) {
    return guarded([&]() { return write_pairs(((LLMBox*)llm)->llm->step(), rids, tokens, capacity); }, -1);
}
SANDY_EXPORT int sandy_llm_drain(void* llm, long long* rids, int* tokens, int capacity) {
    return guarded([&]() { return write_pairs(((LLMBox*)llm)->llm->drain(), rids, tokens, capacity); }, -1);
}
SANDY_EXPORT int sandy_llm_has_work(void* llm) { return ((LLMBox*)llm)->llm->has_work() ? 1 : 0; }
SANDY_EXPORT int sandy_llm_finished(void* llm, long long rid) {
    return guarded([&]() { return ((LLMBox*)llm)->llm->finished(rid) ? 1 : 0; }, -1);
}
SANDY_EXPORT const char* sandy_llm_generate(void* llm, const int* prompt_ids, const int* prompt_lens, int n_prompts,
                                            const char* params_json, sandy_token_fn on_token, void* user) {
    return guarded(
        [&]() -> const char* {
            const Json a = (params_json && *params_json) ? Json::parse(params_json) : Json::object();
            GenerateParams p;
            p.max_tokens = (int)geti(a, "max_tokens", 16);
            if (const Json* v = a.find("temperature")) p.temperature = (float)v->as_double();
            if (const Json* v = a.find("top_p")) p.top_p = (float)v->as_double();
            p.top_k = (int)geti(a, "top_k", 0);
            if (const Json* v = a.find("seed"))
                if (!v->is_null()) p.seed = (uint64_t)v->as_int();
            if (const Json* v = a.find("stop_token_ids")) for (const Json& t : v->items()) p.stop_token_ids.push_back((int)t.as_int());
            p.report = getb(a, "report", false);
            if (on_token) p.on_token = [on_token, user](int index, int token) { return on_token(user, index, token) != 0; };
            std::vector<std::vector<int>> prompts;
            size_t at = 0;
            for (int i = 0; i < n_prompts; i++) {
                prompts.emplace_back(prompt_ids + at, prompt_ids + at + prompt_lens[i]);
                at += (size_t)prompt_lens[i];
            }
            Json out = Json::array();
            for (const GenerateResult& g : ((LLMBox*)llm)->llm->generate(prompts, p)) out.push(result_json(g));
            t_result = out.dump();
            return t_result.c_str();
        },
        (const char*)nullptr);
}
SANDY_EXPORT void* sandy_llm_engine(void* llm) { return &((LLMBox*)llm)->engine_box; }

// ---- Engine ----
SANDY_EXPORT int sandy_engine_step(void* engine, int n_entries, const long long* rids, const int* n_tokens, const int* tokens,
                                   const int* n_want, const int* want, const float* sampling, void** logits, int* rows, int* cols) {
    return guarded(
        [&]() {
            std::vector<StepEntry> entries((size_t)n_entries);
            size_t t_at = 0, w_at = 0, n_rows = 0;
            for (int i = 0; i < n_entries; i++) {
                entries[(size_t)i].rid = rids[i];
                entries[(size_t)i].tokens.assign(tokens + t_at, tokens + t_at + n_tokens[i]);
                entries[(size_t)i].want.assign(want + w_at, want + w_at + n_want[i]);
                t_at += (size_t)n_tokens[i];
                w_at += (size_t)n_want[i];
                if (n_tokens[i]) n_rows += (size_t)n_want[i];
            }
            std::vector<SampleRow> srows;
            if (sampling)
                for (size_t r = 0; r < n_rows; r++)
                    srows.push_back(SampleRow{sampling[4 * r], (int)sampling[4 * r + 1], sampling[4 * r + 2], sampling[4 * r + 3]});
            const Tensor out = ((EngineBox*)engine)->engine->step(entries, sampling ? &srows : nullptr);
            *logits = out.data;
            *rows = (int)out.rows;
            *cols = (int)out.cols;
            return 0;
        },
        1);
}
SANDY_EXPORT int sandy_engine_read_sampled(void* engine, int n, int* out) {
    return guarded(
        [&]() {
            const std::vector<int> t = ((EngineBox*)engine)->engine->read_sampled(n);
            std::memcpy(out, t.data(), t.size() * sizeof(int));
            return 0;
        },
        1);
}
SANDY_EXPORT int sandy_engine_decode_burst_async(void* engine, int n_requests, const long long* rids, const int* first_tokens,
                                                 const float* sampling, const float* uniforms, int n_steps, int in_flight) {
    return guarded(
        [&]() {
            auto* eb = (EngineBox*)engine;
            std::vector<StepEntry> entries((size_t)n_requests);
            std::vector<SampleRow> rows;
            for (int i = 0; i < n_requests; i++) {
                entries[(size_t)i].rid = rids[i];
                entries[(size_t)i].tokens = {first_tokens ? first_tokens[i] : 0};
                entries[(size_t)i].want = {0};
                rows.push_back(sampling ? SampleRow{sampling[4 * i], (int)sampling[4 * i + 1], sampling[4 * i + 2], 0.0f} : SampleRow());
            }
            std::vector<float> u((size_t)n_steps * n_requests, 0.0f);
            if (uniforms) std::memcpy(u.data(), uniforms, u.size() * sizeof(float));
            const BurstHandle h = eb->engine->decode_burst_async(entries, rows, u, n_steps, in_flight);
            const int id = eb->next_burst++;
            eb->bursts[id] = h;
            while (eb->bursts.size() > 8) eb->bursts.erase(eb->bursts.begin());
            return id;
        },
        -1);
}
SANDY_EXPORT int sandy_engine_burst_tokens(void* engine, int burst, int* out) {
    return guarded(
        [&]() {
            auto* eb = (EngineBox*)engine;
            auto it = eb->bursts.find(burst);
            if (it == eb->bursts.end()) throw ValueError("unknown burst handle");
            const BurstHandle h = it->second;
            eb->bursts.erase(it);
            const std::vector<int> t = eb->engine->burst_tokens(h);
            std::memcpy(out, t.data(), t.size() * sizeof(int));
            return 0;
        },
        1);
}
SANDY_EXPORT int sandy_engine_synchronize(void* engine) {
    return guarded([&]() { ((EngineBox*)engine)->engine->synchronize(); return 0; }, 1);
}
SANDY_EXPORT void* sandy_engine_stream(void* engine) { return ((EngineBox*)engine)->engine->stream(); }
SANDY_EXPORT int sandy_engine_mark(void* engine, int which) {
    return guarded(
        [&]() {
            auto* eb = (EngineBox*)engine;
            which = which ? 1 : 0;
            if (!eb->marks[which]) cuda_check(cudaEventCreate(&eb->marks[which]), "creating an event");
            cuda_check(cudaEventRecord(eb->marks[which], eb->engine->stream()), "recording an event");
            return 0;
        },
        1);
}
SANDY_EXPORT int sandy_engine_hold(void* engine, int microseconds) {
    return guarded(
        [&]() {
            ops::spin(((EngineBox*)engine)->engine->stream(), (long long)microseconds * 1000);
            return 0;
        },
        1);
}
SANDY_EXPORT float sandy_engine_elapsed_ms(void* engine) {
    return guarded(
        [&]() {
            auto* eb = (EngineBox*)engine;
            if (!eb->marks[0] || !eb->marks[1]) throw ValueError("both marks must be set first");
            cuda_check(cudaEventSynchronize(eb->marks[1]), "waiting for the second mark");
            float ms = 0;
            cuda_check(cudaEventElapsedTime(&ms, eb->marks[0], eb->marks[1]), "reading the elapsed time");
            return ms;
        },
        -1.0f);
}

}  // extern "C"
