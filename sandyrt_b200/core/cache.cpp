#include "cache.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <functional>
#include <set>

namespace sandy {

size_t dtype_size(DType d) { return d == DType::BF16 ? 2 : 4; }
const char* dtype_name(DType d) { return d == DType::BF16 ? "bfloat16" : (d == DType::F32 ? "float32" : "int32"); }

CacheSpec CacheSpec::paged(int n_kv_heads, int head_dim, int window) {
    CacheSpec s;
    s.kind = Kind::PagedKV;
    s.n_kv_heads = n_kv_heads;
    s.head_dim = head_dim;
    s.window = window;
    return s;
}
CacheSpec CacheSpec::state(std::vector<int64_t> shape, DType dtype) {
    CacheSpec s;
    s.kind = Kind::State;
    s.state_shape = std::move(shape);
    s.state_dtype = dtype;
    return s;
}
bool CacheSpec::operator==(const CacheSpec& o) const {
    return kind == o.kind && n_kv_heads == o.n_kv_heads && head_dim == o.head_dim && window == o.window &&
           state_shape == o.state_shape && state_dtype == o.state_dtype;
}

// ---- PagePool ---------------------------------------------------------------------------------------
PagePool::PagePool(int num_pages) : num_pages_(num_pages) {
    if (num_pages <= 0) throw CacheError("a page pool needs at least one page");
    free_.resize((size_t)num_pages);
    for (int i = 0; i < num_pages; i++) free_[(size_t)i] = i;      // ascending: already a min-heap
    held_.assign((size_t)num_pages, 0);
}

std::vector<int> PagePool::allocate(int n) {
    if (n > (int)free_.size())
        throw OutOfPages("need " + std::to_string(n) + " pages, " + std::to_string(free_.size()) + " of " +
                         std::to_string(num_pages_) + " free");
    std::vector<int> pages;
    pages.reserve((size_t)std::max(n, 0));
    for (int i = 0; i < n; i++) {
        std::pop_heap(free_.begin(), free_.end(), std::greater<int>());
        pages.push_back(free_.back());
        free_.pop_back();
        held_[(size_t)pages.back()] = 1;
    }
    high_water_ = std::max(high_water_, used_pages());
    return pages;
}

void PagePool::release(const std::vector<int>& pages) {
    for (int p : pages) {
        if (p < 0 || p >= num_pages_) throw CacheError("page " + std::to_string(p) + " does not belong to this pool");
        if (!held_[(size_t)p]) throw CacheError("page " + std::to_string(p) + " freed twice");
        held_[(size_t)p] = 0;            // a page named twice in `pages` is caught by the line above
    }
    for (int p : pages) {
        free_.push_back(p);
        std::push_heap(free_.begin(), free_.end(), std::greater<int>());
    }
}

// ---- CacheLayout -------------------------------------------------------------------------------------
CacheLayout CacheLayout::from_specs(const std::vector<CacheSpec>& specs, int page_size) {
    if (page_size <= 0 || (page_size & (page_size - 1)))
        // the reference enforces a power of two as well (src/ir/MidIRMaterializer.cpp:48-49)
        throw CacheError("page size must be a power of two, got " + std::to_string(page_size));
    CacheLayout out;
    out.page_size = page_size;
    for (size_t ci = 0; ci < specs.size(); ci++) {
        const CacheSpec& spec = specs[ci];
        if (spec.kind == CacheSpec::Kind::None) continue;
        if (spec.kind == CacheSpec::Kind::State) { out.state_of_cache[(int)ci] = spec; continue; }
        bool placed = false;
        for (auto& g : out.groups)
            if (g.spec == spec) {
                out.group_of_cache[(int)ci] = {g.index, (int)g.caches.size()};
                g.caches.push_back((int)ci);
                placed = true;
                break;
            }
        if (!placed) {
            CacheGroup g;
            g.index = (int)out.groups.size();
            g.spec = spec;
            g.caches = {(int)ci};
            out.group_of_cache[(int)ci] = {g.index, 0};
            out.groups.push_back(std::move(g));
        }
    }
    return out;
}

// ---- BlockAllocator -------------------------------------------------------------------------------------
BlockAllocator::BlockAllocator(CacheLayout layout, const std::vector<int>& pages_per_group, int max_requests)
    : layout_(std::move(layout)), max_requests_(max_requests) {
    if (pages_per_group.size() != layout_.groups.size()) throw CacheError("one page count per cache group is needed");
    for (int n : pages_per_group) pools_.emplace_back(n);
    for (int s = max_requests - 1; s >= 0; s--) free_slots_.push_back(s);
}

const BlockAllocator::Req& BlockAllocator::get(RequestId rid) const {
    auto it = requests_.find(rid);
    if (it == requests_.end()) throw CacheError("request " + std::to_string(rid) + " is not live");
    return it->second;
}
BlockAllocator::Req& BlockAllocator::get(RequestId rid) {
    return const_cast<Req&>(static_cast<const BlockAllocator*>(this)->get(rid));
}

std::vector<RequestId> BlockAllocator::live() const {
    std::vector<RequestId> out;
    for (const auto& kv : requests_) out.push_back(kv.first);
    std::sort(out.begin(), out.end());
    return out;
}

// Blocks below this index hold only positions no later query of a request of `length` tokens reads.
int BlockAllocator::first_needed_block(int group, int length) const {
    const int window = layout_.groups[(size_t)group].spec.window;
    if (!window) return 0;
    const int first_pos = std::max(0, length - window + 1);     // oldest key the next query (position `length`) reads
    return first_pos / layout_.page_size;
}

std::vector<int> BlockAllocator::pages_needed(RequestId rid, int new_len) const {
    const Req& r = get(rid);
    const int want = (new_len + layout_.page_size - 1) / layout_.page_size;
    std::vector<int> out;
    for (const auto& bl : r.blocks) out.push_back(std::max(0, want - (int)bl.size()));
    return out;
}

std::vector<int> BlockAllocator::pages_for_new_request(int n_tokens) const {
    return std::vector<int>(pools_.size(), (n_tokens + layout_.page_size - 1) / layout_.page_size);
}

bool BlockAllocator::can_reserve(RequestId rid, int new_len) const {
    const std::vector<int> need = pages_needed(rid, new_len);
    for (size_t g = 0; g < need.size(); g++)
        if (need[g] > pools_[g].free_pages()) return false;
    return true;
}

int BlockAllocator::admit(RequestId rid) {
    if (requests_.count(rid)) throw CacheError("request " + std::to_string(rid) + " is already live");
    if (free_slots_.empty()) throw NoFreeSlot("all " + std::to_string(max_requests_) + " state slots are in use");
    Req r;
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    r.blocks.resize(pools_.size());
    r.version = ++stamp_;
    requests_[rid] = std::move(r);
    return requests_[rid].slot;
}

void BlockAllocator::reserve(RequestId rid, int new_len) {
    Req& r = get(rid);
    if (new_len < r.length)
        throw CacheError("request " + std::to_string(rid) + " holds " + std::to_string(r.length) + " tokens, cannot reserve for " +
                         std::to_string(new_len));
    const std::vector<int> need = pages_needed(rid, new_len);
    for (size_t g = 0; g < need.size(); g++)
        if (need[g] > pools_[g].free_pages())
            throw OutOfPages("group " + std::to_string(g) + ": request " + std::to_string(rid) + " needs " +
                             std::to_string(need[g]) + " more pages for " + std::to_string(new_len) + " tokens, " +
                             std::to_string(pools_[g].free_pages()) + " of " + std::to_string(pools_[g].num_pages()) + " free");
    for (size_t g = 0; g < need.size(); g++)
        if (need[g]) {
            const std::vector<int> pages = pools_[g].allocate(need[g]);
            r.blocks[g].insert(r.blocks[g].end(), pages.begin(), pages.end());
            r.version = ++stamp_;
        }
}

void BlockAllocator::commit(RequestId rid, int new_len) {
    Req& r = get(rid);
    if (new_len < r.length)
        throw CacheError("request " + std::to_string(rid) + " cannot shrink from " + std::to_string(r.length) + " to " +
                         std::to_string(new_len));
    if (!r.blocks.empty()) {
        size_t cap = r.blocks[0].size();
        for (const auto& bl : r.blocks) cap = std::min(cap, bl.size());
        if ((long long)new_len > (long long)cap * layout_.page_size)
            throw CacheError("request " + std::to_string(rid) + ": " + std::to_string(new_len) + " tokens were not reserved");
    }
    r.length = new_len;
    for (size_t g = 0; g < r.blocks.size(); g++) {
        auto& bl = r.blocks[g];
        const int first = std::min(first_needed_block((int)g, new_len), (int)bl.size());
        std::vector<int> gone;
        for (int i = 0; i < first; i++)
            if (bl[(size_t)i] != kFreed) gone.push_back(bl[(size_t)i]);
        if (!gone.empty()) {
            pools_[g].release(gone);
            for (int i = 0; i < first; i++) bl[(size_t)i] = kFreed;
            r.version = ++stamp_;
        }
    }
}

void BlockAllocator::release(RequestId rid) {
    Req& r = get(rid);
    for (size_t g = 0; g < r.blocks.size(); g++) {
        std::vector<int> held;
        for (int p : r.blocks[g])
            if (p != kFreed) held.push_back(p);
        pools_[g].release(held);
    }
    free_slots_.push_back(r.slot);
    requests_.erase(rid);
}

void BlockAllocator::check() const {
    for (size_t g = 0; g < pools_.size(); g++) {
        std::vector<int> held;
        for (const auto& kv : requests_)
            for (int p : kv.second.blocks[g])
                if (p != kFreed) held.push_back(p);
        const std::set<int> held_set(held.begin(), held.end());
        if (held_set.size() != held.size()) throw CacheError("group " + std::to_string(g) + ": a page is held twice");
        const auto& free = pools_[g].free_list();
        const std::set<int> free_set(free.begin(), free.end());
        if (free_set.size() != free.size()) throw CacheError("group " + std::to_string(g) + ": a page is on the free list twice");
        for (int p : held)
            if (free_set.count(p)) throw CacheError("group " + std::to_string(g) + ": a held page is on the free list");
        if ((int)(held.size() + free.size()) != pools_[g].num_pages())
            throw CacheError("group " + std::to_string(g) + ": " +
                             std::to_string(pools_[g].num_pages() - (int)held.size() - (int)free.size()) + " pages lost");
    }
    std::set<int> slots;
    for (const auto& kv : requests_) slots.insert(kv.second.slot);
    bool bad = slots.size() != requests_.size() || (int)(slots.size() + free_slots_.size()) != max_requests_;
    for (int s : free_slots_)
        if (slots.count(s)) bad = true;
    if (bad) throw CacheError("state slots are inconsistent");
}

// ---- device side ---------------------------------------------------------------------------------------
namespace {
void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw KernelError(std::string(what) + ": " + cudaGetErrorString(e));
}
}  // namespace

DeviceCaches::DeviceCaches(const CacheLayout& layout, const std::vector<int>& pages_per_group, int max_requests, DType dtype)
    : layout_(layout), pages_per_group_(pages_per_group), max_requests_(max_requests), dtype_(dtype) {
    for (size_t g = 0; g < layout.groups.size(); g++) {
        const CacheSpec& s = layout.groups[g].spec;
        const size_t bytes = layout.groups[g].caches.size() * (size_t)pages_per_group[g] * 2 * (size_t)s.n_kv_heads *
                             (size_t)layout.page_size * (size_t)s.head_dim * dtype_size(dtype);
        void* p = nullptr;
        cuda_ok(cudaMalloc(&p, std::max<size_t>(bytes, 16)), "allocating a cache arena");
        cuda_ok(cudaMemset(p, 0, std::max<size_t>(bytes, 16)), "clearing a cache arena");
        arenas_.push_back(p);
        arena_bytes_.push_back(bytes);
    }
    for (const auto& kv : layout.state_of_cache) {
        size_t n = (size_t)max_requests * dtype_size(kv.second.state_dtype);
        for (int64_t d : kv.second.state_shape) n *= (size_t)d;
        void* p = nullptr;
        cuda_ok(cudaMalloc(&p, std::max<size_t>(n, 16)), "allocating per-request state");
        cuda_ok(cudaMemset(p, 0, std::max<size_t>(n, 16)), "clearing per-request state");
        states_[kv.first] = p;
        state_bytes_[kv.first] = n;
    }
}

DeviceCaches::~DeviceCaches() {
    for (void* p : arenas_) cudaFree(p);
    for (auto& kv : states_) cudaFree(kv.second);
}

KVView DeviceCaches::kv(int cache) const {
    auto it = layout_.group_of_cache.find(cache);
    if (it == layout_.group_of_cache.end()) throw CacheError("cache entry " + std::to_string(cache) + " holds no pages");
    const int g = it->second.first, i = it->second.second;
    const CacheSpec& s = layout_.groups[(size_t)g].spec;
    const size_t esz = dtype_size(dtype_);
    const size_t head_block = (size_t)s.n_kv_heads * (size_t)layout_.page_size * (size_t)s.head_dim;     // one of K or V of a page
    const size_t page_elems = 2 * head_block;
    KVView v;
    char* base = (char*)arenas_[(size_t)g] + (size_t)i * (size_t)pages_per_group_[(size_t)g] * page_elems * esz;
    v.k = base;
    v.v = base + head_block * esz;
    v.page_stride = (long long)page_elems;
    v.num_pages = pages_per_group_[(size_t)g];
    v.n_kv_heads = s.n_kv_heads;
    v.page_size = layout_.page_size;
    v.head_dim = s.head_dim;
    v.group = g;
    v.dtype = dtype_;
    return v;
}

StateView DeviceCaches::state(int cache) const {
    auto it = states_.find(cache);
    if (it == states_.end()) throw CacheError("cache entry " + std::to_string(cache) + " holds no fixed-size state");
    const CacheSpec& s = layout_.state_of_cache.at(cache);
    StateView v;
    v.data = it->second;
    v.rows = max_requests_;
    v.shape = s.state_shape;
    v.row_elems = 1;
    for (int64_t d : s.state_shape) v.row_elems *= d;
    v.dtype = s.state_dtype;
    return v;
}

void DeviceCaches::zero_slot(int slot, void* stream) {
    for (const auto& kv : states_) {
        const size_t row = state_bytes_.at(kv.first) / (size_t)max_requests_;
        if (row) cuda_ok(cudaMemsetAsync((char*)kv.second + (size_t)slot * row, 0, row, (cudaStream_t)stream), "clearing a state slot");
    }
}

void DeviceCaches::poison(void* stream) {
    // all bits set is a NaN in float32 and in bfloat16
    for (size_t g = 0; g < arenas_.size(); g++)
        if (arena_bytes_[g]) cuda_ok(cudaMemsetAsync(arenas_[g], 0xff, arena_bytes_[g], (cudaStream_t)stream), "poisoning the cache");
}

size_t DeviceCaches::bytes() const {
    size_t n = 0;
    for (size_t b : arena_bytes_) n += b;
    for (const auto& kv : state_bytes_) n += kv.second;
    return n;
}

CacheManager::CacheManager(const std::vector<CacheSpec>& specs, int page_size, int64_t max_tokens, int max_requests,
                           DType dtype, void* stream)
    : stream_(stream) {
    CacheLayout layout = CacheLayout::from_specs(specs, page_size);
    const int n_pages = (int)std::max<int64_t>(1, (max_tokens + page_size - 1) / page_size);
    std::vector<int> per_group(layout.groups.size(), n_pages);
    alloc_.reset(new BlockAllocator(std::move(layout), per_group, max_requests));
    device_.reset(new DeviceCaches(alloc_->layout(), per_group, max_requests, dtype));
}

int CacheManager::admit(RequestId rid) {
    const int slot = alloc_->admit(rid);
    device_->zero_slot(slot, stream_);
    return slot;
}

size_t CacheManager::kv_bytes_per_token() const {
    size_t total = 0;
    for (const auto& g : alloc_->layout().groups)
        total += g.caches.size() * 2 * (size_t)g.spec.n_kv_heads * (size_t)g.spec.head_dim * dtype_size(device_->dtype());
    return total;
}

}  // namespace sandy
