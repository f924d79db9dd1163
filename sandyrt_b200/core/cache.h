// The cache manager: page pools, per-request block lists, state slots (host side), and the page
// arenas and per-request states on the device.
//
// What the reference does (one request at a time): a pool of fixed-size pages with a LIFO free
// list, optional page cap, double-free detection (src/core/Allocator.cpp:60-122,
// src/device/cuda/CudaPagedTensor.cpp:232-267); growth by ceil(new_len / page_size) pages
// (:95-137, :555-576); everything returned when the request's session ends (:528-553,
// src/server/Session.cpp:552-563); one list of cache groups per model (`CacheGroupConfig`,
// src/server/Session.h:36-41, src/server/Model.cpp:106-111); every page a separate
// cudaMallocAsync allocation and a table of page pointers per tensor (:232-267, :345-447).
//
// What is different here: the lowest free page goes out first (so that a prompt's pages tend to
// be a run); many requests live at once and share the pools; a request has one block list per
// *group* (all layers of a group use the same page ids), not one page table per tensor; pages of
// a group whose layers only look back `window` positions are given back as soon as the window has
// passed them; every request also holds one *state slot*, a row index into per-request state of
// fixed size; and a page is an index into one arena per group, allocated once:
// [caches in group][num_pages][K|V][Hkv][page_size][D] in the compute dtype.
//
// Everything up to BlockAllocator touches no device, so every decision about pages can be tested
// on a machine without a GPU.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include "errors.h"

namespace sandy {

using RequestId = int64_t;
constexpr int kFreed = -1;      // entry of a block list whose page has been given back (the window has passed it)

enum class DType : int { F32 = 0, BF16 = 1, I32 = 2 };       // F32 and BF16 are the codes the kernels take
size_t dtype_size(DType d);
const char* dtype_name(DType d);

// What a mixer may ask of the cache manager.
struct CacheSpec {
    enum class Kind { None, PagedKV, State };
    Kind kind = Kind::None;
    // PagedKV: keys and values of every position (or of the last `window` positions) in pages
    int n_kv_heads = 0, head_dim = 0;
    int window = 0;                        // 0: all positions stay; n: only the last n are read
    // State: a per-request state of fixed size (a recurrent state, a convolution tail, ...).  It
    // lives in the request's state slot and starts as zeros when the request is admitted.
    std::vector<int64_t> state_shape;
    DType state_dtype = DType::F32;

    static CacheSpec none() { return CacheSpec(); }
    static CacheSpec paged(int n_kv_heads, int head_dim, int window = 0);
    static CacheSpec state(std::vector<int64_t> shape, DType dtype = DType::F32);
    bool operator==(const CacheSpec& o) const;
    bool operator!=(const CacheSpec& o) const { return !(*this == o); }
};

// Page ids 0..num_pages-1; the free page with the lowest id is handed out first (the reference's
// pool is a LIFO list).  A fresh pool hands out 0, 1, 2, ..., and whenever the low end of the pool
// is free again a request's pages follow one another in the cache: the prompt attention kernel
// fetches such runs with one copy per tile.  With few pages a page just freed is still handed out
// again at once.
class PagePool {
public:
    explicit PagePool(int num_pages);
    int num_pages() const { return num_pages_; }
    int free_pages() const { return (int)free_.size(); }
    int used_pages() const { return num_pages_ - (int)free_.size(); }
    int high_water() const { return high_water_; }
    std::vector<int> allocate(int n);                 // OutOfPages if fewer are free; nothing is taken then
    void release(const std::vector<int>& pages);      // CacheError on a foreign page or a page freed twice
    const std::vector<int>& free_list() const { return free_; }
private:
    int num_pages_;
    std::vector<int> free_;          // a min-heap
    std::vector<char> held_;
    int high_water_ = 0;
};

// Cache entries with the same needs; they share page ids and one pool.
struct CacheGroup {
    int index = 0;
    CacheSpec spec;
    std::vector<int> caches;         // cache entries (of the model's run order) in this group
};

// How a model's cache entries fall into paged groups and fixed-size states.
struct CacheLayout {
    int page_size = 16;
    std::vector<CacheGroup> groups;
    std::map<int, std::pair<int, int>> group_of_cache;      // cache entry -> (group, index inside group)
    std::map<int, CacheSpec> state_of_cache;                // cache entry -> fixed-size state
    static CacheLayout from_specs(const std::vector<CacheSpec>& specs, int page_size);
};

// Pages and slots of all live requests.
//   admit(rid)              take a state slot; the request holds no pages yet
//   reserve(rid, new_len)   make room for positions < new_len in every group (all or nothing)
//   commit(rid, new_len)    the step ran: the request now holds new_len tokens; pages a window
//                           has passed are given back
//   release(rid)            the request ended: everything it holds is given back
class BlockAllocator {
public:
    BlockAllocator(CacheLayout layout, const std::vector<int>& pages_per_group, int max_requests);
    const CacheLayout& layout() const { return layout_; }
    int page_size() const { return layout_.page_size; }
    int max_requests() const { return max_requests_; }
    int n_groups() const { return (int)pools_.size(); }
    const PagePool& pool(int group) const { return pools_.at((size_t)group); }

    bool contains(RequestId rid) const { return requests_.count(rid) != 0; }
    std::vector<RequestId> live() const;
    int slot(RequestId rid) const { return get(rid).slot; }
    int length(RequestId rid) const { return get(rid).length; }
    // A number that changes whenever any of the request's block lists changes; a request that is
    // released and admitted again under the same id gets a new one.
    uint64_t block_version(RequestId rid) const { return get(rid).version; }
    const std::vector<int>& block_list(RequestId rid, int group) const { return get(rid).blocks.at((size_t)group); }
    int free_slots() const { return (int)free_slots_.size(); }
    int free_pages(int group = 0) const { return pools_.at((size_t)group).free_pages(); }
    std::vector<int> pages_needed(RequestId rid, int new_len) const;     // per group, for reserve(rid, new_len)
    std::vector<int> pages_for_new_request(int n_tokens) const;
    bool can_reserve(RequestId rid, int new_len) const;

    int admit(RequestId rid);
    void reserve(RequestId rid, int new_len);
    void commit(RequestId rid, int new_len);
    void release(RequestId rid);
    // No page lost, held twice or free while held; no slot lost or shared (tests call this after
    // every operation).  Throws CacheError.
    void check() const;

private:
    struct Req {
        int slot = 0;
        int length = 0;                        // tokens whose keys/values are in the cache
        std::vector<std::vector<int>> blocks;  // per group: page id per block index, kFreed where given back
        uint64_t version = 0;
    };
    const Req& get(RequestId rid) const;
    Req& get(RequestId rid);
    int first_needed_block(int group, int length) const;
    CacheLayout layout_;
    std::vector<PagePool> pools_;
    int max_requests_;
    std::vector<int> free_slots_;
    std::unordered_map<RequestId, Req> requests_;
    uint64_t stamp_ = 0;
};

// ---- device side ---------------------------------------------------------------------------------
// A view of one cache entry's keys and values: [num_pages, Hkv, page_size, D], dense inside a page.
struct KVView {
    void* k = nullptr;
    void* v = nullptr;
    long long page_stride = 0;     // elements between two pages of this entry
    int num_pages = 0, n_kv_heads = 0, page_size = 0, head_dim = 0;
    int group = 0;
    DType dtype = DType::F32;
};

struct StateView {
    void* data = nullptr;          // [max_requests, *shape]
    int rows = 0;                  // max_requests
    std::vector<int64_t> shape;    // of one request's state
    int64_t row_elems = 0;
    DType dtype = DType::F32;
};

class DeviceCaches {
public:
    DeviceCaches(const CacheLayout& layout, const std::vector<int>& pages_per_group, int max_requests, DType dtype);
    ~DeviceCaches();
    DeviceCaches(const DeviceCaches&) = delete;
    DeviceCaches& operator=(const DeviceCaches&) = delete;
    KVView kv(int cache) const;
    StateView state(int cache) const;
    void zero_slot(int slot, void* stream);      // a request was admitted: its fixed-size states start as zeros
    void poison(void* stream);                   // fill every page with NaN (tests: a read of a slot nobody wrote then shows)
    size_t bytes() const;
    DType dtype() const { return dtype_; }
private:
    const CacheLayout& layout_;
    std::vector<int> pages_per_group_;
    int max_requests_;
    DType dtype_;
    std::vector<void*> arenas_;
    std::vector<size_t> arena_bytes_;
    std::map<int, void*> states_;
    std::map<int, size_t> state_bytes_;
};

// BlockAllocator + DeviceCaches for one model on one device.
class CacheManager {
public:
    CacheManager(const std::vector<CacheSpec>& specs, int page_size, int64_t max_tokens, int max_requests, DType dtype,
                 void* stream);
    BlockAllocator& alloc() { return *alloc_; }
    const BlockAllocator& alloc() const { return *alloc_; }
    DeviceCaches& device() { return *device_; }
    const CacheLayout& layout() const { return alloc_->layout(); }
    int page_size() const { return alloc_->page_size(); }
    int max_requests() const { return alloc_->max_requests(); }
    int admit(RequestId rid);                    // takes a slot and zeroes its fixed-size state
    void release(RequestId rid) { alloc_->release(rid); }
    size_t kv_bytes_per_token() const;
private:
    std::unique_ptr<BlockAllocator> alloc_;
    std::unique_ptr<DeviceCaches> device_;
    void* stream_;
};

}  // namespace sandy
