// Next-token choice on the device: greedy, temperature, top-k and top-p, one block per row.
//
// Meaning of the options follows the reference's host sampler (src/server/Sampler.cpp:55-107):
//   1. order the logits from high to low, ties by lower id first (stable sort, :69-74);
//   2. keep the first top_k (:75-76);
//   3. temperature 0, or a non-finite best logit: return the first (:78-79);
//   4. weights w = exp(logit/T - best/T) (:81-91);
//   5. keep the shortest prefix whose cumulative share reaches top_p (:95-100);
//   6. draw from the kept prefix in proportion to w (:102-106).
// The reference sorts on the host and draws with std::discrete_distribution.  Here nothing
// is sorted: the k-th largest logit and the top-p cut are found by bisection on the value
// (a count, or a sum of weights, of everything at or above a trial value), and ties at a
// cut are admitted in id order, which is what a stable sort would do.  The draw is an
// inverse CDF over the kept set in id order with one uniform number per row that the
// caller supplies, so a request's tokens depend on its own seed and step only.
// top_k <= 0 means "no top-k cut" (the whole vocabulary).
//
// A NaN among the logits is an error in the reference (:64-67); here the row's result is
// -1 and bit 0 of *status is raised.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

// Monotone map float -> uint32 (larger float, larger key).
__device__ __forceinline__ unsigned order_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned k) {
    const unsigned b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int t = (lane < (THREADS >> 5)) ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// Exclusive prefix over the block of one float per thread; returns this thread's prefix
// and writes the block total to *total.  Order of additions is fixed.
__device__ __forceinline__ float block_exclusive_scan(float v, float* scratch, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    float wsum = (lane < (THREADS >> 5)) ? scratch[lane] : 0.0f;
    float winc = wsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += n;
    }
    const float warp_prefix = __shfl_sync(0xffffffffu, winc - wsum, warp);
    *total = __shfl_sync(0xffffffffu, winc, 31);
    return warp_prefix + (inc - v);
}

__device__ __forceinline__ int block_exclusive_scan_int(int v, int* scratch, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    int wsum = (lane < (THREADS >> 5)) ? scratch[lane] : 0;
    int winc = wsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += n;
    }
    const int warp_prefix = __shfl_sync(0xffffffffu, winc - wsum, warp);
    *total = __shfl_sync(0xffffffffu, winc, 31);
    return warp_prefix + (inc - v);
}

// Feeding the drawn token straight back into the next decode step, on the device.  When
// `token_ids` is set, the row's token is also written over the step's input token of that row
// (token_ids[logit_rows[r]]), the row's position moves on by one, and the token is recorded
// in out_tokens[step * n_rows + r], where `step` is the row's own counter row_step[r] (it also
// selects the row's uniform number, uniform[step * n_rows + r]).  A whole run of decode steps
// can then be replayed back to back with no trip to the host in between.
struct Advance {
    int* token_ids;
    const int* logit_rows;
    int* positions;
    int* out_tokens;
    int* row_step;
    int n_rows;
};

__device__ __forceinline__ void emit_token(int r, int tok, int* __restrict__ out_token, const Advance& adv, int step) {
    out_token[r] = tok;
    if (adv.token_ids) {
        const int t = adv.logit_rows[r];
        adv.token_ids[t] = tok;
        adv.positions[t] += 1;
        adv.out_tokens[(size_t)step * adv.n_rows + r] = tok;
        adv.row_step[r] = step + 1;
    }
}

// One block per row.  Each thread owns the contiguous id range [begin, end) so that
// "in id order" is "in thread order, then in the thread's own order".
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out_token, int* __restrict__ status, Advance adv) {
    __shared__ float fscratch[32];
    __shared__ int iscratch[32];
    __shared__ float best_val_s[32];
    __shared__ int best_idx_s[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int step = adv.token_ids ? adv.row_step[r] : 0;
    const int per = (vocab + THREADS - 1) / THREADS;
    const int begin = min(vocab, tid * per), end = min(vocab, begin + per);

    // ---- greedy: first index of the maximum; NaN check -----------------------------
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    int has_nan = 0;
    // This pass reads the row strided (thread t takes ids t, t + THREADS, ...: whole cache lines per
    // warp; with each thread on its own contiguous range it cost 13 us for 8 rows of 50257).  A
    // thread meets its ids in ascending order, so it keeps the first of equal values, and the
    // merges below prefer the lower id: the result is the first maximum whatever the layout.
    for (int i = tid; i < vocab; i += THREADS) {
        const float v = row[i];
        if (v != v) has_nan = 1;
        if (v > bv || bi == 0x7fffffff) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { best_val_s[warp] = bv; best_idx_s[warp] = bi; }
    has_nan = block_sum_int(has_nan, iscratch);  // includes __syncthreads
    bv = best_val_s[lane];
    bi = best_idx_s[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (has_nan) {
        if (tid == 0) { emit_token(r, -1, out_token, adv, step); if (status) atomicOr(status, 1); }
        return;
    }
    const float T = temperature ? temperature[r] : 0.0f;
    if (T == 0.0f || !isfinite(bv)) {
        if (tid == 0) emit_token(r, bi, out_token, adv, step);
        return;
    }
    const float best = bv;
    const float invT = 1.0f / T;
    const int k = top_k ? top_k[r] : 0;
    const float p_keep = top_p ? top_p[r] : 1.0f;

    // ---- top-k: value of the k-th largest logit, and how many ties at it are kept ------
    unsigned cut_key = 0u;      // keep everything with key > cut_key, and `ties_kept` of key == cut_key
    int ties_kept = 0x7fffffff; // in id order
    if (k > 0 && k < vocab) {
        unsigned lo = 0u, hi = 0xffffffffu;  // invariant: count(key >= lo) >= k
        while (lo < hi) {
            const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
            int c = 0;
            for (int i = tid; i < vocab; i += THREADS) c += order_key(row[i]) >= mid;    // a count: any order
            c = block_sum_int(c, iscratch);
            if (c >= k) lo = mid; else hi = mid - 1u;
        }
        cut_key = lo;
        int above = 0;
        for (int i = tid; i < vocab; i += THREADS) above += order_key(row[i]) > cut_key;
        above = block_sum_int(above, iscratch);
        ties_kept = k - above;
    }

    // ---- top-p inside the top-k set -------------------------------------------------------
    // member(i): key > cut_key, or key == cut_key and it is among the first ties_kept such ids.
    // Rank of a tie among the ties, in id order:
    int my_ties = 0;
    for (int i = begin; i < end; i++) my_ties += order_key(row[i]) == cut_key;
    int tie_total;
    const int tie_prefix = block_exclusive_scan_int(my_ties, iscratch, &tie_total);

    auto weight = [&](float v) { return expf(v * invT - best * invT); };

    float total = 0.0f;
    {
        int tr = tie_prefix;
        for (int i = begin; i < end; i++) {
            const unsigned key = order_key(row[i]);
            bool in = key > cut_key;
            if (key == cut_key) { in = tr < ties_kept; tr++; }
            if (in) total += weight(row[i]);
        }
        total = block_sum(total, fscratch);
    }

    unsigned p_key = cut_key;         // final cut: keep key > p_key fully ...
    float tie_budget = INFINITY;      // ... and ties at p_key (in id order, inside the top-k set)
                                      // while the cumulative share before them is < top_p
    float mass_above = 0.0f;
    bool p_active = p_keep < 1.0f;
    if (p_active) {
        // largest key value v with  share(key >= v, members) >= top_p
        unsigned lo = cut_key, hi = order_key(best);
        while (lo < hi) {
            const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
            float sum = 0.0f;
            int tr = tie_prefix;
            for (int i = begin; i < end; i++) {
                const unsigned key = order_key(row[i]);
                bool in = key > cut_key;
                if (key == cut_key) { in = tr < ties_kept; tr++; }
                if (in && key >= mid) sum += weight(row[i]);
            }
            sum = block_sum(sum, fscratch);
            if (sum / total >= p_keep) lo = mid; else hi = mid - 1u;
        }
        p_key = lo;
        float sum = 0.0f;
        for (int i = begin; i < end; i++)
            if (order_key(row[i]) > p_key) sum += weight(row[i]);
        mass_above = block_sum(sum, fscratch);
        tie_budget = p_keep;
    }

    // ---- kept set and its total ------------------------------------------------------------
    // kept(i): key > p_key, or key == p_key and (it is a top-k member) and the cumulative share
    // of everything before it in sorted order, mass_above + (ties before it)*w, is < top_p.
    const float w_tie = weight(key_value(p_key));
    int my_pties = 0;
    {
        int tr = tie_prefix;
        for (int i = begin; i < end; i++) {
            const unsigned key = order_key(row[i]);
            bool member = key > cut_key;
            if (key == cut_key) { member = tr < ties_kept; tr++; }
            my_pties += (member && key == p_key);
        }
    }
    int ptie_total;
    const int ptie_prefix = block_exclusive_scan_int(my_pties, iscratch, &ptie_total);

    auto kept_weight = [&](int i, int& tr, int& pr) -> float {
        const float v = row[i];
        const unsigned key = order_key(v);
        bool member = key > cut_key;
        if (key == cut_key) { member = tr < ties_kept; tr++; }
        if (!member) return 0.0f;
        if (key > p_key) return weight(v);
        if (key < p_key) return 0.0f;
        bool in = true;
        if (p_active) in = (mass_above + (float)pr * w_tie) / total < tie_budget;
        pr++;
        return in ? w_tie : 0.0f;
    };

    float mine = 0.0f;
    {
        int tr = tie_prefix, pr = ptie_prefix;
        for (int i = begin; i < end; i++) mine += kept_weight(i, tr, pr);
    }
    float kept_total;
    const float prefix = block_exclusive_scan(mine, fscratch, &kept_total);

    // ---- inverse CDF in id order -----------------------------------------------------------
    const float target = uniform[(size_t)step * (adv.token_ids ? adv.n_rows : 0) + r] * kept_total;
    // The thread whose [prefix, prefix+mine) holds the target walks its range.  The last
    // thread with any weight also takes targets that rounding pushed past the end.
    __shared__ int chosen;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (mine > 0.0f && target >= prefix && target < prefix + mine) {
        int tr = tie_prefix, pr = ptie_prefix;
        float cum = prefix;
        int pick = -1;
        for (int i = begin; i < end; i++) {
            const float w = kept_weight(i, tr, pr);
            if (w > 0.0f) {
                pick = i;
                cum += w;
                if (target < cum) break;
            }
        }
        chosen = pick;
    }
    __syncthreads();
    if (chosen < 0) {
        // rounding: target landed on or beyond the last boundary; take the last kept id
        __shared__ int last_kept;
        if (tid == 0) last_kept = -1;
        __syncthreads();
        if (mine > 0.0f) {
            int tr = tie_prefix, pr = ptie_prefix, pick = -1;
            for (int i = begin; i < end; i++)
                if (kept_weight(i, tr, pr) > 0.0f) pick = i;
            atomicMax(&last_kept, pick);
        }
        __syncthreads();
        if (tid == 0) chosen = last_kept >= 0 ? last_kept : bi;
        __syncthreads();
    }
    if (tid == 0) emit_token(r, chosen, out_token, adv, step);
}

}  // namespace

// logits: float [n_rows, vocab] with row stride ld.  temperature, top_k, top_p, uniform:
// per-row arrays on the device (temperature null = greedy for all rows; top_k null = no
// cut; top_p null = 1).  out_token: int32[n_rows].
// Feedback (all null to switch it off): token_ids / positions are the step's input arrays,
// logit_rows[r] the input row that row r's token replaces, out_tokens an int32 array of
// [steps][n_rows], row_step int32[n_rows] counters (start them at 0); `uniform` then holds
// [steps][n_rows] numbers.
SANDY_API int sandy_sample(const float* logits, int ld, int n_rows, int vocab,
                           const float* temperature, const int* top_k, const float* top_p,
                           const float* uniform, int* out_token, int* status, int* token_ids,
                           const int* logit_rows, int* positions, int* out_tokens, int* row_step,
                           cudaStream_t stream) {
    if (n_rows == 0) return SANDY_OK;
    if (!logits || !out_token || vocab <= 0) return SANDY_ERR_ARGUMENT;
    if (temperature && !uniform) return SANDY_ERR_ARGUMENT;
    if (token_ids && (!logit_rows || !positions || !out_tokens || !row_step)) return SANDY_ERR_ARGUMENT;
    Advance adv{token_ids, logit_rows, positions, out_tokens, row_step, n_rows};
    return sandy_launch(sample_kernel, dim3(n_rows), dim3(THREADS), 0, stream, logits, ld, vocab, temperature, top_k,
                        top_p, uniform, out_token, status, adv);
}
