// Token embedding with the learned position table added in the same pass.
//
//   x[t, :] = wte[id[t], :] + wpe[pos[t], :]
//
// The reference runs two gathers and an add (src/models/gpt2_small.sandy.go:48-50;
// gather kernel src/device/cuda/CudaGatherKernels.cu:97-117, one thread per element).
// Here one block writes one token's row; the sum is formed in 32-bit and rounded once.
// An id outside the table makes the reference's CPU path fail ("embedding id out of
// range", src/core/TensorCalc.cpp:1548-1549) and its CUDA path skip the element; this
// kernel writes zeros for the row and raises `*status` so the host can report it.
#include "common.cuh"

template <typename TT, typename TO>
__global__ void embed_pos_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                                 const TT* __restrict__ wte, const TT* __restrict__ wpe,
                                 TO* __restrict__ out, int width, int vocab, int n_pos,
                                 int* __restrict__ status) {
    // The first kernel of a step lets its successors start only after its own wait has returned: by then
    // every kernel of the steps before has completed, so the step's later kernels may read what those steps
    // wrote (cache pages of older positions, the index arrays) before their own waits.
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int id = ids[t];
    const int p = wpe ? pos[t] : 0;
    const bool ok = id >= 0 && id < vocab && (!wpe || (p >= 0 && p < n_pos));
    if (!ok && threadIdx.x == 0 && status) atomicOr(status, (id >= 0 && id < vocab) ? 2 : 1);
    const TT* trow = wte + (size_t)(ok ? id : 0) * width;
    const TT* prow = wpe ? wpe + (size_t)(ok ? p : 0) * width : nullptr;
    TO* orow = out + (size_t)t * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float v = 0.0f;
        if (ok) {
            v = to_f32(trow[e]);
            if (prow) v += to_f32(prow[e]);
        }
        orow[e] = from_f32<TO>(v);
    }
}

// ids, pos: int32[n_tokens]; wte: [vocab, width]; wpe: [n_pos, width] or null (no table);
// out: [n_tokens, width].  status: device int, bit 0 = bad token id, bit 1 = bad position.
SANDY_API int sandy_embed_pos(const int* ids, const int* pos, const void* wte, const void* wpe,
                              void* out, int n_tokens, int width, int vocab, int n_pos,
                              int table_dtype, int out_dtype, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!ids || !wte || !out || width <= 0) return SANDY_ERR_ARGUMENT;
    const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
#define LAUNCH(TT, TO)                                                                          \
    return sandy_launch(embed_pos_kernel<TT, TO>, dim3(n_tokens), dim3(threads), 0, stream, ids, pos,  \
                        (const TT*)wte, (const TT*)wpe, (TO*)out, width, vocab, n_pos, status)
    if (table_dtype == SANDY_F32 && out_dtype == SANDY_F32) LAUNCH(float, float);
    if (table_dtype == SANDY_BF16 && out_dtype == SANDY_F32) LAUNCH(bf16, float);
    if (table_dtype == SANDY_BF16 && out_dtype == SANDY_BF16) LAUNCH(bf16, bf16);
#undef LAUNCH
    return SANDY_ERR_UNSUPPORTED;
}

// ---- small device utilities the host side uses -------------------------------------------------
SANDY_API int sandy_device_sm_count() { return sandy_sm_count(); }

// Keeps the stream busy for about `nanoseconds` (at most 10 ms) and does nothing else.  Timing
// loops queue their launches behind it, so that the GPU runs them back to back instead of at
// the pace the host issues them.
__global__ void spin_kernel(unsigned long long nanoseconds) {
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    do {
        __nanosleep(200);
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    } while (t - t0 < nanoseconds);
}

SANDY_API int sandy_spin(long long nanoseconds, cudaStream_t stream) {
    if (nanoseconds <= 0) return SANDY_OK;
    if (nanoseconds > 10000000LL) nanoseconds = 10000000LL;
    spin_kernel<<<1, 1, 0, stream>>>((unsigned long long)nanoseconds);
    return sandy_launch_status();
}
