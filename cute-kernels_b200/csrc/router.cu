// Router tail: top-k over the expert logits, softmax over the k selected logits, int32 expert ids.
//
// Replaces the three torch launches after the gate GEMM in MoE_Torch._compute_routing_weights
// (kernels/scattermoe/torch_implementation.py:122-135,195-201: topk / max, softmax(float), type_as) and
// emits the ids as int32 in the layout ck_route reads, instead of an int64 [T, k] tensor.  One warp per
// token; the logits row lives in registers (up to 256 experts), the k winners are extracted by k warp-wide
// arg-max rounds (ties go to the lower expert index).  The gate GEMM itself stays a library GEMM.
#include "ck_common.cuh"

namespace ck {

constexpr int kRouterMaxExperts = 256;
constexpr int kRouterMaxK = 32;
constexpr int kRouterThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kRouterThreads)
    router_topk_softmax_kernel(const T *__restrict__ logits, T *__restrict__ weights, int32_t *__restrict__ ids,
                               int64_t tokens, int E, int k) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    constexpr int kPerLane = kRouterMaxExperts / 32;
    constexpr int kNone = 0x7fffffff;
    for (int64_t t = warp; t < tokens; t += nwarps) {
        uint32_t key[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int e = lane + 32 * i;
            key[i] = e < E ? order_key(DT<T>::up(logits[t * E + e])) : 0u;  // real keys are >= 0x007fffff (-inf)
        }
        float my_val = 0.0f;  // lane j keeps the j-th winner
        int my_idx = 0;
        float vmax = 0.0f;
        unsigned taken = 0u;  // bit i: this lane's i-th logit is already among the winners
        for (int j = 0; j < k; ++j) {
            uint32_t best = 0u;
            int best_e = kNone;
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) {
                const int e = lane + 32 * i;
                // any candidate not yet taken beats "none": masked (-inf) and NaN logits still give k distinct experts
                if (e < E && !((taken >> i) & 1u) && key[i] > best) {
                    best = key[i];
                    best_e = e;
                }
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                const uint32_t ob = __shfl_xor_sync(0xffffffffu, best, d);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, d);
                if (ob > best || (ob == best && oe < best_e)) {
                    best = ob;
                    best_e = oe;
                }
            }
            // one winner for the whole warp, whatever the lanes computed
            best = __shfl_sync(0xffffffffu, best, 0);
            best_e = __shfl_sync(0xffffffffu, best_e, 0);
            const float best_v = key_value(best);
            if (j == 0) vmax = best_v;
            if (lane == j) {
                my_val = best_v;
                my_idx = best_e != kNone ? best_e : 0;  // k <= E, so a candidate always exists; never emit an id outside [0, E)
            }
            if (best_e != kNone && (best_e & 31) == lane) taken |= 1u << (best_e >> 5);  // the owner retires the winner
        }
        // softmax over the k selected logits in fp32 (k <= 32: one per lane); -inf - -inf and NaN rows give NaN weights
        // as torch.softmax does
        const float ex = lane < k ? expf(my_val - vmax) : 0.0f;
        float sum = ex;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        if (lane < k) {
            weights[t * k + lane] = DT<T>::down(ex / sum);
            ids[t * k + lane] = my_idx;
        }
    }
}

// d_logits[t, :] = 0 except d_logits[t, ids[t, j]] = w_j * (dw_j - sum_i w_i dw_i)   (softmax backward, fp32)
template <typename T>
__global__ void __launch_bounds__(kRouterThreads)
    router_topk_softmax_bwd_kernel(const T *__restrict__ weights, const T *__restrict__ d_weights,
                                   const int32_t *__restrict__ ids, T *__restrict__ d_logits, int64_t tokens, int E, int k,
                                   int32_t *__restrict__ dev_status) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t t = warp; t < tokens; t += nwarps) {
        const float w = lane < k ? DT<T>::up(weights[t * k + lane]) : 0.0f;
        const float dw = lane < k ? DT<T>::up(d_weights[t * k + lane]) : 0.0f;
        float dot = w * dw;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
        for (int e = lane; e < E; e += 32) d_logits[t * E + e] = DT<T>::down(0.0f);
        __syncwarp();
        if (lane < k) {
            const int32_t e = ids[t * k + lane];
            if (e >= 0 && e < E) d_logits[t * E + e] = DT<T>::down(w * (dw - dot));
            else if (dev_status) atomicOr(dev_status, CK_DEV_RANGE);  // an id outside [0, E) is skipped, never written through
        }
    }
}

static inline unsigned router_grid(int64_t tokens) {
    int64_t blocks = ceil_div64(tokens, kRouterThreads / 32);
    const int64_t cap = int64_t(num_sms()) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return unsigned(blocks);
}

}  // namespace ck

using namespace ck;

extern "C" int ck_router_topk_softmax(const void *logits, void *weights, int32_t *ids, int64_t tokens, int E, int k,
                                      int dtype, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (tokens < 0 || E <= 0 || k <= 0 || k > E) return CK_ERR_SHAPE;
    if (E > kRouterMaxExperts || k > kRouterMaxK) return CK_ERR_RANGE;
    if (tokens == 0) return CK_OK;
    if (!logits || !weights || !ids) return CK_ERR_SHAPE;
    switch (dtype) {
        case CK_F32: router_topk_softmax_kernel<float><<<router_grid(tokens), kRouterThreads, 0, stream>>>((const float *)logits, (float *)weights, ids, tokens, E, k); break;
        case CK_F16: router_topk_softmax_kernel<__half><<<router_grid(tokens), kRouterThreads, 0, stream>>>((const __half *)logits, (__half *)weights, ids, tokens, E, k); break;
        case CK_BF16: router_topk_softmax_kernel<__nv_bfloat16><<<router_grid(tokens), kRouterThreads, 0, stream>>>((const __nv_bfloat16 *)logits, (__nv_bfloat16 *)weights, ids, tokens, E, k); break;
        default: return CK_ERR_UNSUPPORTED;
    }
    CK_LAUNCH_CHECK("router_topk_softmax_kernel");
    return CK_OK;
}

extern "C" int ck_router_topk_softmax_bwd(const void *weights, const void *d_weights, const int32_t *ids, void *d_logits,
                                          int64_t tokens, int E, int k, int dtype, int32_t *dev_status, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (tokens < 0 || E <= 0 || k <= 0 || k > E) return CK_ERR_SHAPE;
    if (k > kRouterMaxK) return CK_ERR_RANGE;
    if (tokens == 0) return CK_OK;
    if (!weights || !d_weights || !ids || !d_logits) return CK_ERR_SHAPE;
    switch (dtype) {
        case CK_F32: router_topk_softmax_bwd_kernel<float><<<router_grid(tokens), kRouterThreads, 0, stream>>>((const float *)weights, (const float *)d_weights, ids, (float *)d_logits, tokens, E, k, dev_status); break;
        case CK_F16: router_topk_softmax_bwd_kernel<__half><<<router_grid(tokens), kRouterThreads, 0, stream>>>((const __half *)weights, (const __half *)d_weights, ids, (__half *)d_logits, tokens, E, k, dev_status); break;
        case CK_BF16: router_topk_softmax_bwd_kernel<__nv_bfloat16><<<router_grid(tokens), kRouterThreads, 0, stream>>>((const __nv_bfloat16 *)weights, (const __nv_bfloat16 *)d_weights, ids, (__nv_bfloat16 *)d_logits, tokens, E, k, dev_status); break;
        default: return CK_ERR_UNSUPPORTED;
    }
    CK_LAUNCH_CHECK("router_topk_softmax_bwd_kernel");
    return CK_OK;
}
