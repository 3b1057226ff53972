// Shared device/host helpers of the sm_100a MoE expert-path library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ck_b200.h"

namespace ck {

// ---- host-side error plumbing ---------------------------------------------------------------
void set_last_cuda_error(cudaError_t err, const char *where);

#define CK_CUDA_TRY(expr)                                 \
    do {                                                  \
        cudaError_t _e = (expr);                          \
        if (_e != cudaSuccess) {                          \
            ck::set_last_cuda_error(_e, #expr);           \
            return CK_ERR_CUDA;                           \
        }                                                 \
    } while (0)

#define CK_LAUNCH_CHECK(where)                            \
    do {                                                  \
        cudaError_t _e = cudaGetLastError();              \
        if (_e != cudaSuccess) {                          \
            ck::set_last_cuda_error(_e, where);           \
            return CK_ERR_CUDA;                           \
        }                                                 \
    } while (0)

int num_sms();  // SM count of the current device (cached per device)

// ---- dtype traits ------------------------------------------------------------------------------
template <typename T>
struct DT;
template <>
struct DT<float> {
    static constexpr int code = CK_F32;
    __device__ __forceinline__ static float up(float v) { return v; }
    __device__ __forceinline__ static float down(float v) { return v; }
};
template <>
struct DT<__half> {
    static constexpr int code = CK_F16;
    __device__ __forceinline__ static float up(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half down(float v) { return __float2half_rn(v); }
};
template <>
struct DT<__nv_bfloat16> {
    static constexpr int code = CK_BF16;
    __device__ __forceinline__ static float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte vector of T
template <typename T>
struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

// ---- activation math (fp32) -------------------------------------------------------------------
// sigmoid with the argument clamped to +-88.3762626647949, as include/activations.h:9-22 does.
__device__ __forceinline__ float sigmoid_clamped(float x) {
    x = fmaxf(-88.3762626647949f, x);
    x = fminf(88.3762626647949f, x);
    return 1.0f / (1.0f + expf(-x));
}

// fast variant for GEMM epilogues (exp via ex2.approx); relative error ~1e-6
__device__ __forceinline__ float sigmoid_fast(float x) {
    x = fmaxf(-88.0f, fminf(88.0f, x));
    return __fdividef(1.0f, 1.0f + __expf(-x));
}

// ---- router ordering ----------------------------------------------------------------------------
// Total order on the logits: the key of a float grows with its value, every NaN maps to the largest key (torch.topk
// treats NaN as the greatest value) and -0.0 equals +0.0.  With (key, expert) compared lexicographically every lane of a
// butterfly reduction arrives at the same winner, whatever the row holds.
__device__ __forceinline__ uint32_t order_key(float v) {
    if (v != v) return 0xffffffffu;
    const uint32_t b = __float_as_uint(v + 0.0f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

__host__ __device__ __forceinline__ int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace ck
