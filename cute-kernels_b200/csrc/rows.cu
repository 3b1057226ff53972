// Row permutation kernels around the expert-parallel exchange: gather (optionally scaled) into a send
// buffer, k-way weighted combine of returned rows, and per-row dot products for the router-weight grad.
// All three stream whole rows with 16-byte vectors and accumulate in fp32 registers; they replace
// `group` with a coefficient (kernels/scattermoe/triton_implementation/kernels.py:225-280) and the
// bmm / sum(-2) combines of _ScatteredExperts (ops.py:170-174,214,276) when rows have crossed ranks.
#include "ck_common.cuh"

namespace ck {

constexpr int kRowThreads = 256;

template <typename T>
__device__ __forceinline__ void ld16f(const T *p, float (&v)[Vec16<T>::N]) {
    Vec16<T> r;
    *reinterpret_cast<int4 *>(&r) = __ldg(reinterpret_cast<const int4 *>(p));
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) v[i] = DT<T>::up(r.v[i]);
}
template <typename T>
__device__ __forceinline__ void up16f(const int4 &raw, float (&v)[Vec16<T>::N]) {  // 16 bytes already in registers
    Vec16<T> r;
    *reinterpret_cast<int4 *>(&r) = raw;
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) v[i] = DT<T>::up(r.v[i]);
}
template <typename T>
__device__ __forceinline__ void st16f(T *p, const float (&v)[Vec16<T>::N]) {
    Vec16<T> r;
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) r.v[i] = DT<T>::down(v[i]);
    *reinterpret_cast<int4 *>(p) = *reinterpret_cast<const int4 *>(&r);
}

// dst[j, :] = c * src[idx[j] / fan_out, :], c = coeff ? coeff[idx[j]] : 1; zeros where idx[j] < 0
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
    gather_rows_scaled_kernel(const T *__restrict__ src, T *__restrict__ dst, const int32_t *__restrict__ idx,
                              const T *__restrict__ coeff, int64_t n_rows, int fan_out, int64_t vpr) {
    constexpr int VEC = Vec16<T>::N;
    const int64_t nvec = n_rows * vpr;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t v = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += stride) {
        const int64_t j = v / vpr, c = (v - j * vpr) * VEC;
        const int32_t s = idx[j];
        float x[VEC];
        if (s >= 0) {
            ld16f(src + int64_t(s / fan_out) * (vpr * VEC) + c, x);
            if (coeff) {
                const float w = DT<T>::up(coeff[s]);
#pragma unroll
                for (int i = 0; i < VEC; ++i) x[i] *= w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) x[i] = 0.0f;
        }
        st16f(dst + v * VEC, x);
    }
}

// out[t, :] = sum_{j<k} (w ? w[t*k+j] : 1) * src[pos[t*k+j], :]
// The k rows are fetched kCombineBatch at a time, all loads of a batch issued before the first is used (one dependent
// pos -> row load per thread in flight leaves the copy latency bound); the sum keeps the order j = 0 .. k-1.
#ifndef CK_COMBINE_BATCH
#define CK_COMBINE_BATCH 4
#endif
constexpr int kCombineBatch = CK_COMBINE_BATCH;
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
    combine_rows_kernel(const T *__restrict__ src, const int32_t *__restrict__ pos, const T *__restrict__ w,
                        T *__restrict__ out, int64_t tokens, int k, int64_t vpr) {
    constexpr int VEC = Vec16<T>::N;
    const int64_t nvec = tokens * vpr;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t v = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += stride) {
        const int64_t t = v / vpr, c = (v - t * vpr) * VEC;
        float acc[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
        for (int j0 = 0; j0 < k; j0 += kCombineBatch) {
            int64_t r[kCombineBatch];
            float wj[kCombineBatch];
            int4 raw[kCombineBatch];
#pragma unroll
            for (int u = 0; u < kCombineBatch; ++u) {
                const int64_t f = t * k + j0 + u;
                r[u] = -1;  // pos == NULL: the k rows of token t are rows t*k .. t*k+k-1
                if (j0 + u < k) r[u] = pos ? int64_t(pos[f]) : f;
            }
#pragma unroll
            for (int u = 0; u < kCombineBatch; ++u) {
                raw[u] = make_int4(0, 0, 0, 0);
                wj[u] = 0.0f;
                if (r[u] >= 0) {
                    raw[u] = __ldg(reinterpret_cast<const int4 *>(src + r[u] * (vpr * VEC) + c));
                    wj[u] = w ? DT<T>::up(w[t * k + j0 + u]) : 1.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < kCombineBatch; ++u) {
                if (r[u] < 0) continue;  // an absent row adds nothing (not even a signed zero)
                float x[VEC];
                up16f<T>(raw[u], x);
#pragma unroll
                for (int i = 0; i < VEC; ++i) acc[i] = fmaf(wj[u], x[i], acc[i]);
            }
        }
        st16f(out + v * VEC, acc);
    }
}

// dots[f] = sum_c a[pos[f], c] * b[f / k, c]; one warp per f
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
    row_dots_kernel(const T *__restrict__ a, const int32_t *__restrict__ pos, const T *__restrict__ b,
                    T *__restrict__ dots, int64_t n, int k, int64_t vpr) {
    constexpr int VEC = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t f = warp; f < n; f += nwarps) {
        const int32_t r = pos[f];
        float acc = 0.0f;
        if (r >= 0) {
            const T *ar = a + int64_t(r) * (vpr * VEC);
            const T *br = b + (f / k) * (vpr * VEC);
            for (int64_t c = lane; c < vpr; c += 32) {
                float x[VEC], y[VEC];
                ld16f(ar + c * VEC, x);
                ld16f(br + c * VEC, y);
#pragma unroll
                for (int i = 0; i < VEC; ++i) acc = fmaf(x[i], y[i], acc);
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
        if (lane == 0) dots[f] = DT<T>::down(acc);
    }
}

static inline unsigned row_grid(int64_t work) {
    int64_t blocks = ceil_div64(work, kRowThreads);
    const int64_t cap = int64_t(num_sms()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return unsigned(blocks);
}
static inline bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static int gather_scaled_t(const void *src, void *dst, const int32_t *idx, const void *coeff, int64_t n_rows, int fan_out,
                           int64_t cols, cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    if (cols % VEC != 0 || !al16(src) || !al16(dst)) return CK_ERR_SHAPE;
    gather_rows_scaled_kernel<T><<<row_grid(n_rows * (cols / VEC)), kRowThreads, 0, stream>>>(
        (const T *)src, (T *)dst, idx, (const T *)coeff, n_rows, fan_out, cols / VEC);
    CK_LAUNCH_CHECK("gather_rows_scaled_kernel");
    return CK_OK;
}
template <typename T>
static int combine_t(const void *src, const int32_t *pos, const void *w, void *out, int64_t tokens, int k, int64_t cols,
                     cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    if (cols % VEC != 0 || !al16(src) || !al16(out)) return CK_ERR_SHAPE;
    combine_rows_kernel<T><<<row_grid(tokens * (cols / VEC)), kRowThreads, 0, stream>>>((const T *)src, pos, (const T *)w,
                                                                                  (T *)out, tokens, k, cols / VEC);
    CK_LAUNCH_CHECK("combine_rows_kernel");
    return CK_OK;
}
template <typename T>
static int dots_t(const void *a, const int32_t *pos, const void *b, void *dots, int64_t n, int k, int64_t cols,
                  cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    if (cols % VEC != 0 || !al16(a) || !al16(b)) return CK_ERR_SHAPE;
    row_dots_kernel<T><<<row_grid(n * 32), kRowThreads, 0, stream>>>((const T *)a, pos, (const T *)b, (T *)dots, n, k,
                                                                     cols / VEC);
    CK_LAUNCH_CHECK("row_dots_kernel");
    return CK_OK;
}

}  // namespace ck

using namespace ck;

#define CK_ROWS_DISPATCH(dtype, CALL)                           \
    switch (dtype) {                                            \
        case CK_BF16: { using T = __nv_bfloat16; return CALL; } \
        case CK_F16: { using T = __half; return CALL; }         \
        case CK_F32: { using T = float; return CALL; }          \
        default: return CK_ERR_UNSUPPORTED;                     \
    }

extern "C" int ck_moe_gather_rows_scaled(const void *src, void *dst, const int32_t *idx, const void *coeff, int64_t n_rows,
                                         int fan_out, int64_t cols, int dtype, void *stream) {
    if (n_rows < 0 || fan_out <= 0 || cols <= 0) return CK_ERR_SHAPE;
    if (n_rows == 0) return CK_OK;
    if (!src || !dst || !idx) return CK_ERR_SHAPE;
    CK_ROWS_DISPATCH(dtype, (gather_scaled_t<T>(src, dst, idx, coeff, n_rows, fan_out, cols, (cudaStream_t)stream)));
}

extern "C" int ck_moe_combine_rows(const void *src, const int32_t *pos, const void *w, void *out, int64_t tokens, int k,
                                   int64_t cols, int dtype, void *stream) {
    if (tokens < 0 || k <= 0 || cols <= 0) return CK_ERR_SHAPE;
    if (tokens == 0) return CK_OK;
    if (!src || !out) return CK_ERR_SHAPE;
    CK_ROWS_DISPATCH(dtype, (combine_t<T>(src, pos, w, out, tokens, k, cols, (cudaStream_t)stream)));
}

extern "C" int ck_moe_row_dots(const void *a, const int32_t *pos, const void *b, void *dots, int64_t n, int k,
                               int64_t cols, int dtype, void *stream) {
    if (n < 0 || k <= 0 || cols <= 0) return CK_ERR_SHAPE;
    if (n == 0) return CK_OK;
    if (!a || !pos || !b || !dots) return CK_ERR_SHAPE;
    CK_ROWS_DISPATCH(dtype, (dots_t<T>(a, pos, b, dots, n, k, cols, (cudaStream_t)stream)));
}
