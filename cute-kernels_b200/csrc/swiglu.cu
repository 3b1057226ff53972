// Stand-alone SwiGLU forward / backward, row-gather and fp32 -> T cast.
//
// All four are streaming, HBM-bound kernels: 16-byte vector loads and stores, several independent
// vectors in flight per thread, a grid that is a multiple of the SM count.  Rows may be strided
// (the packed [up | gate] form passes two views of one buffer).
#include "ck_common.cuh"

namespace ck {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;

template <typename T>
__device__ __forceinline__ Vec16<T> ldg16(const T *p) {
    Vec16<T> r;
    *reinterpret_cast<int4 *>(&r) = __ldg(reinterpret_cast<const int4 *>(p));
    return r;
}
template <typename T>
__device__ __forceinline__ void stg16(T *p, const Vec16<T> &v) {
    *reinterpret_cast<int4 *>(p) = *reinterpret_cast<const int4 *>(&v);
}

// ---- 16 bytes <-> fp32 lanes with paired conversions (one instruction per two 16-bit elements) ----
template <typename T>
struct Lanes;  // N fp32 values per 16-byte vector
template <>
struct Lanes<float> {
    static constexpr int N = 4;
    __device__ __forceinline__ static void unpack(const int4 &r, float (&v)[4]) {
        v[0] = __int_as_float(r.x); v[1] = __int_as_float(r.y); v[2] = __int_as_float(r.z); v[3] = __int_as_float(r.w);
    }
    __device__ __forceinline__ static int4 pack(const float (&v)[4]) {
        return make_int4(__float_as_int(v[0]), __float_as_int(v[1]), __float_as_int(v[2]), __float_as_int(v[3]));
    }
};
template <>
struct Lanes<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void unpack(const int4 &r, float (&v)[8]) {
        const uint32_t w[4] = {uint32_t(r.x), uint32_t(r.y), uint32_t(r.z), uint32_t(r.w)};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // bf16 is the upper half of an fp32
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static int4 pack(const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        return make_int4(int(w[0]), int(w[1]), int(w[2]), int(w[3]));
    }
};
template <>
struct Lanes<__half> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void unpack(const int4 &r, float (&v)[8]) {
        const uint32_t w[4] = {uint32_t(r.x), uint32_t(r.y), uint32_t(r.z), uint32_t(r.w)};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    __device__ __forceinline__ static int4 pack(const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        return make_int4(int(w[0]), int(w[1]), int(w[2]), int(w[3]));
    }
};

// sigmoid for the streaming kernels.  fp32 tensors keep the clamped expf form of the reference
// (include/activations.h:9-22).  For 16-bit tensors a B200 at full HBM rate has to retire about one
// element per SM per clock; two special-function ops per element (ex2 + rcp) would saturate the SFU
// before the memory system, so sigmoid(x) = 0.5 + 0.5 * tanh(0.5 x) with the one-instruction tanh.approx
// is used: its 2^-11 relative error is a few percent of a bf16 ulp and a quarter of an fp16 ulp.
template <typename T>
__device__ __forceinline__ float sigmoid_stream(float x) {
    if constexpr (sizeof(T) == 4) {
        return sigmoid_clamped(x);
    } else {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
        return fmaf(t, 0.5f, 0.5f);
    }
}
template <typename T>
__device__ __forceinline__ float swiglu_f(float g, float u) { return u * (g * sigmoid_stream<T>(g)); }
template <typename T>
__device__ __forceinline__ void swiglu_b(float g, float u, float dy, float &dg, float &du) {
    const float s = sigmoid_stream<T>(g);
    const float silu = g * s;
    dg = (dy * u) * fmaf(silu, 1.0f - s, s);
    du = dy * silu;
}

// vectors are indexed v in [0, rows * vpr); vpr = cols / VEC.  CONTIG: one row, no index division.
template <typename T, bool CONTIG>
__global__ void __launch_bounds__(kEwThreads)
    swiglu_fwd_vec_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *__restrict__ out, int64_t nvec,
                          int64_t vpr, int64_t in_stride, int64_t out_stride) {
    constexpr int VEC = Lanes<T>::N;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t v0 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * kEwUnroll) {
        int4 g[kEwUnroll], u[kEwUnroll];
        int64_t oo[kEwUnroll];
#pragma unroll
        for (int j = 0; j < kEwUnroll; ++j) {
            const int64_t v = v0 + j * stride;
            if (v < nvec) {
                int64_t io;
                if constexpr (CONTIG) {
                    io = v * VEC;
                    oo[j] = io;
                } else {
                    const int64_t r = v / vpr, c = (v - r * vpr) * VEC;
                    io = r * in_stride + c;
                    oo[j] = r * out_stride + c;
                }
                g[j] = __ldg(reinterpret_cast<const int4 *>(gate + io));
                u[j] = __ldg(reinterpret_cast<const int4 *>(up + io));
            }
        }
#pragma unroll
        for (int j = 0; j < kEwUnroll; ++j) {
            const int64_t v = v0 + j * stride;
            if (v < nvec) {
                float gf[VEC], uf[VEC], of[VEC];
                Lanes<T>::unpack(g[j], gf);
                Lanes<T>::unpack(u[j], uf);
#pragma unroll
                for (int i = 0; i < VEC; ++i) of[i] = swiglu_f<T>(gf[i], uf[i]);
                *reinterpret_cast<int4 *>(out + oo[j]) = Lanes<T>::pack(of);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads)
    swiglu_fwd_scalar_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *__restrict__ out, int64_t n,
                             int64_t cols, int64_t in_stride, int64_t out_stride) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t r = i / cols, c = i - r * cols;
        out[r * out_stride + c] = DT<T>::down(swiglu_f<T>(DT<T>::up(gate[r * in_stride + c]), DT<T>::up(up[r * in_stride + c])));
    }
}

template <typename T, bool CONTIG>
__global__ void __launch_bounds__(kEwThreads)
    swiglu_bwd_vec_kernel(const T *__restrict__ gate, const T *__restrict__ up, const T *__restrict__ dy,
                          T *__restrict__ dgate, T *__restrict__ dup, int64_t nvec, int64_t vpr, int64_t in_stride,
                          int64_t dy_stride, int64_t grad_stride) {
    constexpr int VEC = Lanes<T>::N;
    constexpr int U = 2;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t v0 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * U) {
        int4 g[U], u[U], d[U];
        int64_t oo[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int64_t v = v0 + j * stride;
            if (v < nvec) {
                int64_t io, dyo;
                if constexpr (CONTIG) {
                    io = dyo = oo[j] = v * VEC;
                } else {
                    const int64_t r = v / vpr, c = (v - r * vpr) * VEC;
                    io = r * in_stride + c;
                    dyo = r * dy_stride + c;
                    oo[j] = r * grad_stride + c;
                }
                g[j] = __ldg(reinterpret_cast<const int4 *>(gate + io));
                u[j] = __ldg(reinterpret_cast<const int4 *>(up + io));
                d[j] = __ldg(reinterpret_cast<const int4 *>(dy + dyo));
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int64_t v = v0 + j * stride;
            if (v < nvec) {
                float gf[VEC], uf[VEC], df[VEC], og[VEC], ou[VEC];
                Lanes<T>::unpack(g[j], gf);
                Lanes<T>::unpack(u[j], uf);
                Lanes<T>::unpack(d[j], df);
#pragma unroll
                for (int i = 0; i < VEC; ++i) swiglu_b<T>(gf[i], uf[i], df[i], og[i], ou[i]);
                *reinterpret_cast<int4 *>(dgate + oo[j]) = Lanes<T>::pack(og);
                *reinterpret_cast<int4 *>(dup + oo[j]) = Lanes<T>::pack(ou);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads)
    swiglu_bwd_scalar_kernel(const T *__restrict__ gate, const T *__restrict__ up, const T *__restrict__ dy,
                             T *__restrict__ dgate, T *__restrict__ dup, int64_t n, int64_t cols, int64_t in_stride,
                             int64_t dy_stride, int64_t grad_stride) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t r = i / cols, c = i - r * cols;
        float dg, du;
        swiglu_b<T>(DT<T>::up(gate[r * in_stride + c]), DT<T>::up(up[r * in_stride + c]), DT<T>::up(dy[r * dy_stride + c]),
                    dg, du);
        dgate[r * grad_stride + c] = DT<T>::down(dg);
        dup[r * grad_stride + c] = DT<T>::down(du);
    }
}

// dst[p, :] = src[row_map[p] / fan_out, :], zeros where row_map[p] < 0; p < padded_off[E].
// One warp per padded row: the row index is read once (a broadcast load) and the lanes stream the row in 16-byte
// vectors, four in flight each; no division per vector.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
    gather_rows_kernel(const T *__restrict__ src, T *__restrict__ dst, const int32_t *__restrict__ row_map,
                       const int32_t *__restrict__ padded_off, int E, int64_t cap, int fan_out, int64_t vpr) {
    constexpr int VEC = Vec16<T>::N;
    int64_t rows = padded_off[E];
    if (rows > cap) rows = cap;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t p = warp; p < rows; p += nwarps) {
        const int32_t s = row_map[p];
        int4 *d = reinterpret_cast<int4 *>(dst + p * (vpr * VEC));
        const int4 *sr = reinterpret_cast<const int4 *>(src + int64_t(s < 0 ? 0 : s / fan_out) * (vpr * VEC));
        for (int64_t c0 = lane; c0 < vpr; c0 += 32 * kEwUnroll) {
            int4 x[kEwUnroll];
#pragma unroll
            for (int j = 0; j < kEwUnroll; ++j) {
                const int64_t c = c0 + 32 * j;
                x[j] = make_int4(0, 0, 0, 0);
                if (s >= 0 && c < vpr) x[j] = __ldg(sr + c);
            }
#pragma unroll
            for (int j = 0; j < kEwUnroll; ++j) {
                const int64_t c = c0 + 32 * j;
                if (c < vpr) d[c] = x[j];
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads) cast_from_f32_kernel(const float *__restrict__ src, T *__restrict__ dst, int64_t n) {
    constexpr int VEC = Vec16<T>::N;  // output elements per 16-byte store
    const int64_t nvec = n / VEC;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (int64_t v = tid; v < nvec; v += stride) {
        Vec16<T> o;
        const float4 *s4 = reinterpret_cast<const float4 *>(src + v * VEC);
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
            const float4 f = __ldg(s4 + q);
            o.v[4 * q + 0] = DT<T>::down(f.x);
            o.v[4 * q + 1] = DT<T>::down(f.y);
            o.v[4 * q + 2] = DT<T>::down(f.z);
            o.v[4 * q + 3] = DT<T>::down(f.w);
        }
        stg16(dst + v * VEC, o);
    }
    for (int64_t i = nvec * VEC + tid; i < n; i += stride) dst[i] = DT<T>::down(src[i]);
}

static inline unsigned ew_grid(int64_t work_items, int per_thread) {
    int64_t blocks = ceil_div64(work_items, int64_t(kEwThreads) * per_thread);
    const int64_t cap = int64_t(num_sms()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return unsigned(blocks);
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static int swiglu_fwd_t(const T *gate, const T *up, T *out, int64_t rows, int64_t cols, int64_t in_stride,
                        int64_t out_stride, cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    if (rows > 1 && in_stride == cols && out_stride == cols) {  // contiguous: flatten
        cols *= rows;
        rows = 1;
        in_stride = out_stride = cols;
    }
    const bool ptr_ok = aligned16(gate) && aligned16(up) && aligned16(out);
    if (rows == 1) {
        const int64_t main = ptr_ok ? (cols / VEC) * VEC : 0;
        if (main > 0) {
            swiglu_fwd_vec_kernel<T, true><<<ew_grid(main / VEC, kEwUnroll), kEwThreads, 0, stream>>>(gate, up, out, main / VEC,
                                                                                           main / VEC, main, main);
            CK_LAUNCH_CHECK("swiglu_fwd_vec_kernel");
        }
        if (cols > main) {
            const int64_t rem = cols - main;
            swiglu_fwd_scalar_kernel<T><<<ew_grid(rem, 1), kEwThreads, 0, stream>>>(gate + main, up + main, out + main, rem,
                                                                               rem, rem, rem);
            CK_LAUNCH_CHECK("swiglu_fwd_scalar_kernel");
        }
        return CK_OK;
    }
    if (ptr_ok && cols % VEC == 0 && in_stride % VEC == 0 && out_stride % VEC == 0) {
        const int64_t vpr = cols / VEC;
        swiglu_fwd_vec_kernel<T, false><<<ew_grid(rows * vpr, kEwUnroll), kEwThreads, 0, stream>>>(gate, up, out, rows * vpr, vpr,
                                                                                       in_stride, out_stride);
        CK_LAUNCH_CHECK("swiglu_fwd_vec_kernel");
    } else {
        swiglu_fwd_scalar_kernel<T><<<ew_grid(rows * cols, 1), kEwThreads, 0, stream>>>(gate, up, out, rows * cols, cols,
                                                                                   in_stride, out_stride);
        CK_LAUNCH_CHECK("swiglu_fwd_scalar_kernel");
    }
    return CK_OK;
}

template <typename T>
static int swiglu_bwd_t(const T *gate, const T *up, const T *dy, T *dgate, T *dup, int64_t rows, int64_t cols,
                        int64_t in_stride, int64_t dy_stride, int64_t grad_stride, cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    if (rows > 1 && in_stride == cols && dy_stride == cols && grad_stride == cols) {
        cols *= rows;
        rows = 1;
        in_stride = dy_stride = grad_stride = cols;
    }
    const bool ptr_ok = aligned16(gate) && aligned16(up) && aligned16(dy) && aligned16(dgate) && aligned16(dup);
    if (rows == 1) {
        const int64_t main = ptr_ok ? (cols / VEC) * VEC : 0;
        if (main > 0) {
            swiglu_bwd_vec_kernel<T, true><<<ew_grid(main / VEC, 2), kEwThreads, 0, stream>>>(gate, up, dy, dgate, dup, main / VEC,
                                                                                   main / VEC, main, main, main);
            CK_LAUNCH_CHECK("swiglu_bwd_vec_kernel");
        }
        if (cols > main) {
            const int64_t rem = cols - main;
            swiglu_bwd_scalar_kernel<T><<<ew_grid(rem, 1), kEwThreads, 0, stream>>>(gate + main, up + main, dy + main,
                                                                               dgate + main, dup + main, rem, rem, rem,
                                                                               rem, rem);
            CK_LAUNCH_CHECK("swiglu_bwd_scalar_kernel");
        }
        return CK_OK;
    }
    if (ptr_ok && cols % VEC == 0 && in_stride % VEC == 0 && dy_stride % VEC == 0 && grad_stride % VEC == 0) {
        const int64_t vpr = cols / VEC;
        swiglu_bwd_vec_kernel<T, false><<<ew_grid(rows * vpr, 2), kEwThreads, 0, stream>>>(gate, up, dy, dgate, dup, rows * vpr, vpr,
                                                                               in_stride, dy_stride, grad_stride);
        CK_LAUNCH_CHECK("swiglu_bwd_vec_kernel");
    } else {
        swiglu_bwd_scalar_kernel<T><<<ew_grid(rows * cols, 1), kEwThreads, 0, stream>>>(
            gate, up, dy, dgate, dup, rows * cols, cols, in_stride, dy_stride, grad_stride);
        CK_LAUNCH_CHECK("swiglu_bwd_scalar_kernel");
    }
    return CK_OK;
}

}  // namespace ck

using namespace ck;

extern "C" int ck_swiglu_fwd(const void *gate, const void *up, void *out, int64_t rows, int64_t cols, int64_t in_stride,
                             int64_t out_stride, int dtype, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (rows < 0 || cols < 0 || in_stride < cols || out_stride < cols) return CK_ERR_SHAPE;
    if (rows == 0 || cols == 0) return CK_OK;
    if (!gate || !up || !out) return CK_ERR_SHAPE;
    switch (dtype) {
        case CK_F32: return swiglu_fwd_t<float>((const float *)gate, (const float *)up, (float *)out, rows, cols, in_stride, out_stride, stream);
        case CK_F16: return swiglu_fwd_t<__half>((const __half *)gate, (const __half *)up, (__half *)out, rows, cols, in_stride, out_stride, stream);
        case CK_BF16: return swiglu_fwd_t<__nv_bfloat16>((const __nv_bfloat16 *)gate, (const __nv_bfloat16 *)up, (__nv_bfloat16 *)out, rows, cols, in_stride, out_stride, stream);
        default: return CK_ERR_UNSUPPORTED;
    }
}

extern "C" int ck_swiglu_bwd(const void *gate, const void *up, const void *dy, void *dgate, void *dup, int64_t rows,
                             int64_t cols, int64_t in_stride, int64_t dy_stride, int64_t grad_stride, int dtype,
                             void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (rows < 0 || cols < 0 || in_stride < cols || dy_stride < cols || grad_stride < cols) return CK_ERR_SHAPE;
    if (rows == 0 || cols == 0) return CK_OK;
    if (!gate || !up || !dy || !dgate || !dup) return CK_ERR_SHAPE;
    switch (dtype) {
        case CK_F32: return swiglu_bwd_t<float>((const float *)gate, (const float *)up, (const float *)dy, (float *)dgate, (float *)dup, rows, cols, in_stride, dy_stride, grad_stride, stream);
        case CK_F16: return swiglu_bwd_t<__half>((const __half *)gate, (const __half *)up, (const __half *)dy, (__half *)dgate, (__half *)dup, rows, cols, in_stride, dy_stride, grad_stride, stream);
        case CK_BF16: return swiglu_bwd_t<__nv_bfloat16>((const __nv_bfloat16 *)gate, (const __nv_bfloat16 *)up, (const __nv_bfloat16 *)dy, (__nv_bfloat16 *)dgate, (__nv_bfloat16 *)dup, rows, cols, in_stride, dy_stride, grad_stride, stream);
        default: return CK_ERR_UNSUPPORTED;
    }
}

template <typename T>
static int gather_rows_t(const void *src, void *dst, const int32_t *row_map, const int32_t *padded_off, int E, int64_t cap,
                         int fan_out, int64_t cols, cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    if (cols % VEC != 0 || !aligned16(src) || !aligned16(dst)) return CK_ERR_SHAPE;
    const int64_t vpr = cols / VEC;
    gather_rows_kernel<T><<<ew_grid(cap * 32, 1), kEwThreads, 0, stream>>>((const T *)src, (T *)dst, row_map, padded_off, E,
                                                                           cap, fan_out, vpr);
    CK_LAUNCH_CHECK("gather_rows_kernel");
    return CK_OK;
}

extern "C" int ck_moe_gather_rows(const void *src, void *dst, const int32_t *row_map, const int32_t *padded_off, int E,
                                  int64_t cap, int fan_out, int64_t cols, int dtype, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!src || !dst || !row_map || !padded_off || E <= 0 || cap < 0 || fan_out <= 0 || cols <= 0) return CK_ERR_SHAPE;
    if (cap == 0) return CK_OK;
    switch (dtype) {
        case CK_F32: return gather_rows_t<float>(src, dst, row_map, padded_off, E, cap, fan_out, cols, stream);
        case CK_F16: return gather_rows_t<__half>(src, dst, row_map, padded_off, E, cap, fan_out, cols, stream);
        case CK_BF16: return gather_rows_t<__nv_bfloat16>(src, dst, row_map, padded_off, E, cap, fan_out, cols, stream);
        default: return CK_ERR_UNSUPPORTED;
    }
}

extern "C" int ck_cast_from_f32(const float *src, void *dst, int64_t n, int dtype, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n < 0) return CK_ERR_SHAPE;
    if (n == 0) return CK_OK;
    if (!src || !dst || !aligned16(src) || !aligned16(dst)) return CK_ERR_SHAPE;
    switch (dtype) {
        case CK_F32:
            CK_CUDA_TRY(cudaMemcpyAsync(dst, src, sizeof(float) * n, cudaMemcpyDeviceToDevice, stream));
            return CK_OK;
        case CK_F16:
            cast_from_f32_kernel<__half><<<ew_grid(n / 8 + 1, 1), kEwThreads, 0, stream>>>(src, (__half *)dst, n);
            break;
        case CK_BF16:
            cast_from_f32_kernel<__nv_bfloat16><<<ew_grid(n / 8 + 1, 1), kEwThreads, 0, stream>>>(src, (__nv_bfloat16 *)dst, n);
            break;
        default: return CK_ERR_UNSUPPORTED;
    }
    CK_LAUNCH_CHECK("cast_from_f32_kernel");
    return CK_OK;
}
