// RMSNorm and fused residual-add + RMSNorm, forward and backward: HBM-bound streaming kernels.
//
// Replaces the reference's rmsnorm_cute / fused_residual_add_rmsnorm_cute (kernels/rmsnorm/__init__.py:12-77,
// kernels/fused_residual_add_rmsnorm/__init__.py:15-132, Triton kernels underneath); the math is that of
// rmsnorm_torch / fused_residual_add_rmsnorm_torch (torch_implementation.py of both):
//
//   forward    a = x * multiplier + residual            (only with a residual; a = x otherwise)
//              r = rsqrt(mean(a^2) + eps)                (fp32)
//              y = a * r * weight                        (fp32 throughout, one rounding to the tensor dtype, as F.rms_norm)
//   backward   g = dy * weight
//              da = r * g - a * r^3 * mean(g * a) + d_added      (d_added: gradient arriving through the residual stream)
//              d_residual = da, dx = da * multiplier,  d_weight[j] = sum_rows dy[., j] * a[., j] * r
//
// One thread group per row keeps the row in registers between the reduction and the write, so every tensor crosses
// HBM exactly once: forward 2 (4 with a residual) and backward 3 (5) elements of traffic per element.  Rows of up to
// 1 KiB use a warp per row (shuffle reduction only), longer rows a 256-thread block per row; rows that do not fit the
// register budget, or whose pointers / width are not 16-byte aligned, take a block-per-row kernel that re-reads the row
// (an L2 hit) instead.  The weight gradient is accumulated per thread over the rows it visits (the reference's Triton kernel
// does the same per program, then tl.atomic_add); here every block stores its sums as one row of a caller-owned fp32
// buffer and a second small kernel adds the rows in a fixed order: no atomics, reproducible.
#include "ck_common.cuh"

namespace ck {

constexpr int kNormBlock = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// sum over the G threads that share a row (G = 32: the warp; G = kNormBlock: the block, through shared memory)
template <int G>
__device__ __forceinline__ float group_sum(float v, float *red) {
    v = warp_sum(v);
    if constexpr (G == 32) return v;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // red may still be read from the previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < G / 32 ? red[lane] : 0.0f;
    return warp_sum(t);
}

template <typename T>
__device__ __forceinline__ void load_vec(const T *p, float *v) {
    const Vec16<T> raw = *reinterpret_cast<const Vec16<T> *>(p);
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) v[i] = DT<T>::up(raw.v[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T *p, const float *v) {
    Vec16<T> raw;
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) raw.v[i] = DT<T>::down(v[i]);
    __stcs(reinterpret_cast<int4 *>(p), *reinterpret_cast<const int4 *>(&raw));  // written once, read by a later kernel
}
// value as the tensor dtype would hold it
template <typename T>
__device__ __forceinline__ float rounded(float v) { return DT<T>::up(DT<T>::down(v)); }

// ---- forward -------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void unpack_vec(const int4 &raw, float *v) {
    const Vec16<T> &r = reinterpret_cast<const Vec16<T> &>(raw);
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) v[i] = DT<T>::up(r.v[i]);
}
template <typename T>
__device__ __forceinline__ int4 pack_vec(const float *v) {
    Vec16<T> r;
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) r.v[i] = DT<T>::down(v[i]);
    return reinterpret_cast<const int4 &>(r);
}

// G threads per row, VPT 16-byte vectors per thread (vector j of a thread covers columns (j * G + t) * VEC ...).  Rows stay
// packed in registers; the next row of the group is already in flight while the current one is reduced and written.
template <typename T, int G, int VPT>
__global__ void __launch_bounds__(kNormBlock)
    rmsnorm_fwd_kernel(const T *__restrict__ x, const T *__restrict__ residual, const T *__restrict__ weight, T *__restrict__ out,
                       T *__restrict__ added, float *__restrict__ inv_rms, int64_t rows, int H, float eps, float multiplier) {
    constexpr int VEC = Vec16<T>::N;
    __shared__ float red[kNormBlock / 32];
    const int t = threadIdx.x % G;
    const int rows_per_block = kNormBlock / G;
    const int nvec = H / VEC;
    const int64_t stride = int64_t(gridDim.x) * rows_per_block;
    int4 wp[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = j * G + t;
        wp[j] = make_int4(0, 0, 0, 0);
        if (weight != nullptr && c < nvec) wp[j] = *reinterpret_cast<const int4 *>(weight + int64_t(c) * VEC);
    }
    const float inv_h = 1.0f / float(H);
    int4 xp[VPT], rp[VPT];
    auto fetch = [&](int64_t row) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = j * G + t;
            if (row < rows && c < nvec) {
                const int64_t off = row * int64_t(H) + int64_t(c) * VEC;
                xp[j] = __ldcs(reinterpret_cast<const int4 *>(x + off));
                if (residual != nullptr) rp[j] = __ldcs(reinterpret_cast<const int4 *>(residual + off));
            }
        }
    };
    int64_t row = int64_t(blockIdx.x) * rows_per_block + threadIdx.x / G;
    fetch(row);
    for (; row < rows; row += stride) {
        float a[VPT][VEC];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = j * G + t;
            if (c < nvec) {
                unpack_vec<T>(xp[j], a[j]);
                if (residual != nullptr) {
                    float r[VEC];
                    unpack_vec<T>(rp[j], r);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) a[j][i] = rounded<T>(__fadd_rn(rounded<T>(__fmul_rn(a[j][i], multiplier)), r[i]));
                    if (added != nullptr) store_vec<T>(added + row * int64_t(H) + int64_t(c) * VEC, a[j]);
                }
#pragma unroll
                for (int i = 0; i < VEC; ++i) ss = fmaf(a[j][i], a[j][i], ss);
            }
        }
        fetch(row + stride);  // the next row's loads fly during the reduction and the stores below
        ss = group_sum<G>(ss, red);
        const float r = rsqrtf(ss * inv_h + eps);
        if (inv_rms != nullptr && t == 0) inv_rms[row] = r;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = j * G + t;
            if (c < nvec) {
                float y[VEC], w[VEC];
                if (weight != nullptr) {
                    unpack_vec<T>(wp[j], w);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) y[i] = a[j][i] * r * w[i];
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) y[i] = a[j][i] * r;
                }
                store_vec<T>(out + row * int64_t(H) + int64_t(c) * VEC, y);
            }
        }
    }
}

// any width / alignment: one block per row, the row is read twice (the second read hits L2)
template <typename T>
__global__ void __launch_bounds__(kNormBlock)
    rmsnorm_fwd_generic_kernel(const T *__restrict__ x, const T *__restrict__ residual, const T *__restrict__ weight,
                               T *__restrict__ out, T *__restrict__ added, float *__restrict__ inv_rms, int64_t rows, int64_t H,
                               float eps, float multiplier) {
    __shared__ float red[kNormBlock / 32];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *xr = x + row * H;
        const T *rr = residual ? residual + row * H : nullptr;
        T *ar = (added && residual) ? added + row * H : nullptr;
        float ss = 0.0f;
        for (int64_t c = threadIdx.x; c < H; c += kNormBlock) {
            float a = DT<T>::up(xr[c]);
            if (rr) a = rounded<T>(__fadd_rn(rounded<T>(__fmul_rn(a, multiplier)), DT<T>::up(rr[c])));
            if (ar) ar[c] = DT<T>::down(a);
            ss = fmaf(a, a, ss);
        }
        ss = group_sum<kNormBlock>(ss, red);
        const float r = rsqrtf(ss / float(H) + eps);
        if (inv_rms && threadIdx.x == 0) inv_rms[row] = r;
        for (int64_t c = threadIdx.x; c < H; c += kNormBlock) {
            float a = DT<T>::up(xr[c]);
            if (rr) a = rounded<T>(__fadd_rn(rounded<T>(__fmul_rn(a, multiplier)), DT<T>::up(rr[c])));
            const float wv = weight ? DT<T>::up(weight[c]) : 1.0f;
            out[row * H + c] = DT<T>::down(a * r * wv);
        }
    }
}

// ---- backward ------------------------------------------------------------------------------------------
// The weight gradient leaves every block as one row of dw_part [gridDim.x, H] (plain stores); rmsnorm_dw_reduce_kernel adds
// the rows in a fixed order, so the result is reproducible and no atomics hit the same H addresses from every block.
// ADDED: a gradient arrives through the residual stream too (d_added); its rows are prefetched with the others, which takes
// the registers of a second resident block.
template <typename T, int G, int VPT, bool ADDED>
__global__ void __launch_bounds__(kNormBlock, (VPT <= 2 && !ADDED) ? 2 : 1)
    rmsnorm_bwd_kernel(const T *__restrict__ a_in, const T *__restrict__ weight, const T *__restrict__ dy, const T *__restrict__ d_added,
                       const float *__restrict__ inv_rms, T *__restrict__ dx, T *__restrict__ d_residual, float *__restrict__ dw_part,
                       int64_t rows, int H, float eps, float multiplier) {
    constexpr int VEC = Vec16<T>::N;
    __shared__ float red[kNormBlock / 32];
    const int t = threadIdx.x % G;
    const int rows_per_block = kNormBlock / G;
    const int nvec = H / VEC;
    const int64_t stride = int64_t(gridDim.x) * rows_per_block;
    int4 wp[VPT];
    float dw[VPT][VEC];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = j * G + t;
        wp[j] = make_int4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < VEC; ++i) dw[j][i] = 0.0f;
        if (weight != nullptr && c < nvec) wp[j] = *reinterpret_cast<const int4 *>(weight + int64_t(c) * VEC);
    }
    const float inv_h = 1.0f / float(H);
    // rows stay packed (16 bytes per register quad) and are unpacked where they are used; two rows beyond the current one
    // are in flight, which is what keeps enough bytes outstanding per SM at the occupancy the accumulators allow
    // rows in flight per thread group: the current one and two more.  Measured on [16384, 4096] bf16: two in flight with three
    // resident blocks (80 registers, spills) 132 us; keeping g * w unpacked across the reduction (spills at 128 registers)
    // 134 us; this form 102 us.  The kernel issues 58 % of its slots at a quarter of the warp slots: instruction bound.
    constexpr int kSlots = 3;
    int4 ap[kSlots][VPT], gp[kSlots][VPT], ep[kSlots][ADDED ? VPT : 1];
    auto fetch = [&](int slot, int64_t row) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = j * G + t;
            if (row < rows && c < nvec) {
                const int64_t off = row * int64_t(H) + int64_t(c) * VEC;
                ap[slot][j] = __ldcs(reinterpret_cast<const int4 *>(a_in + off));
                gp[slot][j] = __ldcs(reinterpret_cast<const int4 *>(dy + off));
                if constexpr (ADDED) ep[slot][j] = __ldcs(reinterpret_cast<const int4 *>(d_added + off));
            }
        }
    };
    auto process = [&](int slot, int64_t row) {
        float ss = 0.0f, dot = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = j * G + t;
            if (c < nvec) {
                float a[VEC], g[VEC], w[VEC];
                unpack_vec<T>(ap[slot][j], a);
                unpack_vec<T>(gp[slot][j], g);
                if (weight != nullptr) unpack_vec<T>(wp[j], w);
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    ss = fmaf(a[i], a[i], ss);
                    dot = fmaf(weight != nullptr ? g[i] * w[i] : g[i], a[i], dot);
                }
            }
        }
        float r;
        if (inv_rms != nullptr) {
            r = inv_rms[row];
        } else {
            ss = group_sum<G>(ss, red);
            r = rsqrtf(ss * inv_h + eps);
        }
        dot = group_sum<G>(dot, red);
        const float coef = dot * inv_h * r * r * r;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = j * G + t;
            if (c < nvec) {
                const int64_t off = row * int64_t(H) + int64_t(c) * VEC;
                float a[VEC], g[VEC], w[VEC], da[VEC];
                unpack_vec<T>(ap[slot][j], a);
                unpack_vec<T>(gp[slot][j], g);
                if (weight != nullptr) unpack_vec<T>(wp[j], w);
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    da[i] = r * (weight != nullptr ? g[i] * w[i] : g[i]) - coef * a[i];
                    dw[j][i] = fmaf(g[i], a[i] * r, dw[j][i]);
                }
                if constexpr (ADDED) {
                    float e[VEC];
                    unpack_vec<T>(ep[slot][j], e);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) da[i] += e[i];
                }
                if (d_residual != nullptr) store_vec<T>(d_residual + off, da);
#pragma unroll
                for (int i = 0; i < VEC; ++i) da[i] *= multiplier;
                store_vec<T>(dx + off, da);
            }
        }
    };
    int64_t row = int64_t(blockIdx.x) * rows_per_block + threadIdx.x / G;
    fetch(0, row);
    // the slot index must be a compile-time constant for the arrays to stay in registers: kSlots rows per trip
    if constexpr (kSlots == 3) {
        fetch(1, row + stride);
        while (row < rows) {
            fetch(2, row + 2 * stride);
            process(0, row);
            row += stride;
            if (row >= rows) break;
            fetch(0, row + 2 * stride);
            process(1, row);
            row += stride;
            if (row >= rows) break;
            fetch(1, row + 2 * stride);
            process(2, row);
            row += stride;
        }
    } else {
        while (row < rows) {
            fetch(1, row + stride);
            process(0, row);
            row += stride;
            if (row >= rows) break;
            fetch(0, row + stride);
            process(1, row);
            row += stride;
        }
    }
    if (dw_part != nullptr) {
        float *mine = dw_part + int64_t(blockIdx.x) * H;
        if constexpr (G == 32) {
            // the warps of a block hold different rows over the same columns: add them up in shared memory, warp by warp
            __shared__ float acc[VPT * 32 * VEC];
            for (int wq = 0; wq < kNormBlock / 32; ++wq) {
                if ((threadIdx.x >> 5) == wq) {
#pragma unroll
                    for (int j = 0; j < VPT; ++j)
#pragma unroll
                        for (int i = 0; i < VEC; ++i) {
                            const int idx = (j * 32 + t) * VEC + i;
                            acc[idx] = (wq == 0 ? 0.0f : acc[idx]) + dw[j][i];
                        }
                }
                __syncthreads();
            }
            for (int i = threadIdx.x; i < H; i += kNormBlock) mine[i] = acc[i];
        } else {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int c = j * G + t;
                if (c < nvec) {
                    *reinterpret_cast<float4 *>(mine + int64_t(c) * VEC) = make_float4(dw[j][0], dw[j][1], dw[j][2], dw[j][3]);
                    if constexpr (VEC == 8)
                        *reinterpret_cast<float4 *>(mine + int64_t(c) * VEC + 4) = make_float4(dw[j][4], dw[j][5], dw[j][6], dw[j][7]);
                }
            }
        }
    }
}

// d_weight[c] = sum over the parts of dw_part[i, c], written in the weight's dtype.  A block owns 8 columns (one 32-byte
// sector per part row); its 32 part lanes take the parts i = lane, lane + 32, ... with all of their loads in flight at once
// (the rows were just written: L2 hits, and a single chain per column would cost hundreds of L2 round trips), then the 32
// partial sums are added in lane order.  The order of every addition is fixed by the code: reproducible.
constexpr int kDwCols = 8;
template <typename T>
__global__ void __launch_bounds__(kNormBlock) rmsnorm_dw_reduce_kernel(const float *__restrict__ dw_part, int parts, int64_t H,
                                                                       T *__restrict__ d_weight) {
    constexpr int kLanes = kNormBlock / kDwCols;  // 32 part lanes
    constexpr int kUnroll = 16;                   // up to 16 x 32 = 512 parts per pass
    __shared__ float acc[kLanes][kDwCols + 1];
    const int col = threadIdx.x % kDwCols, lane = threadIdx.x / kDwCols;
    const int64_t c = int64_t(blockIdx.x) * kDwCols + col;
    float total = 0.0f;
    if (c < H) {
        for (int base = lane; base < parts; base += kUnroll * kLanes) {
            float v[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int q = base + u * kLanes;
                v[u] = q < parts ? dw_part[int64_t(q) * H + c] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) total += v[u];
        }
    }
    acc[lane][col] = total;
    __syncthreads();
    if (lane == 0 && c < H) {
        float sum = acc[0][col];
#pragma unroll
        for (int l = 1; l < kLanes; ++l) sum += acc[l][col];
        d_weight[c] = DT<T>::down(sum);
    }
}

template <typename T>
__global__ void __launch_bounds__(kNormBlock)
    rmsnorm_bwd_generic_kernel(const T *__restrict__ a_in, const T *__restrict__ weight, const T *__restrict__ dy,
                               const T *__restrict__ d_added, const float *__restrict__ inv_rms, T *__restrict__ dx,
                               T *__restrict__ d_residual, float *__restrict__ dw_part, int64_t rows, int64_t H, float eps,
                               float multiplier) {
    __shared__ float red[kNormBlock / 32];
    float *mine = dw_part ? dw_part + int64_t(blockIdx.x) * H : nullptr;  // zeroed by the host; each thread owns its columns
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *ar = a_in + row * H;
        const T *gr = dy + row * H;
        float ss = 0.0f, dot = 0.0f;
        for (int64_t c = threadIdx.x; c < H; c += kNormBlock) {
            const float a = DT<T>::up(ar[c]);
            const float wv = weight ? DT<T>::up(weight[c]) : 1.0f;
            ss = fmaf(a, a, ss);
            dot = fmaf(DT<T>::up(gr[c]) * wv, a, dot);
        }
        float r;
        if (inv_rms) {
            r = inv_rms[row];
        } else {
            ss = group_sum<kNormBlock>(ss, red);
            r = rsqrtf(ss / float(H) + eps);
        }
        dot = group_sum<kNormBlock>(dot, red);
        const float coef = dot / float(H) * r * r * r;
        for (int64_t c = threadIdx.x; c < H; c += kNormBlock) {
            const float a = DT<T>::up(ar[c]);
            const float g = DT<T>::up(gr[c]);
            const float wv = weight ? DT<T>::up(weight[c]) : 1.0f;
            float da = r * g * wv - coef * a;
            if (d_added) da += DT<T>::up(d_added[row * H + c]);
            if (d_residual) d_residual[row * H + c] = DT<T>::down(da);
            dx[row * H + c] = DT<T>::down(da * multiplier);
            if (mine) mine[c] += g * (a * r);
        }
    }
}

// ---- launch --------------------------------------------------------------------------------------------
static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static unsigned norm_grid(int64_t row_groups, int blocks_per_sm) {
    int64_t g = row_groups;
    const int64_t cap = int64_t(num_sms()) * blocks_per_sm;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return unsigned(g);
}

template <typename T, int G, int VPT>
static void launch_fwd(const void *x, const void *res, const void *w, void *out, void *added, float *inv, int64_t rows, int H,
                       float eps, float mult, cudaStream_t s) {
    const int rpb = kNormBlock / G;
    rmsnorm_fwd_kernel<T, G, VPT><<<norm_grid(ceil_div64(rows, rpb), 8), kNormBlock, 0, s>>>(
        (const T *)x, (const T *)res, (const T *)w, (T *)out, (T *)added, inv, rows, H, eps, mult);
}
// blocks of the backward launch = rows of the weight-gradient partial buffer: at most kBwdBlocksPerSm per SM
constexpr int kBwdBlocksPerSm = 4;
static unsigned bwd_grid(int64_t rows, int rows_per_block, int blocks_per_sm = kBwdBlocksPerSm) {
    return norm_grid(ceil_div64(rows, rows_per_block), blocks_per_sm);
}

// The grid is exactly what is resident at once (every block then walks the same number of rows: no second, ragged wave,
// and no more partial weight-gradient rows than needed); returns the number of blocks launched.
template <typename T, int G, int VPT, bool ADDED>
static unsigned launch_bwd_t(const void *a, const void *w, const void *dy, const void *dadd, const float *inv, void *dx, void *dres,
                           float *dw_part, int64_t rows, int H, float eps, float mult, cudaStream_t s) {
    static int resident = 0;  // blocks of this instantiation per SM
    if (resident == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, rmsnorm_bwd_kernel<T, G, VPT, ADDED>, kNormBlock, 0) != cudaSuccess || n < 1) n = 1;
        resident = n > kBwdBlocksPerSm ? kBwdBlocksPerSm : n;
    }
    const unsigned grid = bwd_grid(rows, kNormBlock / G, resident);
    rmsnorm_bwd_kernel<T, G, VPT, ADDED><<<grid, kNormBlock, 0, s>>>(
        (const T *)a, (const T *)w, (const T *)dy, (const T *)dadd, inv, (T *)dx, (T *)dres, dw_part, rows, H, eps, mult);
    return grid;
}
template <typename T, int G, int VPT>
static unsigned launch_bwd(const void *a, const void *w, const void *dy, const void *dadd, const float *inv, void *dx, void *dres,
                           float *dw_part, int64_t rows, int H, float eps, float mult, cudaStream_t s) {
    return dadd ? launch_bwd_t<T, G, VPT, true>(a, w, dy, dadd, inv, dx, dres, dw_part, rows, H, eps, mult, s)
                : launch_bwd_t<T, G, VPT, false>(a, w, dy, dadd, inv, dx, dres, dw_part, rows, H, eps, mult, s);
}

// picks (G, VPT) for a row of nvec 16-byte vectors; false: use the generic kernels
#define CK_NORM_DISPATCH(T, nvec, CALL_W, CALL_B)                      \
    if ((nvec) <= 32) { CALL_W(T, 32, 1); }                            \
    else if ((nvec) <= 64) { CALL_W(T, 32, 2); }                       \
    else if ((nvec) <= 128) { CALL_W(T, 32, 4); }                      \
    else if ((nvec) <= 256) { CALL_B(T, kNormBlock, 1); }              \
    else if ((nvec) <= 512) { CALL_B(T, kNormBlock, 2); }              \
    else if ((nvec) <= 1024) { CALL_B(T, kNormBlock, 4); }             \
    else { CALL_B(T, kNormBlock, 8); }

template <typename T>
static int rmsnorm_fwd_t(const void *x, const void *res, const void *w, void *out, void *added, float *inv, int64_t rows, int64_t H,
                         float eps, float mult, cudaStream_t s) {
    constexpr int VEC = Vec16<T>::N;
    const bool vec_ok = H % VEC == 0 && H / VEC <= 2048 && aligned16(x) && aligned16(out) && (!res || aligned16(res)) &&
                        (!w || aligned16(w)) && (!added || aligned16(added));
    if (vec_ok) {
        const int nvec = int(H / VEC);
#define FWD_CALL(TT, GG, VV) launch_fwd<TT, GG, VV>(x, res, w, out, added, inv, rows, int(H), eps, mult, s)
        CK_NORM_DISPATCH(T, nvec, FWD_CALL, FWD_CALL)
#undef FWD_CALL
    } else {
        rmsnorm_fwd_generic_kernel<T><<<norm_grid(rows, 8), kNormBlock, 0, s>>>((const T *)x, (const T *)res, (const T *)w, (T *)out,
                                                                                 (T *)added, inv, rows, H, eps, mult);
    }
    CK_LAUNCH_CHECK("rmsnorm_fwd_kernel");
    return CK_OK;
}

template <typename T>
static bool bwd_vectorised(const void *a, const void *w, const void *dy, const void *dadd, const void *dx, const void *dres, int64_t H) {
    constexpr int VEC = Vec16<T>::N;
    return H % VEC == 0 && H / VEC <= 1024 && aligned16(a) && aligned16(dy) && aligned16(dx) && (!w || aligned16(w)) &&
           (!dadd || aligned16(dadd)) && (!dres || aligned16(dres));
}
template <typename T>
static int rmsnorm_bwd_t(const void *a, const void *w, const void *dy, const void *dadd, const float *inv, void *dx, void *dres,
                         float *dw_part, void *dw, int64_t rows, int64_t H, float eps, float mult, cudaStream_t s) {
    constexpr int VEC = Vec16<T>::N;
    unsigned parts;
    if (bwd_vectorised<T>(a, w, dy, dadd, dx, dres, H)) {
        const int nvec = int(H / VEC);
        parts = 0;
#define BWD_CALL(TT, GG, VV) parts = launch_bwd<TT, GG, VV>(a, w, dy, dadd, inv, dx, dres, dw_part, rows, int(H), eps, mult, s)
        CK_NORM_DISPATCH(T, nvec, BWD_CALL, BWD_CALL)
#undef BWD_CALL
    } else {
        parts = bwd_grid(rows, 1);
        if (dw_part) CK_CUDA_TRY(cudaMemsetAsync(dw_part, 0, size_t(parts) * size_t(H) * sizeof(float), s));
        rmsnorm_bwd_generic_kernel<T><<<parts, kNormBlock, 0, s>>>((const T *)a, (const T *)w, (const T *)dy, (const T *)dadd, inv, (T *)dx,
                                                                    (T *)dres, dw_part, rows, H, eps, mult);
    }
    CK_LAUNCH_CHECK("rmsnorm_bwd_kernel");
    if (dw) {
        rmsnorm_dw_reduce_kernel<T><<<unsigned(ceil_div64(H, kDwCols)), kNormBlock, 0, s>>>(dw_part, int(parts), H, (T *)dw);
        CK_LAUNCH_CHECK("rmsnorm_dw_reduce_kernel");
    }
    return CK_OK;
}

}  // namespace ck

using namespace ck;

extern "C" int ck_rmsnorm_fwd(const void *x, const void *residual, const void *weight, void *out, void *added_out,
                              float *inv_rms_out, int64_t rows, int64_t H, float eps, float multiplier, int dtype,
                              void *stream) {
    if (rows < 0 || H <= 0 || H > INT32_MAX) return CK_ERR_SHAPE;
    if (rows == 0) return CK_OK;
    if (!x || !out) return CK_ERR_SHAPE;
    if (added_out && !residual) return CK_ERR_SHAPE;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
        case CK_F32: return rmsnorm_fwd_t<float>(x, residual, weight, out, added_out, inv_rms_out, rows, H, eps, multiplier, s);
        case CK_F16: return rmsnorm_fwd_t<__half>(x, residual, weight, out, added_out, inv_rms_out, rows, H, eps, multiplier, s);
        case CK_BF16: return rmsnorm_fwd_t<__nv_bfloat16>(x, residual, weight, out, added_out, inv_rms_out, rows, H, eps, multiplier, s);
        default: return CK_ERR_UNSUPPORTED;
    }
}

extern "C" int64_t ck_rmsnorm_bwd_parts(int64_t rows, int64_t H) {
    if (rows <= 0 || H <= 0) return 0;
    // the largest grid any of the backward kernels would use for this shape (a warp per row, or a block per row)
    const unsigned a = bwd_grid(rows, kNormBlock / 32), b = bwd_grid(rows, 1);
    return int64_t(a > b ? a : b);
}

extern "C" int ck_rmsnorm_bwd(const void *a, const void *weight, const void *dy, const void *d_added, const float *inv_rms,
                              void *dx, void *d_residual, float *dw_partial, void *d_weight, int64_t rows, int64_t H, float eps,
                              float multiplier, int dtype, void *stream) {
    if (rows < 0 || H <= 0 || H > INT32_MAX) return CK_ERR_SHAPE;
    if (d_weight && !dw_partial) return CK_ERR_SHAPE;
    cudaStream_t s = (cudaStream_t)stream;
    if (rows == 0) {
        if (d_weight) CK_CUDA_TRY(cudaMemsetAsync(d_weight, 0, size_t(H) * (dtype == CK_F32 ? 4 : 2), s));
        return CK_OK;
    }
    if (!a || !dy || !dx) return CK_ERR_SHAPE;
    float *part = d_weight ? dw_partial : nullptr;
    switch (dtype) {
        case CK_F32: return rmsnorm_bwd_t<float>(a, weight, dy, d_added, inv_rms, dx, d_residual, part, d_weight, rows, H, eps, multiplier, s);
        case CK_F16: return rmsnorm_bwd_t<__half>(a, weight, dy, d_added, inv_rms, dx, d_residual, part, d_weight, rows, H, eps, multiplier, s);
        case CK_BF16: return rmsnorm_bwd_t<__nv_bfloat16>(a, weight, dy, d_added, inv_rms, dx, d_residual, part, d_weight, rows, H, eps, multiplier, s);
        default: return CK_ERR_UNSUPPORTED;
    }
}
