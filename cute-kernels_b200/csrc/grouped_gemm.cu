// Grouped GEMMs of the MoE expert path on tcgen05 tensor cores.
//
// One persistent, warp-specialised kernel template covers the GEMMs of a forward + backward pass (and the router's gate
// projection).  Rows of every activation matrix live in the "padded grouped" layout produced by ck_route: the rows routed
// to expert e occupy [padded_off[e], padded_off[e+1]), a multiple of 128 rows, pad rows are zero.  A 128-row tile therefore
// belongs to exactly one expert and needs no row masks on the operand side.
//
// Two flavours of the same design (ck_set_gemm_cta_pair):
//   CTA pair (default)  clusters of two CTAs share a 256 x 256 tile: each owns 128 rows and loads half of the B tile, one
//                       tcgen05.mma.cta_group::2 issued by the leader reads both halves; 6-stage ring of 32 KiB per CTA
//   single CTA          128 x 256 tile, cta_group::1, 4 stages of 48 KiB
// Warp roles (one CTA per SM, fp32 accumulators in TMEM, 2 x 256 columns, double buffered):
//     TMA producer   global -> 128B-swizzled shared memory through an mbarrier ring
//     MMA issuer     tcgen05.mma, 32 bytes of K per instruction, commits free the stages / publish the accumulators
//     epilogue       one or two groups of four warps: tcgen05.ld of the finished accumulator + the fused tail (activation,
//                    activation backward, router-weight grad, scatter-add combine, router top-k, or a plain / scattered /
//                    peer-memory store)
// The producer and issuer loops are run by their whole warp, converged, with one elected lane issuing the predicated
// TMA / MMA / commit instructions, and each probes the next stage's barrier before it issues the current stage's work:
// a single thread's instruction stream between two k-blocks is otherwise what the tensor pipe waits for.
//
// Every mbarrier wait is bounded by wall-clock time; when one runs out the CTA raises CK_DEV_TIMEOUT in the caller's
// status word, lets in-flight copies land, frees TMEM and returns.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include "ck_common.cuh"
#include "sm100_ptx.cuh"

namespace ck {

enum { MODE_STORE = 0, MODE_UP_ACT = 1, MODE_SCATTER_ADD = 2, MODE_ACT_BWD = 3, MODE_WGRAD = 4,
       MODE_UP_ACT1 = 5, MODE_ACT1_BWD = 6,  // 5, 6: the un-gated up projection (one pre-activation per output) and its backward
       MODE_ROUTER = 7 };                    // gate projection with the router tail (top-k, softmax, int32 ids) in the epilogue

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int kStages = 4;
constexpr int kRowBytes = 128;                       // one swizzle row
constexpr int kAStageBytes = BM * kRowBytes;         // 16 KiB
constexpr int kBStageBytes = BN * kRowBytes;         // 32 KiB
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;                       // 2 accumulators x 256 fp32 columns
constexpr uint64_t kWaitLimitNs = 4000000000ull;     // 4 s per wait, far above any legitimate stall
constexpr int kMaxSchedExperts = CK_ROUTE_MAX_EXPERTS;

struct GemmParams {
    CUtensorMap tmA;
    CUtensorMap tmB;
    const int32_t *mtile_off;   // [E+1] (all modes but WGRAD); NULL: one group of m_tiles_w m-tiles (E must be 1)
    const int32_t *padded_off;  // [E+1] (WGRAD)
    const int32_t *row_map;     // [cap]
    const void *gate_w;         // router weights, flat [T*k], dtype T (may be NULL)
    const void *h_in;           // ACT_BWD: saved [cap, 2I] pre-activation
    void *out0;                 // STORE/WGRAD: y | UP_ACT: act | ACT_BWD: dh
    void *out1;                 // UP_ACT: h (may be NULL) | ROUTER: router weights [tokens, top_k]
    int32_t *ids_out;           // ROUTER: expert ids [tokens, top_k]
    // ROUTER: rows of the gate weight each TMA box of B holds (the boxes cover only rows that exist: a box that hangs over the
    // end of the tensor is filled row by row at a fraction of the normal rate).  CTA pair: the leader's box (rows 0 ..) and the
    // second CTA's (rows 128 .., tensor map tmOut; 0 = no load); single CTA: one box of b_rows_lead rows.
    int b_rows_lead;
    int b_rows_peer;
    float *out32;               // SCATTER_ADD target [T, N]
    const void *bias;           // per-expert bias of the GEMM's output features, [E, bias_ld] of T (may be NULL):
                                //   UP_ACT: [up | gate] packed, bias_ld = 2I; UP_ACT1: bias_ld = I; STORE / SCATTER_ADD: bias_ld = N,
                                //   scaled by the row's router weight when gate_w is given
    int bias_ld;
    float *dgates;              // ACT_BWD: [T*k] fp32, atomically accumulated (used when dgates_part is NULL)
    float *dgates_part;         // ACT_BWD: [n_parts, cap] fp32 per-(n-tile, epilogue group) partial sums, plain stores
    int32_t *dev_status;
    int E;
    int n_tiles;   // tiles along N
    int m_tiles_w; // WGRAD: tiles along M
    int N;         // valid output columns (UP_ACT / ACT_BWD: I)
    int K;         // contraction length in elements (not WGRAD)
    int M;         // WGRAD: output rows
    int top_k;
    int act_kind;
    int n_fastest; // WGRAD tile order
    int64_t cap;   // rows allocated for the padded layout
    int gather_fan;   // > 0: A rows are gathered by TMA from the un-permuted token matrix: token = row_map[p] / gather_fan
    int gather_b_fan; // WGRAD, > 0: the same for the B operand
    int l2_hint_a;    // ptx::L2_EVICT_* for the tiled loads of A / B (CTA-pair kernels)
    int l2_hint_b;
    uint64_t wait_limit_ns;  // bound of every mbarrier wait (0: kWaitLimitNs)
    // STORE with peer destinations (n_peers > 0): row row_map[p] of the result belongs to global slot
    // g = dst_flat ? dst_flat[row_map[p]] : row_map[p] and is
    // stored at peer_out[g / peer_rows] + (g % peer_rows) * N (another GPU's memory over NVLink, or this GPU's own buffer)
    const int32_t *dst_flat;
    int64_t peer_rows;
    int n_peers;
    void *peer_out[CK_MAX_PEERS];
    // A rows copied in by row index (CTA-pair kernels, UP_ACT / ACT_BWD, gather_fan > 0): padded row p comes from row
    // row_map[p] / gather_fan of a_src, or -- with n_src_peers > 0 -- from global slot g = row_map[p]: row
    // (g % src_peer_rows) / gather_fan of peer_src[g / src_peer_rows] (another GPU's memory over NVLink, or this GPU's own)
    const void *a_src;
    int64_t src_peer_rows;
    int n_src_peers;
    const void *peer_src[CK_MAX_PEERS];
    void *rows_out;       // not NULL: the gathered rows are also written out as the grouped [cap, K] matrix (tmOut)
    CUtensorMap tmOut;
};
constexpr int kPeerRowBits = 26;  // rowinfo = rank << 26 | row: up to 32 ranks of 2^26 rows

struct TileCoord {
    int e;       // expert
    int m_tile;  // global padded m-tile (not WGRAD) or m-tile of dW (WGRAD)
    int n_tile;
    int k_row0;  // WGRAD: first padded row of the expert
    int k_iters;
    bool valid;  // CTA-pair kernels: this CTA's half of the pair tile holds real rows
};

template <typename T>
struct GemmTraits {
    static constexpr int kElem = sizeof(T);
    static constexpr int BK = kRowBytes / kElem;       // elements of K per stage (64 or 32)
    static constexpr int UMMA_K = 32 / kElem;          // elements of K per instruction (16 or 8)
    static constexpr int kSteps = BK / UMMA_K;         // 4
    static constexpr bool kTf32 = (kElem == 4);
    static constexpr int kMnBoxElems = kRowBytes / kElem;  // MN elements per 128-byte swizzle row
    static constexpr int kMnBoxBytes = BK * kRowBytes;     // one {128 B of MN} x {BK rows of K} box
};

template <typename T>
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn, bool b_mn, int mma_m = BM) {
    const uint32_t fmt = (sizeof(T) == 4) ? 2u : (DT<T>::code == CK_BF16 ? 1u : 0u);
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           (uint32_t(BN >> 3) << 17) | (uint32_t(mma_m >> 4) << 24);
}

struct SmemCtl {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_ptr;
    volatile int abort_flag;
    uint64_t wait_limit_ns;
    int32_t sched[kMaxSchedExperts + 1];
};

constexpr size_t kGemmSmemBytes_noepi = 1024 /*alignment slack*/ + size_t(kStages) * (kAStageBytes + kBStageBytes) + sizeof(SmemCtl);

// bounded wait: false when the CTA is aborting or the time limit (ctl->wait_limit_ns) ran out
// BACKOFF: sleep between polls (epilogue warps: 32 polling lanes would otherwise compete for issue slots with the
// producer / MMA lanes that share their scheduler)
// CLUSTER: acquire at cluster scope (the barrier is also arrived at by ordinary lanes of the pair's other CTA)
template <bool BACKOFF = false, bool CLUSTER = false, typename Ctl>
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, Ctl *ctl, int32_t *dev_status) {
    auto passed = [&]() { return CLUSTER ? ptx::mbar_try_wait_cluster(bar, parity) : ptx::mbar_try_wait(bar, parity); };
    if (passed()) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (BACKOFF) __nanosleep(100);
        if (passed()) return true;
        if ((++spins & 63u) == 0) {
            if (ctl->abort_flag) return false;
            if (ptx::globaltimer_ns() - t0 > ctl->wait_limit_ns) {
                ctl->abort_flag = 1;
                if (dev_status) atomicOr(dev_status, CK_DEV_TIMEOUT);
                return false;
            }
        }
    }
}

template <int MODE>
__device__ __forceinline__ int total_tiles(const GemmParams &p, const SmemCtl *ctl) {
    if constexpr (MODE == MODE_WGRAD) return p.E * p.m_tiles_w * p.n_tiles;
    return (ctl->sched[p.E] - ctl->sched[0]) * p.n_tiles;  // mtile_off may start above 0: a window of the padded rows
}

template <int MODE, int BK>
__device__ __forceinline__ TileCoord decode_tile(const GemmParams &p, const SmemCtl *ctl, int t) {
    TileCoord c;
    c.valid = true;
    if constexpr (MODE == MODE_WGRAD) {
        const int per_e = p.m_tiles_w * p.n_tiles;
        c.e = t / per_e;
        const int local = t - c.e * per_e;
        if (p.n_fastest) {
            c.m_tile = local / p.n_tiles;
            c.n_tile = local - c.m_tile * p.n_tiles;
        } else {
            c.n_tile = local / p.m_tiles_w;
            c.m_tile = local - c.n_tile * p.m_tiles_w;
        }
        c.k_row0 = ctl->sched[c.e];
        c.k_iters = (ctl->sched[c.e + 1] - c.k_row0) / BK;
    } else {
        // experts in order; inside an expert n-major with the m-tiles fastest, so that concurrently
        // running CTAs share one weight panel and the expert's activation rows stay L2 resident
        t += ctl->sched[0] * p.n_tiles;
        int lo = 0, hi = p.E;  // find e with sched[e]*n_tiles <= t < sched[e+1]*n_tiles
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (ctl->sched[mid] * p.n_tiles <= t) lo = mid; else hi = mid;
        }
        c.e = lo;
        const int m0 = ctl->sched[lo];
        const int mt = ctl->sched[lo + 1] - m0;
        const int local = t - m0 * p.n_tiles;
        c.n_tile = local / mt;
        c.m_tile = m0 + (local - c.n_tile * mt);
        c.k_row0 = 0;
        c.k_iters = (p.K + BK - 1) / BK;
    }
    return c;
}

// ---- epilogue helpers ----------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void store8(T *ptr, const float *v) {
    if constexpr (sizeof(T) == 4) {
        reinterpret_cast<float4 *>(ptr)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4 *>(ptr)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        Vec16<T> o;
#pragma unroll
        for (int i = 0; i < 8; ++i) o.v[i] = DT<T>::down(v[i]);
        *reinterpret_cast<int4 *>(ptr) = *reinterpret_cast<const int4 *>(&o);
    }
}
template <typename T>
__device__ __forceinline__ void load8(const T *ptr, float *v) {
    if constexpr (sizeof(T) == 4) {
        const float4 a = reinterpret_cast<const float4 *>(ptr)[0];
        const float4 b = reinterpret_cast<const float4 *>(ptr)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        Vec16<T> o;
        *reinterpret_cast<int4 *>(&o) = *reinterpret_cast<const int4 *>(ptr);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = DT<T>::up(o.v[i]);
    }
}

// sigmoid in the epilogues: 16-bit tensors take sigmoid(x) = 0.5 + 0.5 tanh(0.5 x) with the single-instruction
// tanh.approx (relative error 2^-11, a few percent of a bf16 ulp); fp32 tensors keep the exp / divide form.
template <typename T>
__device__ __forceinline__ float sigmoid_epi(float x) {
    if constexpr (sizeof(T) == 4) {
        return sigmoid_fast(x);
    } else {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
        return fmaf(t, 0.5f, 0.5f);
    }
}
template <typename T>
__device__ __forceinline__ float act_fwd(int kind, float u, float g) {
    const float s = sigmoid_epi<T>(g);
    return kind == CK_ACT_SWIGLU ? u * g * s : u * s;
}
// returns a = act(u, g); d(out)/du and d(out)/dg multipliers
template <typename T>
__device__ __forceinline__ void act_bwd(int kind, float u, float g, float &a, float &du_m, float &dg_m) {
    const float s = sigmoid_epi<T>(g);
    if (kind == CK_ACT_SWIGLU) {
        const float silu = g * s;
        a = u * silu;
        du_m = silu;
        dg_m = u * (s + silu * (1.0f - s));
    } else {
        a = u * s;
        du_m = s;
        dg_m = u * s * (1.0f - s);
    }
}

// tanh-approximated GELU (torch.nn.GELU(approximate="tanh")): value and derivative
template <typename T>
__device__ __forceinline__ float tanh_epi(float x) {
    if constexpr (sizeof(T) == 4) {
        return tanhf(x);
    } else {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
        return t;
    }
}
template <typename T>
__device__ __forceinline__ float gelu_fwd(float x) {
    const float u = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
    return 0.5f * x * (1.0f + tanh_epi<T>(u));
}
template <typename T>
__device__ __forceinline__ void gelu_bwd(float x, float &a, float &da) {
    const float x2 = x * x;
    const float t = tanh_epi<T>(0.7978845608028654f * fmaf(0.044715f * x2, x, x));
    a = 0.5f * x * (1.0f + t);
    da = 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * 0.7978845608028654f * fmaf(3.0f * 0.044715f, x2, 1.0f);
}

// 32 consecutive bias values of the tile's expert (the same for every row of the tile), zeros where absent or out of range
template <typename T>
__device__ __forceinline__ void load_bias32(const GemmParams &p, int e, int col0, int ncols, float *b) {
#pragma unroll
    for (int i = 0; i < 32; ++i) b[i] = 0.0f;
    if (p.bias == nullptr) return;
    const T *src = reinterpret_cast<const T *>(p.bias) + int64_t(e) * p.bias_ld;
    if (col0 + 32 <= ncols) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) load8<T>(src + col0 + i, b + i);  // bias_ld and col0 are multiples of 8: 16-byte loads
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i < ncols) b[i] = DT<T>::up(src[col0 + i]);
    }
}

// ---- fused tail of one 128 x 256 tile: executed by the four epilogue warps of a CTA --------------------
//
// tcgen05.ld hands every thread one accumulator ROW.  Writing rows straight from registers makes each
// warp-wide global access touch 32 different rows (32 LSU wavefronts of 16 bytes): on tiles with a short
// K loop the load/store unit, not the tensor pipe, then sets the pace.  The tail therefore computes in the
// row-per-thread domain and moves data between registers and global memory through a small per-warp
// shared-memory stage, so that every global access is a run of 64 or 128 contiguous bytes of one row.
constexpr int kStagePitchWords = 36;                           // 32 payload words + 4 pad: conflict-free v4 / v2 access
constexpr int kStagePitchWords16 = 20;                         // 16 payload words (32 x 16-bit) + 4 pad: the same properties
constexpr int kStageWarpBytes = 32 * kStagePitchWords * 4;     // 4608 B per epilogue warp
constexpr int kEpiWarps = 4;
constexpr int kEpiSmemBytes = kEpiWarps * (kStageWarpBytes + 32 * 4);  // stages + per-row info

struct EpiSmem {
    uint32_t *stage;  // [32][PITCH] words, private to the warp
    int32_t *rowinfo; // [32] per-row index (row_map entry), private to the warp
};

// thread `lane` (owner of tile row `lane` of this warp) writes / reads its WORDS consecutive words
template <int WORDS, int PITCH>
__device__ __forceinline__ void stage_put_row(uint32_t *stage, int lane, const uint32_t *w) {
    uint4 *dst = reinterpret_cast<uint4 *>(stage + lane * PITCH);
#pragma unroll
    for (int q = 0; q < WORDS / 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
}
template <int WORDS, int PITCH>
__device__ __forceinline__ void stage_get_row(const uint32_t *stage, int lane, uint32_t *w) {
    const uint4 *src = reinterpret_cast<const uint4 *>(stage + lane * PITCH);
#pragma unroll
    for (int q = 0; q < WORDS / 4; ++q) {
        const uint4 v = src[q];
        w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
    }
}

// 32 fp32 values -> WORDS words of T (16 words for 16-bit types, 32 for fp32)
template <typename T>
__device__ __forceinline__ void pack32(const float *v, uint32_t *w) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(v[i]);
    } else if constexpr (DT<T>::code == CK_BF16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
    }
}
template <typename T>
__device__ __forceinline__ void unpack32(const uint32_t *w, float *v) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(w[i]);
    } else if constexpr (DT<T>::code == CK_BF16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
}

// Geometry of one staged pass over 32 rows x 32 elements of T: each lane moves 8 bytes, LPR lanes cover a row.
template <typename T>
struct RowPass {
    static constexpr int kWords = 32 * int(sizeof(T)) / 4;   // words per row: 16 or 32
    static constexpr int kLpr = kWords / 2;                  // lanes per row: 8 or 16
    static constexpr int kRpi = 32 / kLpr;                   // rows per instruction: 4 or 2
    static constexpr int kIters = 32 / kRpi;                 // 8 or 16
    static constexpr int kElemsPerLane = 8 / int(sizeof(T)); // 4 or 2
    // Row handled by `lane` in iteration `it`.  For 16-bit types four rows share an instruction; pairing rows
    // r and r+4 inside each half-warp puts their 16-word runs 16 banks apart (pitch 36 words), so the 8-byte
    // shared-memory accesses stay conflict free.
    __device__ __forceinline__ static int row(int it, int lane) {
        if constexpr (kLpr == 16) return it * 2 + (lane >> 4);
        else return 8 * (it >> 1) + 2 * (it & 1) + ((lane >> 3) & 1) * 4 + (lane >> 4);
    }
};

// rows of the stage -> global: row r goes to base(r) + col0 .. col0+31 (elements of T); base(r) == nullptr skips
template <typename T, int PITCH, typename RowPtr>
__device__ __forceinline__ void stage_write_rows(const uint32_t *stage, int lane, int col0, int ncols, RowPtr row_ptr) {
    using RP = RowPass<T>;
    const int sub = lane % RP::kLpr;
    const int col = col0 + sub * RP::kElemsPerLane;
#pragma unroll
    for (int it = 0; it < RP::kIters; ++it) {
        const int r = RP::row(it, lane);
        const uint2 v = *reinterpret_cast<const uint2 *>(stage + r * PITCH + 2 * sub);
        T *dst = row_ptr(r);
        if (dst != nullptr && col < ncols) __stcs(reinterpret_cast<uint2 *>(dst + col), v);  // written once: evict-first, keeps the operand panels in L2
    }
}
// global -> rows of the stage (zeros where the row is absent or the columns are out of range)
template <typename T, int PITCH, typename RowPtr>
__device__ __forceinline__ void stage_read_rows(uint32_t *stage, int lane, int col0, int ncols, RowPtr row_ptr) {
    using RP = RowPass<T>;
    const int sub = lane % RP::kLpr;
    const int col = col0 + sub * RP::kElemsPerLane;
#pragma unroll
    for (int it = 0; it < RP::kIters; ++it) {
        const int r = RP::row(it, lane);
        const T *src = row_ptr(r);
        uint2 v = make_uint2(0u, 0u);
        if (src != nullptr && col < ncols) v = *reinterpret_cast<const uint2 *>(src + col);
        *reinterpret_cast<uint2 *>(stage + r * PITCH + 2 * sub) = v;
    }
}

// the same transfer split in two, so the global loads of the next chunk fly while the current one is processed
template <typename T, typename RowPtr>
__device__ __forceinline__ void rows_prefetch(uint2 *regs, int lane, int col0, int ncols, RowPtr row_ptr) {
    using RP = RowPass<T>;
    const int col = col0 + (lane % RP::kLpr) * RP::kElemsPerLane;
#pragma unroll
    for (int it = 0; it < RP::kIters; ++it) {
        const T *src = row_ptr(RP::row(it, lane));
        regs[it] = make_uint2(0u, 0u);
        if (src != nullptr && col < ncols) regs[it] = __ldcs(reinterpret_cast<const uint2 *>(src + col));  // read once: evict-first
    }
}
template <typename T, int PITCH>
__device__ __forceinline__ void rows_to_stage(uint32_t *stage, int lane, const uint2 *regs) {
    using RP = RowPass<T>;
    const int sub = lane % RP::kLpr;
#pragma unroll
    for (int it = 0; it < RP::kIters; ++it)
        *reinterpret_cast<uint2 *>(stage + RP::row(it, lane) * PITCH + 2 * sub) = regs[it];
}

// element pair (i, i + 1) of a row chunk held as packed words of T
template <typename T>
__device__ __forceinline__ void get2(const uint32_t *w, int i, float &a, float &b) {
    if constexpr (sizeof(T) == 4) {
        a = __uint_as_float(w[i]);
        b = __uint_as_float(w[i + 1]);
    } else if constexpr (DT<T>::code == CK_BF16) {
        a = __uint_as_float(w[i >> 1] << 16);
        b = __uint_as_float(w[i >> 1] & 0xffff0000u);
    } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i >> 1]));
        a = f.x;
        b = f.y;
    }
}
template <typename T>
__device__ __forceinline__ void put2(uint32_t *w, int i, float a, float b) {
    if constexpr (sizeof(T) == 4) {
        w[i] = __float_as_uint(a);
        w[i + 1] = __float_as_uint(b);
    } else if constexpr (DT<T>::code == CK_BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        w[i >> 1] = *reinterpret_cast<const uint32_t *>(&h);
    } else {
        const __half2 h = __floats2half2_rn(a, b);
        w[i >> 1] = *reinterpret_cast<const uint32_t *>(&h);
    }
}

// Fused tail of one 128-row tile for the columns [cc_begin, cc_end) of its accumulator (steps of 32).  With two
// epilogue warp groups each group takes half of the columns; `part` numbers the (n-tile, group) pair for per-part
// outputs.  PITCH = words per row of the warp's shared-memory stage.
template <typename T, int MODE, int PITCH>
__device__ __forceinline__ void epilogue_tile(const GemmParams &p, const TileCoord &c, uint32_t tbase, int row_in_tile,
                                              const EpiSmem &es, int cc_begin, int cc_end, int part) {
    const bool have_acc = c.k_iters > 0;
    const int lane = row_in_tile & 31;
    const int row0 = row_in_tile - lane;  // first tile row of this warp
    using RP = RowPass<T>;
    static_assert(PITCH >= RP::kWords + 4 || MODE == MODE_SCATTER_ADD || MODE == MODE_ROUTER, "stage rows too narrow for this dtype");

    if constexpr (MODE == MODE_STORE || MODE == MODE_WGRAD) {
        // per-row destination: grouped row, scattered row (row_map) or a row of dW[e]
        T *my_out = nullptr;
        if constexpr (MODE == MODE_WGRAD) {
            const int m = c.m_tile * BM + row_in_tile;
            if (m < p.M) my_out = reinterpret_cast<T *>(p.out0) + (int64_t(c.e) * p.M + m) * int64_t(p.N);
        } else {
            int64_t orow = int64_t(c.m_tile) * BM + row_in_tile;
            bool row_ok = true;
            if (p.row_map) {  // scatter store: padded row -> caller's row order (each row written once)
                const int32_t src = p.row_map[orow];
                row_ok = src >= 0;
                orow = src;
            }
            if (row_ok) my_out = reinterpret_cast<T *>(p.out0) + orow * int64_t(p.N);
        }
        // publish the 32 row pointers of this warp as (valid, row index) pairs through rowinfo
        int64_t my_off = my_out ? (my_out - reinterpret_cast<T *>(p.out0)) / int64_t(p.N) : -1;
        const bool to_peers = MODE == MODE_STORE && p.n_peers > 0;
        if (to_peers && my_off >= 0) {
            const int64_t g = p.dst_flat ? int64_t(p.dst_flat[my_off]) : my_off;  // no table: row_map already holds the slot
            const int64_t rk = g / p.peer_rows;
            if (g >= 0 && rk < p.n_peers) {
                my_off = (rk << kPeerRowBits) | (g - rk * p.peer_rows);
            } else {
                my_off = -1;
                if (p.dev_status) atomicOr(p.dev_status, CK_DEV_RANGE);
            }
        }
        es.rowinfo[lane] = int32_t(my_off);  // row index in units of N elements: < 2^31 rows
        __syncwarp();
        auto row_ptr = [&](int r) -> T * {
            const int32_t o = es.rowinfo[r];
            if (o < 0) return nullptr;
            if (to_peers)
                return reinterpret_cast<T *>(p.peer_out[o >> kPeerRowBits]) + int64_t(o & ((1 << kPeerRowBits) - 1)) * int64_t(p.N);
            return reinterpret_cast<T *>(p.out0) + int64_t(o) * int64_t(p.N);
        };
        const int n0 = c.n_tile * BN;
        float bias_w = 1.0f;  // STORE with a bias: the row's router weight (the rows were scaled by it upstream)
        if constexpr (MODE == MODE_STORE) {
            if (p.bias != nullptr && p.gate_w != nullptr) {
                const int32_t src = p.row_map ? p.row_map[int64_t(c.m_tile) * BM + row_in_tile] : -1;
                bias_w = src >= 0 ? DT<T>::up(reinterpret_cast<const T *>(p.gate_w)[src]) : 0.0f;
            }
        }
#pragma unroll 1
        for (int cc = cc_begin; cc < cc_end; cc += 32) {
            uint32_t r[32];
            if (have_acc) {
                ptx::tmem_ld32(tbase + cc, r);
                ptx::tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            if constexpr (MODE == MODE_STORE) {
                if (p.bias != nullptr) {  // y = x W^T + b[e], scaled like the rows themselves when they carry a router weight
                    float bv[32];
                    load_bias32<T>(p, c.e, n0 + cc, p.N, bv);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = fmaf(bias_w, bv[i], v[i]);
                }
            }
            uint32_t w[RP::kWords];
            pack32<T>(v, w);
            stage_put_row<RP::kWords, PITCH>(es.stage, lane, w);
            __syncwarp();
            stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, row_ptr);
            __syncwarp();
        }
    } else if constexpr (MODE == MODE_UP_ACT) {
        const int64_t prow0 = int64_t(c.m_tile) * BM + row0;
        const int32_t src = p.row_map[prow0 + lane];
        float wgt = 1.0f;
        if (p.gate_w) wgt = (src >= 0) ? DT<T>::up(reinterpret_cast<const T *>(p.gate_w)[src]) : 0.0f;
        T *act = reinterpret_cast<T *>(p.out0) + prow0 * int64_t(p.N);
        T *h = p.out1 ? reinterpret_cast<T *>(p.out1) + prow0 * int64_t(2 * p.N) : nullptr;
        const int64_t ld_act = p.N, ld_h = 2 * int64_t(p.N);
        const int n0 = c.n_tile * (BN / 2);
#pragma unroll 1
        for (int cc = cc_begin; cc < cc_end; cc += 32) {
            if (n0 + cc >= p.N) break;  // whole chunk past the valid columns (uniform across the warp)
            uint32_t ru[32], rg[32];
            ptx::tmem_ld32(tbase + cc, ru);
            ptx::tmem_ld32(tbase + BN / 2 + cc, rg);
            ptx::tmem_ld_wait();
            if (p.bias != nullptr) {  // pre-activations include the expert's bias: [up | gate] packed like the weight
                float bv[32];
                load_bias32<T>(p, c.e, n0 + cc, p.N, bv);
#pragma unroll
                for (int i = 0; i < 32; ++i) ru[i] = __float_as_uint(__uint_as_float(ru[i]) + bv[i]);
                load_bias32<T>(p, c.e, p.N + n0 + cc, 2 * p.N, bv);
#pragma unroll
                for (int i = 0; i < 32; ++i) rg[i] = __float_as_uint(__uint_as_float(rg[i]) + bv[i]);
            }
            uint32_t w[RP::kWords];
#pragma unroll
            for (int i = 0; i < 32; i += 2)
                put2<T>(w, i, wgt * act_fwd<T>(p.act_kind, __uint_as_float(ru[i]), __uint_as_float(rg[i])),
                        wgt * act_fwd<T>(p.act_kind, __uint_as_float(ru[i + 1]), __uint_as_float(rg[i + 1])));
            stage_put_row<RP::kWords, PITCH>(es.stage, lane, w);
            __syncwarp();
            stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return act + r * ld_act; });
            __syncwarp();
            if (h) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) put2<T>(w, i, __uint_as_float(ru[i]), __uint_as_float(ru[i + 1]));
                stage_put_row<RP::kWords, PITCH>(es.stage, lane, w);
                __syncwarp();
                stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return h + r * ld_h; });
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 32; i += 2) put2<T>(w, i, __uint_as_float(rg[i]), __uint_as_float(rg[i + 1]));
                stage_put_row<RP::kWords, PITCH>(es.stage, lane, w);
                __syncwarp();
                stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return h + r * ld_h + p.N; });
                __syncwarp();
            }
        }
    } else if constexpr (MODE == MODE_SCATTER_ADD) {
        const int64_t prow = int64_t(c.m_tile) * BM + row_in_tile;
        const int32_t src = p.row_map[prow];
        es.rowinfo[lane] = src >= 0 ? src / p.top_k : -1;  // destination token row
        __syncwarp();
        const int n0 = c.n_tile * BN;
        const int sub = lane & 7;  // 8 lanes x 16 bytes cover the 32 fp32 columns of one row
        float bias_w = 0.0f;  // with a bias: this row's router weight (the activations were scaled by it upstream)
        if (p.bias != nullptr && src >= 0) bias_w = p.gate_w ? DT<T>::up(reinterpret_cast<const T *>(p.gate_w)[src]) : 1.0f;
#pragma unroll 1
        for (int cc = cc_begin; cc < cc_end; cc += 32) {
            uint32_t r[32];
            ptx::tmem_ld32(tbase + cc, r);
            ptx::tmem_ld_wait();
            if (p.bias != nullptr) {
                float bv[32];
                load_bias32<T>(p, c.e, n0 + cc, p.N, bv);
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(fmaf(bias_w, bv[i], __uint_as_float(r[i])));
            }
            stage_put_row<32, PITCH>(es.stage, lane, r);
            __syncwarp();
            const int col = n0 + cc + 4 * sub;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int rr = it * 4 + (lane >> 3);
                const int32_t tok = es.rowinfo[rr];
                const float4 v = *reinterpret_cast<const float4 *>(es.stage + rr * PITCH + 4 * sub);
                if (tok >= 0 && col < p.N) ptx::red_add_v4(p.out32 + int64_t(tok) * int64_t(p.N) + col, v.x, v.y, v.z, v.w);
            }
            __syncwarp();
        }
    } else if constexpr (MODE == MODE_ACT_BWD) {
        const int64_t prow0 = int64_t(c.m_tile) * BM + row0;
        const int32_t src = p.row_map[prow0 + lane];
        float wgt = (src >= 0) ? 1.0f : 0.0f;
        if (p.gate_w && src >= 0) wgt = DT<T>::up(reinterpret_cast<const T *>(p.gate_w)[src]);
        const int64_t ld_h = 2 * int64_t(p.N);
        const T *h = reinterpret_cast<const T *>(p.h_in) + prow0 * ld_h;
        T *dh = reinterpret_cast<T *>(p.out0) + prow0 * ld_h;
        const int n0 = c.n_tile * BN;
        float dgate_w = 0.0f;
        uint2 pu[RP::kIters], pg[RP::kIters];  // saved up / gate values of the next chunk, in flight
        auto h_up = [&](int r) -> const T * { return h + r * ld_h; };
        auto h_gate = [&](int r) -> const T * { return h + r * ld_h + p.N; };
        if (n0 + cc_begin < p.N) {
            rows_prefetch<T>(pu, lane, n0 + cc_begin, p.N, h_up);
            rows_prefetch<T>(pg, lane, n0 + cc_begin, p.N, h_gate);
        }
#pragma unroll 1
        for (int cc = cc_begin; cc < cc_end; cc += 32) {
            if (n0 + cc >= p.N) break;  // whole chunk past the valid columns (uniform across the warp)
            uint32_t wu[RP::kWords], wg[RP::kWords];  // this row's 32 up / gate values, packed; overwritten by the results
            rows_to_stage<T, PITCH>(es.stage, lane, pu);
            __syncwarp();
            stage_get_row<RP::kWords, PITCH>(es.stage, lane, wu);
            __syncwarp();
            rows_to_stage<T, PITCH>(es.stage, lane, pg);
            __syncwarp();
            stage_get_row<RP::kWords, PITCH>(es.stage, lane, wg);
            __syncwarp();
            if (cc + 32 < cc_end && n0 + cc + 32 < p.N) {
                rows_prefetch<T>(pu, lane, n0 + cc + 32, p.N, h_up);
                rows_prefetch<T>(pg, lane, n0 + cc + 32, p.N, h_gate);
            }
            uint32_t r[32];
            ptx::tmem_ld32(tbase + cc, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float u0, u1, g0, g1;
                get2<T>(wu, i, u0, u1);
                get2<T>(wg, i, g0, g1);
                float a0, du0, dg0, a1, du1, dg1;
                act_bwd<T>(p.act_kind, u0, g0, a0, du0, dg0);
                act_bwd<T>(p.act_kind, u1, g1, a1, du1, dg1);
                const float acc0 = __uint_as_float(r[i]), acc1 = __uint_as_float(r[i + 1]);
                dgate_w = fmaf(a0, acc0, dgate_w);
                dgate_w = fmaf(a1, acc1, dgate_w);
                const float da0 = wgt * acc0, da1 = wgt * acc1;
                put2<T>(wu, i, da0 * du0, da1 * du1);
                put2<T>(wg, i, da0 * dg0, da1 * dg1);
            }
            stage_put_row<RP::kWords, PITCH>(es.stage, lane, wu);
            __syncwarp();
            stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return dh + r * ld_h; });
            __syncwarp();
            stage_put_row<RP::kWords, PITCH>(es.stage, lane, wg);
            __syncwarp();
            stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return dh + r * ld_h + p.N; });
            __syncwarp();
        }
        // router-weight grad of this row over this part's columns: a plain store into the part's slice when the caller
        // gave a partial buffer (summed later in a fixed order: reproducible), else an atomic add into dgates
        if (p.dgates_part) p.dgates_part[int64_t(part) * p.cap + prow0 + lane] = dgate_w;
        else if (p.dgates && src >= 0) atomicAdd(p.dgates + src, dgate_w);
    } else if constexpr (MODE == MODE_UP_ACT1) {
        // un-gated up projection: pre = x W^T + b, act = w * gelu_tanh(pre); pre is saved for the backward pass
        const int64_t prow0 = int64_t(c.m_tile) * BM + row0;
        const int32_t src = p.row_map[prow0 + lane];
        float wgt = 1.0f;
        if (p.gate_w) wgt = (src >= 0) ? DT<T>::up(reinterpret_cast<const T *>(p.gate_w)[src]) : 0.0f;
        T *act = reinterpret_cast<T *>(p.out0) + prow0 * int64_t(p.N);
        T *h = p.out1 ? reinterpret_cast<T *>(p.out1) + prow0 * int64_t(p.N) : nullptr;
        const int64_t ld = p.N;
        const int n0 = c.n_tile * BN;
#pragma unroll 1
        for (int cc = cc_begin; cc < cc_end; cc += 32) {
            if (n0 + cc >= p.N) break;
            uint32_t r[32];
            ptx::tmem_ld32(tbase + cc, r);
            ptx::tmem_ld_wait();
            if (p.bias != nullptr) {
                float bv[32];
                load_bias32<T>(p, c.e, n0 + cc, p.N, bv);
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + bv[i]);
            }
            uint32_t w[RP::kWords];
#pragma unroll
            for (int i = 0; i < 32; i += 2)
                put2<T>(w, i, wgt * gelu_fwd<T>(__uint_as_float(r[i])), wgt * gelu_fwd<T>(__uint_as_float(r[i + 1])));
            stage_put_row<RP::kWords, PITCH>(es.stage, lane, w);
            __syncwarp();
            stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, [&](int rr) -> T * { return act + rr * ld; });
            __syncwarp();
            if (h) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) put2<T>(w, i, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                stage_put_row<RP::kWords, PITCH>(es.stage, lane, w);
                __syncwarp();
                stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, [&](int rr) -> T * { return h + rr * ld; });
                __syncwarp();
            }
        }
    } else if constexpr (MODE == MODE_ROUTER) {
        // Gate projection of the router: the accumulator row IS the token's logits (N = number of experts <= 256).  The
        // thread rounds them to the tensor dtype (what the reference's F.linear returns and what top-k then sees), writes
        // them out, keeps the k largest in a sorted register list (total order of order_key: NaN greatest, ties to the lower
        // expert index, as torch.topk / the stand-alone router kernel), and finishes with softmax over the k kept logits.
        constexpr int kMaxK = 8;
        const int64_t token = int64_t(c.m_tile) * BM + row_in_tile;
        const bool live = token < p.M;
        uint32_t tk[kMaxK];
        int te[kMaxK];
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) { tk[j] = 0u; te[j] = 0; }  // real keys are >= 0x007fffff (-inf)
        T *logits = reinterpret_cast<T *>(p.out0) + token * int64_t(p.N);
#pragma unroll 1
        for (int cc = cc_begin; cc < cc_end; cc += 32) {
            if (cc >= p.N) break;
            uint32_t r[32];
            ptx::tmem_ld32(tbase + cc, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i0 = 0; i0 < 32; i0 += 8) {
                if (cc + i0 >= p.N) break;  // N is a multiple of 8
                float v8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v8[i] = DT<T>::up(DT<T>::down(__uint_as_float(r[i0 + i])));
                if (live) store8<T>(logits + cc + i0, v8);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t key = order_key(v8[i]);
                    const int e = cc + i0 + i;
                    // branch-free insertion into the descending list; equal keys stay behind earlier (lower) experts
#pragma unroll
                    for (int j = kMaxK - 1; j >= 0; --j) {
                        const bool before_prev = j > 0 && key > tk[j - 1];
                        const bool before_cur = key > tk[j];
                        tk[j] = before_prev ? tk[j - 1] : (before_cur ? key : tk[j]);
                        te[j] = before_prev ? te[j - 1] : (before_cur ? e : te[j]);
                    }
                }
            }
        }
        if (live) {
            const float vmax = key_value(tk[0]);
            float ex[kMaxK];
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < kMaxK; ++j) {
                ex[j] = j < p.top_k ? expf(key_value(tk[j]) - vmax) : 0.0f;
                sum += ex[j];
            }
            T *wout = reinterpret_cast<T *>(p.out1) + token * int64_t(p.top_k);
            int32_t *iout = p.ids_out + token * int64_t(p.top_k);
#pragma unroll
            for (int j = 0; j < kMaxK; ++j) {
                if (j < p.top_k) {
                    wout[j] = DT<T>::down(ex[j] / sum);
                    iout[j] = te[j];
                }
            }
        }
    } else if constexpr (MODE == MODE_ACT1_BWD) {
        // backward of the above: g = dy W_proj (accumulator), d_pre = w * g * gelu'(pre), router-weight grad = sum gelu(pre) * g
        const int64_t prow0 = int64_t(c.m_tile) * BM + row0;
        const int32_t src = p.row_map[prow0 + lane];
        float wgt = (src >= 0) ? 1.0f : 0.0f;
        if (p.gate_w && src >= 0) wgt = DT<T>::up(reinterpret_cast<const T *>(p.gate_w)[src]);
        const int64_t ld = p.N;
        const T *h = reinterpret_cast<const T *>(p.h_in) + prow0 * ld;
        T *dh = reinterpret_cast<T *>(p.out0) + prow0 * ld;
        const int n0 = c.n_tile * BN;
        float dgate_w = 0.0f;
        uint2 pu[RP::kIters];
        auto h_row = [&](int rr) -> const T * { return h + rr * ld; };
        if (n0 + cc_begin < p.N) rows_prefetch<T>(pu, lane, n0 + cc_begin, p.N, h_row);
#pragma unroll 1
        for (int cc = cc_begin; cc < cc_end; cc += 32) {
            if (n0 + cc >= p.N) break;
            uint32_t wu[RP::kWords];
            rows_to_stage<T, PITCH>(es.stage, lane, pu);
            __syncwarp();
            stage_get_row<RP::kWords, PITCH>(es.stage, lane, wu);
            __syncwarp();
            if (cc + 32 < cc_end && n0 + cc + 32 < p.N) rows_prefetch<T>(pu, lane, n0 + cc + 32, p.N, h_row);
            uint32_t r[32];
            ptx::tmem_ld32(tbase + cc, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float x0, x1, a0, a1, d0, d1;
                get2<T>(wu, i, x0, x1);
                gelu_bwd<T>(x0, a0, d0);
                gelu_bwd<T>(x1, a1, d1);
                const float acc0 = __uint_as_float(r[i]), acc1 = __uint_as_float(r[i + 1]);
                dgate_w = fmaf(a0, acc0, dgate_w);
                dgate_w = fmaf(a1, acc1, dgate_w);
                put2<T>(wu, i, wgt * acc0 * d0, wgt * acc1 * d1);
            }
            stage_put_row<RP::kWords, PITCH>(es.stage, lane, wu);
            __syncwarp();
            stage_write_rows<T, PITCH>(es.stage, lane, n0 + cc, p.N, [&](int rr) -> T * { return dh + rr * ld; });
            __syncwarp();
        }
        if (p.dgates_part) p.dgates_part[int64_t(part) * p.cap + prow0 + lane] = dgate_w;
        else if (p.dgates && src >= 0) atomicAdd(p.dgates + src, dgate_w);
    }
}

constexpr size_t kGemmSmemBytes = kGemmSmemBytes_noepi + kEpiSmemBytes;

// ---- the kernel ------------------------------------------------------------------------------------
template <typename T, int MODE, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1) grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
    using TR = GemmTraits<T>;
    constexpr bool A_MN = (MODE == MODE_WGRAD);
    static_assert(MODE != MODE_WGRAD || B_MN, "wgrad contracts over rows: both operands are MN-major");
    constexpr int BK = TR::BK;
    constexpr uint32_t kIdesc = make_idesc<T>(A_MN, B_MN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_u32 & 1023u)) & 1023u;
    uint8_t *smem = smem_raw + pad;
    const uint32_t smem_a = raw_u32 + pad;
    const uint32_t smem_b = smem_a + kStages * kAStageBytes;
    SmemCtl *ctl = reinterpret_cast<SmemCtl *>(smem + kStages * (kAStageBytes + kBStageBytes));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // ---- setup -------------------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&ctl->tmem_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&ctl->tmem_empty[b]), 4);
        }
        ctl->abort_flag = 0;
        ctl->wait_limit_ns = p.wait_limit_ns ? p.wait_limit_ns : kWaitLimitNs;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&p.tmA);
        ptx::prefetch_tensormap(&p.tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_ptr), kTmemCols);
        ptx::tmem_relinquish();
    }
    {
        const int32_t *src = (MODE == MODE_WGRAD) ? p.padded_off : p.mtile_off;
        for (int i = threadIdx.x; i <= p.E; i += kGemmThreads) ctl->sched[i] = src ? src[i] : (i == 0 ? 0 : p.m_tiles_w);
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_ptr;
    int ntiles = total_tiles<MODE>(p, ctl);
    {
        // the tile tables come from device memory: never walk past the rows the caller allocated
        const int64_t rows = (MODE == MODE_WGRAD) ? int64_t(ctl->sched[p.E]) : int64_t(ctl->sched[p.E]) * BM;
        if (rows > p.cap || rows < 0) {
            ntiles = 0;
            if (threadIdx.x == 0 && p.dev_status) atomicOr(p.dev_status, CK_DEV_META);
        }
    }

    if (warp == 0) {
        // =================================== TMA producer ===================================
        // Lane 0 waits for free stages, arms the barrier and issues the tiled loads; when an operand is gathered
        // (TMA gather4 straight from the un-permuted token matrix) every lane fetches four rows of it.
        const bool gather_a = p.gather_fan > 0;
        const bool gather_b = (MODE == MODE_WGRAD) && p.gather_b_fan > 0;
        if (gather_a || gather_b) {
            int stage = 0;
            uint32_t phase = 0;
            int ok = 1;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                const TileCoord c = decode_tile<MODE, BK>(p, ctl, t);
                int ridx[4] = {0, 0, 0, 0};
                if (MODE != MODE_WGRAD && gather_a) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int32_t src = p.row_map[int64_t(c.m_tile) * BM + 4 * lane + q];
                        ridx[q] = src >= 0 ? src / p.gather_fan : 0;  // pad rows fetch token 0; the epilogue weights them by 0
                    }
                }
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    const uint32_t full = ptx::smem_u32(&ctl->full[stage]);
                    if (lane == 0) {
                        ok = wait_barrier(ptx::smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.dev_status) ? 1 : 0;
                        if (ok) ptx::mbar_expect_tx(full, kAStageBytes + kBStageBytes);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBStageBytes;
                    if constexpr (MODE == MODE_WGRAD) {
                        const int krow = c.k_row0 + kb * BK;
                        constexpr int kQ = BK / 4;  // gather4 operations per {128 B x BK rows} box
                        if (gather_a) {
                            for (int g = lane; g < (BM / TR::kMnBoxElems) * kQ; g += 32) {
                                const int j = g / kQ, q = g - j * kQ;
                                int r4[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int32_t src = p.row_map[krow + 4 * q + i];
                                    r4[i] = src >= 0 ? src / p.gather_fan : 0;  // the other operand is zero on pad rows
                                }
                                ptx::tma_gather4(sa + j * TR::kMnBoxBytes + q * 512, &p.tmA, full, c.m_tile * BM + j * TR::kMnBoxElems, r4[0], r4[1], r4[2], r4[3]);
                            }
                        } else if (lane == 0) {
#pragma unroll
                            for (int j = 0; j < BM / TR::kMnBoxElems; ++j)
                                ptx::tma_load_2d(sa + j * TR::kMnBoxBytes, &p.tmA, full, c.m_tile * BM + j * TR::kMnBoxElems, krow);
                        }
                        if (gather_b) {
                            for (int g = lane; g < (BN / TR::kMnBoxElems) * kQ; g += 32) {
                                const int j = g / kQ, q = g - j * kQ;
                                int r4[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int32_t src = p.row_map[krow + 4 * q + i];
                                    r4[i] = src >= 0 ? src / p.gather_b_fan : 0;
                                }
                                ptx::tma_gather4(sb + j * TR::kMnBoxBytes + q * 512, &p.tmB, full, c.n_tile * BN + j * TR::kMnBoxElems, r4[0], r4[1], r4[2], r4[3]);
                            }
                        } else if (lane == 0) {
#pragma unroll
                            for (int j = 0; j < BN / TR::kMnBoxElems; ++j)
                                ptx::tma_load_2d(sb + j * TR::kMnBoxBytes, &p.tmB, full, c.n_tile * BN + j * TR::kMnBoxElems, krow);
                        }
                    } else {
                        const int k0 = kb * BK;
                        if (gather_a) ptx::tma_gather4(sa + lane * 512, &p.tmA, full, k0, ridx[0], ridx[1], ridx[2], ridx[3]);
                        else if (lane == 0) ptx::tma_load_2d(sa, &p.tmA, full, k0, c.m_tile * BM);
                        if (lane == 0) {
                            if constexpr (B_MN) {
#pragma unroll
                                for (int j = 0; j < BN / TR::kMnBoxElems; ++j)
                                    ptx::tma_load_3d(sb + j * TR::kMnBoxBytes, &p.tmB, full, c.n_tile * BN + j * TR::kMnBoxElems, k0, c.e);
                            } else if constexpr (MODE == MODE_UP_ACT) {
                                // 128 rows of W_up followed by the matching 128 rows of W_gate
                                ptx::tma_load_3d(sb, &p.tmB, full, k0, c.n_tile * (BN / 2), c.e);
                                ptx::tma_load_3d(sb + kBStageBytes / 2, &p.tmB, full, k0, p.N + c.n_tile * (BN / 2), c.e);
                            } else {
                                ptx::tma_load_3d(sb, &p.tmB, full, k0, c.n_tile * BN, c.e);
                            }
                        }
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok && lane == 0) {
                // aborting: give copies already in flight time to land before the CTA exits
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        } else {
            // The whole warp runs the loop converged and one elected lane issues (uniform loop control, addresses and
            // coordinates); the next stage's "empty" barrier is probed before this stage's loads go out.
            const uint32_t elected = ptx::elect_one();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            bool ready = false;
            const uint32_t empty0 = ptx::smem_u32(&ctl->empty[0]);
            const uint32_t full0 = ptx::smem_u32(&ctl->full[0]);
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                const TileCoord c = decode_tile<MODE, BK>(p, ctl, t);
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    if (!ready) {
                        const bool w = wait_barrier(empty0 + 8u * stage, phase ^ 1u, ctl, p.dev_status);
                        if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    }
                    int nstage = stage + 1;
                    uint32_t nphase = phase;
                    if (nstage == kStages) { nstage = 0; nphase ^= 1u; }
                    ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(empty0 + 8u * nstage, nphase ^ 1u)) != 0;
                    const uint32_t full = full0 + 8u * stage;
                    ptx::mbar_expect_tx_elected(elected, full,
                                                MODE == MODE_ROUTER ? kAStageBytes + uint32_t(p.b_rows_lead) * kRowBytes : kAStageBytes + kBStageBytes);
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBStageBytes;
                    if constexpr (MODE == MODE_WGRAD) {
                        const int krow = c.k_row0 + kb * BK;
#pragma unroll
                        for (int j = 0; j < BM / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d_elected(elected, sa + j * TR::kMnBoxBytes, &p.tmA, full, c.m_tile * BM + j * TR::kMnBoxElems, krow);
#pragma unroll
                        for (int j = 0; j < BN / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d_elected(elected, sb + j * TR::kMnBoxBytes, &p.tmB, full, c.n_tile * BN + j * TR::kMnBoxElems, krow);
                    } else {
                        const int k0 = kb * BK;
                        ptx::tma_load_2d_elected(elected, sa, &p.tmA, full, k0, c.m_tile * BM);
                        if constexpr (B_MN) {
#pragma unroll
                            for (int j = 0; j < BN / TR::kMnBoxElems; ++j)
                                ptx::tma_load_3d_elected(elected, sb + j * TR::kMnBoxBytes, &p.tmB, full, c.n_tile * BN + j * TR::kMnBoxElems, k0, c.e);
                        } else if constexpr (MODE == MODE_UP_ACT) {
                            // 128 rows of W_up followed by the matching 128 rows of W_gate
                            ptx::tma_load_3d_elected(elected, sb, &p.tmB, full, k0, c.n_tile * (BN / 2), c.e);
                            ptx::tma_load_3d_elected(elected, sb + kBStageBytes / 2, &p.tmB, full, k0, p.N + c.n_tile * (BN / 2), c.e);
                        } else {
                            ptx::tma_load_3d_elected(elected, sb, &p.tmB, full, k0, c.n_tile * BN, c.e);
                        }
                    }
                    stage = nstage;
                    phase = nphase;
                }
            }
            if (!ok) {
                // aborting: give copies already in flight time to land before the CTA exits
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // =================================== MMA issuer =====================================
        // The warp runs the loop converged, one elected lane issues; the next stage's barrier is probed before this
        // stage's MMAs go out (see the CTA-pair kernel below for why the path between two k-blocks has to be short).
        {
            const uint32_t elected = ptx::elect_one();
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            bool ready = false;
            const uint32_t full0 = ptx::smem_u32(&ctl->full[0]);
            const uint32_t empty0 = ptx::smem_u32(&ctl->empty[0]);
            uint64_t adesc0, bdesc0;
            if constexpr (A_MN) adesc0 = ptx::umma_desc_mnmajor<TR::kTf32>(smem_a, TR::kMnBoxBytes);
            else adesc0 = ptx::umma_desc_kmajor(smem_a);
            if constexpr (B_MN) bdesc0 = ptx::umma_desc_mnmajor<TR::kTf32>(smem_b, TR::kMnBoxBytes);
            else bdesc0 = ptx::umma_desc_kmajor(smem_b);
            constexpr uint32_t kAStep = A_MN ? (TR::UMMA_K * kRowBytes) >> 4 : 32u >> 4;  // per k-step, in 16-byte units
            constexpr uint32_t kBStep = B_MN ? (TR::UMMA_K * kRowBytes) >> 4 : 32u >> 4;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++it) {
                const TileCoord c = decode_tile<MODE, BK>(p, ctl, t);
                const int buf = it & 1;
                {
                    const bool w = wait_barrier(ptx::smem_u32(&ctl->tmem_empty[buf]), ((uint32_t(it) >> 1) & 1u) ^ 1u, ctl, p.dev_status);
                    if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(buf) * BN;
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    if (!ready) {
                        const bool w = wait_barrier(full0 + 8u * stage, phase, ctl, p.dev_status);
                        if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    }
                    int nstage = stage + 1;
                    uint32_t nphase = phase;
                    if (nstage == kStages) { nstage = 0; nphase ^= 1u; }
                    ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(full0 + 8u * nstage, nphase)) != 0;
                    const uint64_t adesc = adesc0 + uint64_t(uint32_t(stage) * uint32_t(kAStageBytes >> 4));
                    const uint64_t bdesc = bdesc0 + uint64_t(uint32_t(stage) * uint32_t(kBStageBytes >> 4));
#pragma unroll
                    for (int k = 0; k < TR::kSteps; ++k)
                        ptx::umma_ss_elected<TR::kTf32>(elected, d_tmem, adesc + uint64_t(k * kAStep), bdesc + uint64_t(k * kBStep), kIdesc,
                                                        (kb | k) != 0 ? 1u : 0u);
                    ptx::tc_commit_elected(elected, empty0 + 8u * stage);  // frees the stage when these MMAs retire
                    stage = nstage;
                    phase = nphase;
                }
                if (!ok) break;
                ptx::tc_commit_elected(elected, ptx::smem_u32(&ctl->tmem_full[buf]));  // accumulator complete
            }
            if (!ok) {
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        }
        __syncwarp();
    } else {
        // =================================== epilogue =======================================
        const int quarter = warp & 3;              // TMEM lanes this warp may read
        const int row_in_tile = quarter * 32 + lane;
        uint8_t *epi_base = reinterpret_cast<uint8_t *>(ctl) + ((sizeof(SmemCtl) + 15) & ~size_t(15));
        EpiSmem es;
        es.stage = reinterpret_cast<uint32_t *>(epi_base + quarter * kStageWarpBytes);
        es.rowinfo = reinterpret_cast<int32_t *>(epi_base + kEpiWarps * kStageWarpBytes + quarter * 128);
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++it) {
            const TileCoord c = decode_tile<MODE, BK>(p, ctl, t);
            const int buf = it & 1;
            if (!wait_barrier<true>(ptx::smem_u32(&ctl->tmem_full[buf]), (uint32_t(it) >> 1) & 1u, ctl, p.dev_status)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t tbase = tmem_base + uint32_t(buf) * BN + (uint32_t(quarter * 32) << 16);
            epilogue_tile<T, MODE, kStagePitchWords>(p, c, tbase, row_in_tile, es, 0, (MODE == MODE_UP_ACT) ? BN / 2 : BN, c.n_tile);
            // release the accumulator buffer
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctl->tmem_empty[buf]));
        }
        if (MODE == MODE_STORE && p.n_peers > 0) __threadfence_system();  // stores to other GPUs land before the kernel ends
    }

    // ---- teardown ------------------------------------------------------------------------------------
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- CTA-pair variant --------------------------------------------------------------------------------
// Two CTAs on one TPC share a 256 x 256 tile: each owns 128 rows of it (its own A tile and accumulators)
// and loads only half of the B tile; one tcgen05.mma.cta_group::2 issued by the leader CTA reads both
// halves.  Per CTA and k-block that is 32 KiB instead of 48 KiB from L2 and leaves room for a 6-stage
// ring, which is what keeps the tensor pipe fed.  TMA loads are plain (non-multicast) per CTA; the
// leader's mbarrier collects the transaction bytes of both CTAs.
//
// Warp roles (one warp group of control warps + one or two warp groups of epilogue warps):
//   warp 0      TMA producer: B always, A when it is a plain tiled load
//   warp 1      MMA issuer (leader CTA only)
//   warps 2, 3  row-indexed A producer (UP_ACT / ACT_BWD with p.gather_fan > 0): warp 2 copies 16-byte pieces of the
//               routed token rows -- named by row_map, living in this GPU's memory or in a peer's -- straight into the
//               128-byte-swizzled stage with cp.async, so no grouped copy of the token matrix has to exist before the
//               GEMM; lane 0 of warp 3 forwards each finished k-block to the tensor core's barrier and, on the first
//               n-tile of every m-tile, stores the stage back out as the grouped copy (TMA store) that the
//               weight-gradient GEMM contracts over later.
//   warps 4..   epilogue; UP_ACT and ACT_BWD run two groups of four warps, each on half of the tile's columns, with
//               registers moved from the control warps to the epilogue warps (setmaxnreg).
#ifndef CK_PAIR_STAGES
#define CK_PAIR_STAGES 6
#endif
#ifndef CK_STORE_TWO_GROUPS
#define CK_STORE_TWO_GROUPS 1
#endif
constexpr int kBHalfStageBytes = kBStageBytes / 2;  // 16 KiB

template <typename T, int MODE>
struct PairCfg {
    static constexpr bool kHeavyEpilogue = (MODE == MODE_UP_ACT || MODE == MODE_ACT_BWD || MODE == MODE_UP_ACT1 || MODE == MODE_ACT1_BWD);
    // The plain row store is light per element, but with a short contraction (K of a fine-grained expert: 22 k-blocks) four
    // warps need longer for a tile's 128 x 256 results than the tensor pipe needs for the next tile: it gets eight as well.
    static constexpr bool kTwoGroups = kHeavyEpilogue || (CK_STORE_TWO_GROUPS && MODE == MODE_STORE);
    static constexpr int kEpiGroups = kTwoGroups ? 2 : 1;
    static constexpr int kEpiWarpsTotal = 4 * kEpiGroups;
    static constexpr int kThreads = 128 + 32 * kEpiWarpsTotal;
    // words per row of an epilogue warp's stage: 32 fp32 payload words, or 16 for rows of 16-bit results
    static constexpr int kPitch = (sizeof(T) == 4 || MODE == MODE_SCATTER_ADD) ? kStagePitchWords : kStagePitchWords16;
    static constexpr int kEpiBytes = kEpiWarpsTotal * (32 * kPitch * 4 + 32 * 4);
    // fp32 tensors with two epilogue groups need the wide stages for eight warps: one pipeline stage less
    static constexpr int kStages = (kTwoGroups && sizeof(T) == 4) ? CK_PAIR_STAGES - 1 : CK_PAIR_STAGES;
    static constexpr bool kCanGather = kHeavyEpilogue;
    // registers per thread after the hand-over (two epilogue groups only): 128 x 80 + 256 x 208 <= 384 x 168
    static constexpr int kRegsControl = 80;
    static constexpr int kRegsEpilogue = 208;
};

template <int STAGES>
struct SmemCtlPairT {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t a_full[STAGES];  // row-indexed A producer: the copies of one k-block have landed in this CTA
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_ptr;
    volatile int abort_flag;
    uint64_t wait_limit_ns;
    int32_t sched[kMaxSchedExperts + 1];   // m-tile offsets (or padded row offsets for WGRAD)
    int32_t psched[kMaxSchedExperts + 1];  // pair-tile offsets per expert; WGRAD: experts in the order their tiles are handed out
    int32_t gather_src[BM];                // row-indexed A producer: source of every row of the current tile
};

template <typename T, int MODE>
constexpr size_t pair_smem_bytes() {
    using C = PairCfg<T, MODE>;
    return 1024 + size_t(C::kStages) * (kAStageBytes + kBHalfStageBytes) + ((sizeof(SmemCtlPairT<C::kStages>) + 15) & ~size_t(15)) +
           C::kEpiBytes;
}

template <int MODE, int BK, typename Ctl>
__device__ __forceinline__ TileCoord decode_pair_tile(const GemmParams &p, const Ctl *ctl, int t, int rank) {
    TileCoord c;
    if constexpr (MODE == MODE_WGRAD) {
        const int mpairs = (p.m_tiles_w + 1) >> 1;
        const int per_e = mpairs * p.n_tiles;
        const int slot = t / per_e;
        c.e = ctl->psched[slot];
        const int local = t - slot * per_e;
        int pm;
        if (p.n_fastest) {
            pm = local / p.n_tiles;
            c.n_tile = local - pm * p.n_tiles;
        } else {
            c.n_tile = local / mpairs;
            pm = local - c.n_tile * mpairs;
        }
        c.m_tile = 2 * pm + rank;
        c.valid = c.m_tile < p.m_tiles_w;
        c.k_row0 = ctl->sched[c.e];
        c.k_iters = (ctl->sched[c.e + 1] - c.k_row0) / BK;
    } else {
        int lo = 0, hi = p.E;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (ctl->psched[mid] * p.n_tiles <= t) lo = mid; else hi = mid;
        }
        c.e = lo;
        const int p0 = ctl->psched[lo];
        const int pairs = ctl->psched[lo + 1] - p0;
        const int local = t - p0 * p.n_tiles;
        c.n_tile = local / pairs;
        const int pm = local - c.n_tile * pairs;
        const int m0 = ctl->sched[lo];
        const int mt = ctl->sched[lo + 1] - m0;
        c.valid = (2 * pm + rank) < mt;
        c.m_tile = m0 + 2 * pm + (c.valid ? rank : 0);  // an odd tail repeats the leader's rows; its result is dropped
        c.k_row0 = 0;
        c.k_iters = (p.K + BK - 1) / BK;
    }
    return c;
}

// Cycle accounting of the CTA-pair kernel's roles (compiled in with -DCK_GEMM_PROFILE only; `make EXTRA=-DCK_GEMM_PROFILE`).
// Every launch overwrites one row of counters per CTA; ck_gemm_profile_read copies them out.  This is how the issue
// loops were tuned: with the data always present (PROF_MMA_READY = PROF_KBLOCKS) and the tensor pipe still idle a sixth
// of the time, the limit was the issuing thread's own instruction stream, not memory.
#ifdef CK_GEMM_PROFILE
enum {
    PROF_MMA_WAIT_TMEM = 0,  // issuer: cycles waiting for the epilogue to free an accumulator buffer
    PROF_MMA_WAIT_FULL,      // issuer: cycles in the blocking wait for a stage (entered only when the probe said "not yet")
    PROF_MMA_TOTAL,          // issuer: cycles from first to last tile
    PROF_TILES,              // pair tiles of this CTA pair
    PROF_EPI_WAIT,           // first epilogue warp: cycles waiting for an accumulator
    PROF_EPI_BUSY,           // first epilogue warp: cycles in the fused tail
    PROF_EPI_LAST_WAIT,      // the same for the last epilogue warp
    PROF_EPI_LAST_BUSY,
    PROF_MMA_READY,          // issuer: k-blocks whose stage had already landed when the probe looked
    PROF_KBLOCKS,            // issuer: k-blocks
    PROF_TMA_READY,          // producer: k-blocks whose stage was already free
    PROF_TMA_WAIT,           // producer: cycles in the blocking wait for a free stage
    PROF_TMA_TOTAL,          // producer: cycles from first to last tile
    kProfSlots = 16
};
constexpr int kProfMaxCtas = 160;
__device__ unsigned long long g_prof[kProfMaxCtas * kProfSlots];
#define CK_PROF(...) __VA_ARGS__
#define PROF_T0() const long long _pt0 = clock64()
#define PROF_ADD(var) var += clock64() - _pt0
#define PROF_PUT(slot, v) g_prof[(blockIdx.x % kProfMaxCtas) * kProfSlots + (slot)] = (unsigned long long)(v)
#else
#define CK_PROF(...)
#define PROF_T0()
#define PROF_ADD(var)
#define PROF_PUT(slot, v)
#endif
template <typename T, int MODE, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<T, MODE>::kThreads, 1)
    grouped_gemm_pair_kernel(const __grid_constant__ GemmParams p) {
    using TR = GemmTraits<T>;
    using CFG = PairCfg<T, MODE>;
    using Ctl = SmemCtlPairT<CFG::kStages>;
    constexpr int kNStages = CFG::kStages;
    constexpr bool A_MN = (MODE == MODE_WGRAD);
    constexpr int BK = TR::BK;
    constexpr uint32_t kIdesc = make_idesc<T>(A_MN, B_MN, 2 * BM);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_u32 & 1023u)) & 1023u;
    uint8_t *smem = smem_raw + pad;
    const uint32_t smem_a = raw_u32 + pad;
    const uint32_t smem_b = smem_a + kNStages * kAStageBytes;
    Ctl *ctl = reinterpret_cast<Ctl *>(smem + kNStages * (kAStageBytes + kBHalfStageBytes));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rank = int(ptx::cluster_ctarank());  // 0 = leader
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    // A rows copied in by warps 2 and 3 (cp.async by row index) instead of a tiled TMA load
    const bool row_gather = CFG::kCanGather && p.gather_fan > 0;
    // transaction bytes per stage on the leader's barrier: both CTAs' TMA loads
    const uint32_t stage_tx = MODE == MODE_ROUTER ? 2u * kAStageBytes + uint32_t(p.b_rows_lead + p.b_rows_peer) * kRowBytes
                              : row_gather     ? 2u * kBHalfStageBytes
                                               : 2u * (kAStageBytes + kBHalfStageBytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kNStages; ++s) {
            // full: the producer's expect_tx arrival, plus the row forwarders of both CTAs
            ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), row_gather ? 3 : 1);
            // empty: the MMA commit, plus this CTA's row forwarder (its store back out has read the stage)
            ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), row_gather ? 2 : 1);
            ptx::mbar_init(ptx::smem_u32(&ctl->a_full[s]), 32);  // the copier warp's lanes, via their cp.async operations
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&ctl->tmem_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&ctl->tmem_empty[b]), 2 * CFG::kEpiWarpsTotal);  // the epilogue warps of both CTAs
        }
        ctl->abort_flag = 0;
        ctl->wait_limit_ns = p.wait_limit_ns ? p.wait_limit_ns : kWaitLimitNs;
        ptx::fence_mbar_init();
        if (!row_gather) ptx::prefetch_tensormap(&p.tmA);
        else if (p.rows_out) ptx::prefetch_tensormap(&p.tmOut);
        ptx::prefetch_tensormap(&p.tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(&ctl->tmem_ptr), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    {
        const int32_t *src = (MODE == MODE_WGRAD) ? p.padded_off : p.mtile_off;
        for (int i = threadIdx.x; i <= p.E; i += CFG::kThreads) ctl->sched[i] = src ? src[i] : (i == 0 ? 0 : p.m_tiles_w);
    }
    __syncthreads();
    if (MODE != MODE_WGRAD && threadIdx.x == 0) {
        int acc = 0;
        ctl->psched[0] = 0;
        for (int e = 0; e < p.E; ++e) {
            acc += (ctl->sched[e + 1] - ctl->sched[e] + 1) >> 1;
            ctl->psched[e + 1] = acc;
        }
    }
    if constexpr (MODE == MODE_WGRAD) {
        // A weight-gradient tile costs as many k-blocks as its expert has rows, and the tiles go to the CTA pairs round robin:
        // handing out the experts with the most rows first (ties by index) evens out the pairs' totals under skewed routing
        // (64 experts, top-8, biased router: heaviest pair 1.12 x the mean in expert order, 1.05-1.07 x in this order).
        // Up to kLptMaxExperts experts (one thread ranks one expert against all others); more experts keep their order.
        constexpr int kLptMaxExperts = 128;
        for (int e = threadIdx.x; e < p.E; e += CFG::kThreads) {
            int pos = e;
            if (p.E <= kLptMaxExperts) {
                const int rows = ctl->sched[e + 1] - ctl->sched[e];
                pos = 0;
                for (int f = 0; f < p.E; ++f) {
                    const int rf = ctl->sched[f + 1] - ctl->sched[f];
                    pos += (rf > rows || (rf == rows && f < e)) ? 1 : 0;
                }
            }
            ctl->psched[pos] = e;
        }
    }
    ptx::tc_fence_before();
    ptx::cluster_sync_all();  // barriers of both CTAs initialised and visible; TMEM address published
    ptx::tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_ptr;

    int ntiles;
    if constexpr (MODE == MODE_WGRAD) ntiles = p.E * ((p.m_tiles_w + 1) >> 1) * p.n_tiles;
    else ntiles = ctl->psched[p.E] * p.n_tiles;
    {
        const int64_t rows = (MODE == MODE_WGRAD) ? int64_t(ctl->sched[p.E]) : int64_t(ctl->sched[p.E]) * BM;
        if (rows > p.cap || rows < 0) {
            ntiles = 0;
            if (threadIdx.x == 0 && p.dev_status) atomicOr(p.dev_status, CK_DEV_META);
        }
    }

    // The control warps need few registers; with two epilogue groups they hand theirs over.  Each setmaxnreg sits inside
    // the branch its warp group runs, so that the register budget of one side never constrains the other side's code.
    if (warp < 4) {
    if constexpr (CFG::kEpiGroups == 2) ptx::setmaxnreg_dec<CFG::kRegsControl>();
    if (warp == 0) {
        // ================= TMA producer (one per CTA: own A rows, own half of B) =================
        const bool gather_a = (MODE == MODE_WGRAD) && p.gather_fan > 0;
        const bool gather_b = (MODE == MODE_WGRAD) && p.gather_b_fan > 0;
        if (gather_a || gather_b) {
            // wgrad with an operand gathered by TMA gather4 from the un-permuted matrix: every lane fetches four rows
            int stage = 0;
            uint32_t phase = 0;
            int ok = 1;
            for (int t = pair_id; t < ntiles && ok; t += num_pairs) {
                const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, rank);
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    if (lane == 0) {
                        ok = wait_barrier(ptx::smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.dev_status) ? 1 : 0;
                        if (ok && rank == 0) ptx::mbar_expect_tx(ptx::smem_u32(&ctl->full[stage]), stage_tx);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    const uint32_t full = ptx::mapa_shared(ptx::smem_u32(&ctl->full[stage]), 0);  // the leader's barrier
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBHalfStageBytes;
                    const int nb0 = c.n_tile * BN + rank * (BN / 2);  // this CTA's half of the N range
                    const int krow = c.k_row0 + kb * BK;
                    constexpr int kQ = BK / 4;
                    if (gather_a) {
                        for (int g = lane; g < (BM / TR::kMnBoxElems) * kQ; g += 32) {
                            const int j = g / kQ, q = g - j * kQ;
                            int r4[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int32_t src = p.row_map[krow + 4 * q + i];
                                r4[i] = src >= 0 ? src / p.gather_fan : 0;
                            }
                            ptx::tma_gather4_pair(sa + j * TR::kMnBoxBytes + q * 512, &p.tmA, full, c.m_tile * BM + j * TR::kMnBoxElems, r4[0], r4[1], r4[2], r4[3]);
                        }
                    } else if (lane == 0) {
#pragma unroll
                        for (int j = 0; j < BM / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d_pair(sa + j * TR::kMnBoxBytes, &p.tmA, full, c.m_tile * BM + j * TR::kMnBoxElems, krow);
                    }
                    if (gather_b) {
                        for (int g = lane; g < ((BN / 2) / TR::kMnBoxElems) * kQ; g += 32) {
                            const int j = g / kQ, q = g - j * kQ;
                            int r4[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int32_t src = p.row_map[krow + 4 * q + i];
                                r4[i] = src >= 0 ? src / p.gather_b_fan : 0;
                            }
                            ptx::tma_gather4_pair(sb + j * TR::kMnBoxBytes + q * 512, &p.tmB, full, nb0 + j * TR::kMnBoxElems, r4[0], r4[1], r4[2], r4[3]);
                        }
                    } else if (lane == 0) {
#pragma unroll
                        for (int j = 0; j < (BN / 2) / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d_pair(sb + j * TR::kMnBoxBytes, &p.tmB, full, nb0 + j * TR::kMnBoxElems, krow);
                    }
                    if (++stage == kNStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok && lane == 0) {
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        } else {
            // The whole warp runs the loop converged and one elected lane issues, so that loop control, addresses and
            // coordinates stay warp-uniform; the next stage's "empty" barrier is probed before this stage's loads go out.
            const uint32_t elected = ptx::elect_one();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            bool ready = false;
            const uint64_t pol_a = ptx::l2_policy(p.l2_hint_a), pol_b = ptx::l2_policy(p.l2_hint_b);
            const uint32_t empty0 = ptx::smem_u32(&ctl->empty[0]);
            const uint32_t full0_local = ptx::smem_u32(&ctl->full[0]);
            const uint32_t full0 = ptx::mapa_shared(full0_local, 0);  // the leader's barriers
            CK_PROF(long long pp_hit = 0, pp_wait = 0; const long long pp_start = clock64();)
            for (int t = pair_id; t < ntiles && ok; t += num_pairs) {
                TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, rank);
                const int nb0 = c.n_tile * BN + rank * (BN / 2);  // this CTA's half of the N range
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    CK_PROF(pp_hit += ready ? 1 : 0;)
                    if (!ready) {
                        PROF_T0();
                        const bool w = wait_barrier(empty0 + 8u * stage, phase ^ 1u, ctl, p.dev_status);
                        PROF_ADD(pp_wait);
                        if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    }
                    int nstage = stage + 1;
                    uint32_t nphase = phase;
                    if (nstage == kNStages) { nstage = 0; nphase ^= 1u; }
                    ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(empty0 + 8u * nstage, nphase ^ 1u)) != 0;
                    if (rank == 0) ptx::mbar_expect_tx_elected(elected, full0_local + 8u * stage, stage_tx);
                    const uint32_t full = full0 + 8u * stage;
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBHalfStageBytes;
                    if constexpr (MODE == MODE_WGRAD) {
                        const int krow = c.k_row0 + kb * BK;
#pragma unroll
                        for (int j = 0; j < BM / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d_pair_hint_elected(elected, sa + j * TR::kMnBoxBytes, &p.tmA, full, c.m_tile * BM + j * TR::kMnBoxElems, krow, pol_a);
#pragma unroll
                        for (int j = 0; j < (BN / 2) / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d_pair_hint_elected(elected, sb + j * TR::kMnBoxBytes, &p.tmB, full, nb0 + j * TR::kMnBoxElems, krow, pol_b);
                    } else {
                        const int k0 = kb * BK;
                        if (!row_gather) ptx::tma_load_2d_pair_hint_elected(elected, sa, &p.tmA, full, k0, c.m_tile * BM, pol_a);
                        if constexpr (B_MN) {
#pragma unroll
                            for (int j = 0; j < (BN / 2) / TR::kMnBoxElems; ++j)
                                ptx::tma_load_3d_pair_hint_elected(elected, sb + j * TR::kMnBoxBytes, &p.tmB, full, nb0 + j * TR::kMnBoxElems, k0, c.e, pol_b);
                        } else if constexpr (MODE == MODE_UP_ACT) {
                            // leader: 128 rows of W_up, peer: the matching 128 rows of W_gate
                            ptx::tma_load_3d_pair_hint_elected(elected, sb, &p.tmB, full, k0, rank * p.N + c.n_tile * (BN / 2), c.e, pol_b);
                        } else if constexpr (MODE == MODE_ROUTER) {
                            // only the rows of the gate weight that exist; the rest of the B tile feeds accumulator columns nobody reads
                            if (rank == 0) ptx::tma_load_3d_pair_hint_elected(elected, sb, &p.tmB, full, k0, 0, 0, pol_b);
                            else if (p.b_rows_peer > 0) ptx::tma_load_3d_pair_hint_elected(elected, sb, &p.tmOut, full, k0, BN / 2, 0, pol_b);
                        } else {
                            ptx::tma_load_3d_pair_hint_elected(elected, sb, &p.tmB, full, k0, nb0, c.e, pol_b);
                        }
                    }
                    stage = nstage;
                    phase = nphase;
                }
            }
            CK_PROF(if (elected) { PROF_PUT(PROF_TMA_READY, pp_hit); PROF_PUT(PROF_TMA_WAIT, pp_wait); PROF_PUT(PROF_TMA_TOTAL, clock64() - pp_start); })
            if (!ok) {
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ================= MMA issuer: the leader CTA drives both tensor cores =================
        // One thread feeds the tensor cores, and the instructions it runs between the last MMA of one k-block and the first
        // of the next are a gap in which the pipe drains (measured: 4 x 128 cycles of MMA + ~80 cycles of gap per k-block,
        // more when epilogue warps compete for the scheduler's issue slots).  The loop therefore keeps that path short: the
        // next stage's barrier is probed (non-blocking) BEFORE this stage's MMAs are issued, so the probe's latency hides
        // behind them and the blocking wait is only entered when the data really is late; operand descriptors advance by
        // constant adds; no tcgen05 fence sits between TMA-filled stages (the mbarrier orders the async-proxy writes).
        if (rank == 0) {
            // the whole warp runs the loop converged (uniform control and descriptor arithmetic); one elected lane issues
            const uint32_t elected = ptx::elect_one();
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            CK_PROF(long long prof_a = 0, prof_b = 0, prof_hit = 0, prof_n = 0; const long long prof_start = clock64();)
            const uint32_t full0 = ptx::smem_u32(&ctl->full[0]);
            const uint32_t empty0 = ptx::smem_u32(&ctl->empty[0]);
            // descriptors of stage 0, k-step 0; a stage further adds (stage bytes >> 4) to the low word
            uint64_t adesc0, bdesc0;
            if constexpr (A_MN) adesc0 = ptx::umma_desc_mnmajor<TR::kTf32>(smem_a, TR::kMnBoxBytes);
            else adesc0 = ptx::umma_desc_kmajor(smem_a);
            if constexpr (B_MN) bdesc0 = ptx::umma_desc_mnmajor<TR::kTf32>(smem_b, TR::kMnBoxBytes);
            else bdesc0 = ptx::umma_desc_kmajor(smem_b);
            constexpr uint32_t kAStep = A_MN ? (TR::UMMA_K * kRowBytes) >> 4 : 32u >> 4;  // per k-step, in 16-byte units
            constexpr uint32_t kBStep = B_MN ? (TR::UMMA_K * kRowBytes) >> 4 : 32u >> 4;
            auto probe = [&](int st, uint32_t ph) -> bool {
                // rows written by the other CTA's row-gather warps are released at cluster scope
                const bool r = row_gather ? ptx::mbar_test_wait_cluster(full0 + 8u * st, ph) : ptx::mbar_test_wait(full0 + 8u * st, ph);
                return __all_sync(0xffffffffu, r) != 0;  // one answer for the warp
            };
            bool ready = false;
            for (int t = pair_id; t < ntiles && ok; t += num_pairs, ++it) {
                const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, 0);
                const int buf = it & 1;
                { PROF_T0();
                const bool w = wait_barrier(ptx::smem_u32(&ctl->tmem_empty[buf]), ((uint32_t(it) >> 1) & 1u) ^ 1u, ctl, p.dev_status);
                PROF_ADD(prof_a);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; } }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(buf) * BN;
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    CK_PROF(prof_hit += ready ? 1 : 0; ++prof_n;)
                    if (!ready) {
                        PROF_T0();
                        const bool w = row_gather ? wait_barrier<false, true>(full0 + 8u * stage, phase, ctl, p.dev_status)
                                                  : wait_barrier<false, false>(full0 + 8u * stage, phase, ctl, p.dev_status);
                        PROF_ADD(prof_b);
                        if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    }
                    int nstage = stage + 1;
                    uint32_t nphase = phase;
                    if (nstage == kNStages) { nstage = 0; nphase ^= 1u; }
                    ready = probe(nstage, nphase);  // consumed in the next iteration (possibly of the next tile)
                    const uint64_t adesc = adesc0 + uint64_t(uint32_t(stage) * uint32_t(kAStageBytes >> 4));
                    const uint64_t bdesc = bdesc0 + uint64_t(uint32_t(stage) * uint32_t(kBHalfStageBytes >> 4));
#pragma unroll
                    for (int k = 0; k < TR::kSteps; ++k)
                        ptx::umma_ss_pair_elected<TR::kTf32>(elected, d_tmem, adesc + uint64_t(k * kAStep), bdesc + uint64_t(k * kBStep), kIdesc,
                                                             (kb | k) != 0 ? 1u : 0u);
                    ptx::tc_commit_pair_elected(elected, empty0 + 8u * stage, 3);  // frees the stage in both CTAs
                    stage = nstage;
                    phase = nphase;
                }
                if (!ok) break;
                ptx::tc_commit_pair_elected(elected, ptx::smem_u32(&ctl->tmem_full[buf]), 3);  // accumulators of both CTAs complete
            }
            CK_PROF(if (elected) {
                PROF_PUT(PROF_MMA_WAIT_TMEM, prof_a); PROF_PUT(PROF_MMA_WAIT_FULL, prof_b); PROF_PUT(PROF_MMA_TOTAL, clock64() - prof_start);
                PROF_PUT(PROF_TILES, it); PROF_PUT(PROF_MMA_READY, prof_hit); PROF_PUT(PROF_KBLOCKS, prof_n);
            })
            if (!ok) {
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        }
        __syncwarp();
    } else {
        // ================= row-indexed A producer =================
        // warp 2 copies, lane 0 of warp 3 forwards.  The copier never waits for its own copies: every lane ties the
        // k-block's cp.async operations to the CTA-local barrier a_full[stage] (cp.async.mbarrier.arrive.noinc) and runs
        // ahead as far as the ring allows.  The forwarder has no memory operations of its own in flight, so its proxy
        // fence and its release towards the leader CTA cost nothing: it waits for a_full, makes the rows visible to the
        // tensor core (generic -> async proxy), stores the stage back out where asked, and arrives on the leader's
        // full barrier.  Its second arrival, on this CTA's empty barrier, holds the stage until that store has read it.
        if constexpr (CFG::kCanGather) {
            if (row_gather && warp == 2) {
                const int chunk = lane & 7;         // which 16 bytes of a 128-byte row
                const int rsub = lane >> 3;         // rows rsub, rsub + 4, ... of the tile
                constexpr int kRowsPerLane = BM / 4;
                constexpr int kElemsPerChunk = 16 / int(sizeof(T));
                int stage = 0;
                uint32_t phase = 0;
                int ok = 1;
                for (int t = pair_id; t < ntiles && ok; t += num_pairs) {
                    const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, rank);
                    // sources of the tile's 128 rows, (peer << 26 | row) or -1 for a pad row, parked in shared memory
                    __syncwarp();  // every lane has issued the previous tile's copies
                    for (int r = lane; r < BM; r += 32) {
                        const int32_t g = p.row_map[int64_t(c.m_tile) * BM + r];
                        int32_t v = -1;
                        if (g >= 0) {
                            if (p.n_src_peers > 0) {
                                const int64_t rk = int64_t(g) / p.src_peer_rows;
                                if (rk < p.n_src_peers) v = int32_t((rk << kPeerRowBits) | ((int64_t(g) - rk * p.src_peer_rows) / p.gather_fan));
                                else if (p.dev_status) atomicOr(p.dev_status, CK_DEV_RANGE);
                            } else {
                                v = g / p.gather_fan;
                            }
                        }
                        ctl->gather_src[r] = v;
                    }
                    __syncwarp();
                    for (int kb = 0; kb < c.k_iters; ++kb) {
                        if (lane == 0) ok = wait_barrier(ptx::smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.dev_status) ? 1 : 0;
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (!ok) break;
                        const int col = kb * BK + chunk * kElemsPerChunk;
                        const bool in_k = col < p.K;
                        const uint32_t sa = smem_a + stage * kAStageBytes;
#pragma unroll 8
                        for (int i = 0; i < kRowsPerLane; ++i) {
                            const int r = rsub + 4 * i;
                            const uint32_t dst = sa + uint32_t(r) * kRowBytes + (uint32_t(chunk ^ (r & 7)) << 4);
                            const int32_t v = ctl->gather_src[r];
                            const bool live = v >= 0 && in_k;
                            const T *base = reinterpret_cast<const T *>(p.n_src_peers > 0 ? p.peer_src[live ? (v >> kPeerRowBits) : 0] : p.a_src);
                            const int64_t row = live ? int64_t(v & ((1 << kPeerRowBits) - 1)) : 0;
                            ptx::cp_async_16(dst, base + row * int64_t(p.K) + (live ? col : 0), live ? 16u : 0u);  // 0 bytes read: zero fill
                        }
                        ptx::cp_async_mbar_arrive_noinc(ptx::smem_u32(&ctl->a_full[stage]));
                        if (++stage == kNStages) { stage = 0; phase ^= 1u; }
                    }
                }
                ptx::cp_async_wait_all();  // nothing of this CTA's is in flight when it leaves
            } else if (row_gather && lane == 0) {
                const uint32_t leader_full0 = ptx::mapa_shared(ptx::smem_u32(&ctl->full[0]), 0);
                const bool store_rows = p.rows_out != nullptr;
                int stage = 0;
                uint32_t phase = 0;
                bool ok = true;
                for (int t = pair_id; t < ntiles && ok; t += num_pairs) {
                    const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, rank);
                    const bool store_tile = store_rows && c.valid && c.n_tile == 0;
                    for (int kb = 0; kb < c.k_iters; ++kb) {
                        if (!wait_barrier<true>(ptx::smem_u32(&ctl->a_full[stage]), phase, ctl, p.dev_status)) { ok = false; break; }
                        ptx::fence_proxy_async();
                        if (store_tile) {
                            ptx::tma_store_2d(&p.tmOut, smem_a + stage * kAStageBytes, kb * BK, c.m_tile * BM);
                            ptx::bulk_commit_group();
                        }
                        ptx::mbar_arrive_cluster(leader_full0 + uint32_t(stage) * 8u);
                        if (store_tile) ptx::bulk_wait_group_read<0>();  // the stage may be refilled once the store has read it
                        ptx::mbar_arrive(ptx::smem_u32(&ctl->empty[stage]));
                        if (++stage == kNStages) { stage = 0; phase ^= 1u; }
                    }
                }
                ptx::bulk_wait_group_all();  // the stores are complete before the kernel ends
            }
        }
        __syncwarp();
    }
    } else {
        // ================= epilogue: each CTA drains its own 128 rows =================
        if constexpr (CFG::kEpiGroups == 2) ptx::setmaxnreg_inc<CFG::kRegsEpilogue>();
        const int ew = warp - 4;
        const int group = ew >> 2;
        const int quarter = warp & 3;  // TMEM lanes this warp may read
        const int row_in_tile = quarter * 32 + lane;
        uint8_t *epi_base = reinterpret_cast<uint8_t *>(ctl) + ((sizeof(Ctl) + 15) & ~size_t(15));
        constexpr int kWarpStageBytes = 32 * CFG::kPitch * 4;
        EpiSmem es;
        es.stage = reinterpret_cast<uint32_t *>(epi_base + ew * kWarpStageBytes);
        es.rowinfo = reinterpret_cast<int32_t *>(epi_base + CFG::kEpiWarpsTotal * kWarpStageBytes + ew * 128);
        const uint32_t leader_empty0 = ptx::mapa_shared(ptx::smem_u32(&ctl->tmem_empty[0]), 0);
        const uint32_t leader_empty1 = ptx::mapa_shared(ptx::smem_u32(&ctl->tmem_empty[1]), 0);
        constexpr int kCols = (MODE == MODE_UP_ACT) ? BN / 2 : BN;       // accumulator columns the tail walks over
        constexpr int kColsPerGroup = kCols / CFG::kEpiGroups;
        int it = 0;
        bool ok = true;
        CK_PROF(long long prof_w = 0, prof_e = 0;)
        for (int t = pair_id; t < ntiles && ok; t += num_pairs, ++it) {
            const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, rank);
            const int buf = it & 1;
            { PROF_T0();
            if (!wait_barrier<true>(ptx::smem_u32(&ctl->tmem_full[buf]), (uint32_t(it) >> 1) & 1u, ctl, p.dev_status)) { ok = false; break; }
            PROF_ADD(prof_w); }
            ptx::tc_fence_after();
            const uint32_t tbase = tmem_base + uint32_t(buf) * BN + (uint32_t(quarter * 32) << 16);
            { PROF_T0();
            if (c.valid)
                epilogue_tile<T, MODE, CFG::kPitch>(p, c, tbase, row_in_tile, es, group * kColsPerGroup, (group + 1) * kColsPerGroup,
                                                    c.n_tile * CFG::kEpiGroups + group);
            PROF_ADD(prof_e); }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(buf ? leader_empty1 : leader_empty0);
        }
        CK_PROF(if (lane == 0 && ew == 0) { PROF_PUT(PROF_EPI_WAIT, prof_w); PROF_PUT(PROF_EPI_BUSY, prof_e); }
                if (lane == 0 && ew == CFG::kEpiWarpsTotal - 1) { PROF_PUT(PROF_EPI_LAST_WAIT, prof_w); PROF_PUT(PROF_EPI_LAST_BUSY, prof_e); })
        if (MODE == MODE_STORE && p.n_peers > 0) __threadfence_system();  // stores to other GPUs land before the kernel ends
    }

    // teardown: nobody leaves while the partner may still read its shared memory or signal its barriers
    ptx::tc_fence_before();
    ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr) {
        set_last_cuda_error(e, "cudaGetDriverEntryPointByVersion(cuTensorMapEncodeTiled)");
        return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
    return fn;
}

template <typename T>
static CUtensorMapDataType tm_dtype() {
    if (sizeof(T) == 4) return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    return DT<T>::code == CK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// rank-2 or rank-3 row-major tensor; dims innermost first; box innermost first
template <typename T>
static int encode_map(CUtensorMap *tm, const void *base, int rank, const uint64_t *dims, const uint32_t *box,
                      bool mn_major = false) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return CK_ERR_CUDA;
    cuuint64_t gdims[3];
    cuuint64_t gstrides[2];
    cuuint32_t gbox[3];
    cuuint32_t estr[3] = {1, 1, 1};
    uint64_t stride = sizeof(T);
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        stride *= dims[i];
        if (i < rank - 1) gstrides[i] = stride;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (dims[0] * sizeof(T)) % 16 != 0) return CK_ERR_SHAPE;
    // 32-bit MN-major operands are read by the MMA in the 128-byte swizzle with 32-byte atomicity
    const CUtensorMapSwizzle swz = (mn_major && sizeof(T) == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    CUresult r = fn(tm, tm_dtype<T>(), (cuuint32_t)rank, const_cast<void *>(base), gdims, gstrides, gbox, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char what[256];
        snprintf(what, sizeof(what), "cuTensorMapEncodeTiled(base=%p rank=%d dims=%llu,%llu,%llu box=%u,%u,%u elem=%d mn=%d) -> %d",
                 base, rank, (unsigned long long)gdims[0], (unsigned long long)gdims[1], (unsigned long long)(rank > 2 ? gdims[2] : 0),
                 gbox[0], gbox[1], rank > 2 ? gbox[2] : 0u, int(sizeof(T)), int(mn_major), int(r));
        set_last_cuda_error(cudaErrorInvalidValue, what);
        return CK_ERR_CUDA;
    }
    return CK_OK;
}

// 1 = CTA-pair kernels (cta_group::2), 0 = single-CTA kernels; initial value from CK_GEMM_CTA_PAIR
static int g_cta_pair = -1;
static bool use_cta_pair() {
    if (g_cta_pair < 0) {
        const char *e = getenv("CK_GEMM_CTA_PAIR");
        g_cta_pair = (e && e[0] == '0') ? 0 : 1;
    }
    return g_cta_pair != 0;
}

// SMs the persistent GEMM grids may occupy (0 = all of them); initial value from CK_GEMM_SMS.  A smaller budget leaves
// SMs free for kernels of other streams (row pulls over NVLink, collectives) to run beside a GEMM instead of in its tail.
static int g_sm_budget = -1;
static int gemm_sms() {
    if (g_sm_budget < 0) {
        const char *e = getenv("CK_GEMM_SMS");
        g_sm_budget = e ? atoi(e) : 0;
        if (g_sm_budget < 0) g_sm_budget = 0;
    }
    const int all = num_sms();
    return (g_sm_budget > 0 && g_sm_budget < all) ? g_sm_budget : all;
}

template <typename T, int MODE, bool B_MN>
static int launch_gemm(GemmParams &p, int64_t max_tiles, cudaStream_t stream) {
    // L2 policy of the operand loads.  Inside an expert the tiles run with one dimension fastest: the panels along it
    // are shared by the tiles in flight and then never needed again (evict-first); the panels of the other operand are
    // what every following wave comes back to (evict-last while one expert's share of them, rows x K, is of L2 size).
    if (MODE == MODE_WGRAD) {
        p.l2_hint_a = p.n_fastest ? ptx::L2_EVICT_NORMAL : ptx::L2_EVICT_LAST;
        p.l2_hint_b = p.n_fastest ? ptx::L2_EVICT_LAST : ptx::L2_EVICT_NORMAL;
    } else {
        p.l2_hint_a = (p.K <= 8192) ? ptx::L2_EVICT_LAST : ptx::L2_EVICT_NORMAL;
        p.l2_hint_b = ptx::L2_EVICT_NORMAL;
    }
    if (use_cta_pair()) {
        auto kern2 = grouped_gemm_pair_kernel<T, MODE, B_MN>;
        constexpr size_t smem_bytes = pair_smem_bytes<T, MODE>();
        static_assert(smem_bytes <= 227 * 1024, "the CTA-pair kernel's shared memory exceeds what one CTA may own");
        CK_CUDA_TRY(cudaFuncSetAttribute(kern2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
        int64_t pairs = gemm_sms() / 2;
        if (pairs > max_tiles) pairs = max_tiles;  // upper bound: a pair tile covers at least one single tile
        if (pairs < 1) return CK_OK;
        kern2<<<dim3((unsigned)(2 * pairs)), PairCfg<T, MODE>::kThreads, smem_bytes, stream>>>(p);
        CK_LAUNCH_CHECK("grouped_gemm_pair_kernel");
        return CK_OK;
    }
    auto kern = grouped_gemm_kernel<T, MODE, B_MN>;
    CK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmemBytes));
    int64_t grid = gemm_sms();
    if (grid > max_tiles) grid = max_tiles;
    if (grid < 1) return CK_OK;
    kern<<<dim3((unsigned)grid), kGemmThreads, kGemmSmemBytes, stream>>>(p);
    CK_LAUNCH_CHECK("grouped_gemm_kernel");
    return CK_OK;
}

// activations [cap, K] as K-major A: box {BK, 128}
template <typename T>
static int map_a_kmajor(CUtensorMap *tm, const void *a, int64_t cap, int K) {
    const uint64_t dims[2] = {uint64_t(K), uint64_t(cap)};
    const uint32_t box[2] = {uint32_t(GemmTraits<T>::BK), uint32_t(BM)};
    return encode_map<T>(tm, a, 2, dims, box);
}
// weights [E, rows, K] as K-major B: box {BK, box_rows, 1}
template <typename T>
static int map_w_kmajor(CUtensorMap *tm, const void *w, int E, int rows, int K, int box_rows) {
    const uint64_t dims[3] = {uint64_t(K), uint64_t(rows), uint64_t(E)};
    const uint32_t box[3] = {uint32_t(GemmTraits<T>::BK), uint32_t(box_rows), 1};
    return encode_map<T>(tm, w, 3, dims, box);
}
// weights [E, K, N] as MN-major B: box {128 bytes of N, BK rows of K, 1}
template <typename T>
static int map_w_mnmajor(CUtensorMap *tm, const void *w, int E, int K, int N) {
    const uint64_t dims[3] = {uint64_t(N), uint64_t(K), uint64_t(E)};
    const uint32_t box[3] = {uint32_t(GemmTraits<T>::kMnBoxElems), uint32_t(GemmTraits<T>::BK), 1};
    return encode_map<T>(tm, w, 3, dims, box, true);
}
// activations [cap, cols] as MN-major operand of wgrad: box {128 bytes of cols, BK rows}
template <typename T>
static int map_act_mnmajor(CUtensorMap *tm, const void *a, int64_t cap, int cols) {
    const uint64_t dims[2] = {uint64_t(cols), uint64_t(cap)};
    const uint32_t box[2] = {uint32_t(GemmTraits<T>::kMnBoxElems), uint32_t(GemmTraits<T>::BK)};
    return encode_map<T>(tm, a, 2, dims, box, true);
}

// token matrix [rows, K] addressed row by row for TMA gather4: box {BK, 1}
template <typename T>
static int map_a_gather(CUtensorMap *tm, const void *a, int64_t rows, int K) {
    const uint64_t dims[2] = {uint64_t(K), uint64_t(rows)};
    const uint32_t box[2] = {uint32_t(GemmTraits<T>::BK), 1};
    return encode_map<T>(tm, a, 2, dims, box);
}

static bool dims_ok(int64_t cap, int a, int b) { return cap > 0 && cap % BM == 0 && a > 0 && b > 0 && a % 8 == 0 && b % 8 == 0; }

// Where the A rows of the up projection / dgrad-down come from when they are not a ready-made grouped matrix.
struct RowSource {
    const void *src = nullptr;           // un-permuted [src_rows, K] matrix on this GPU
    int64_t src_rows = 0;
    int fan = 0;                         // > 0: padded row p reads row row_map[p] / fan (local) or (g % S) / fan of peer g / S
    const void *const *peers = nullptr;  // host array of n_peers device pointers (every rank's matrix as mapped here)
    int n_peers = 0;
    int64_t rows_per_peer = 0;           // S: global slots per rank
    void *rows_out = nullptr;            // also write the gathered rows out as the grouped [cap, K] matrix
};

// grouped copy [cap, K] written back from the A stages: box {BK, 128} (one stage)
template <typename T>
static int map_rows_out(CUtensorMap *tm, void *a, int64_t cap, int K) {
    const uint64_t dims[2] = {uint64_t(K), uint64_t(cap)};
    const uint32_t box[2] = {uint32_t(GemmTraits<T>::BK), uint32_t(BM)};
    return encode_map<T>(tm, a, 2, dims, box);
}

// fills the A side of the launch: a tiled map of the grouped matrix, or the row-index source
template <typename T>
static int set_a_operand(GemmParams &p, const void *grouped, const RowSource *rs, int64_t cap, int K) {
    if (!rs || rs->fan <= 0) return map_a_kmajor<T>(&p.tmA, grouped, cap, K);
    p.gather_fan = rs->fan;
    if (!use_cta_pair()) {
        // single-CTA flavour: TMA gather4 from the local matrix; no peers, no write-back
        if (rs->n_peers > 0 || rs->rows_out) return CK_ERR_UNSUPPORTED;
        return map_a_gather<T>(&p.tmA, rs->src, rs->src_rows, K);
    }
    if (rs->n_peers > 0) {
        if (rs->n_peers > CK_MAX_PEERS || rs->rows_per_peer <= 0) return CK_ERR_SHAPE;
        if (rs->rows_per_peer > (int64_t(1) << kPeerRowBits) || rs->rows_per_peer * rs->n_peers > INT32_MAX) return CK_ERR_RANGE;
        p.n_src_peers = rs->n_peers;
        p.src_peer_rows = rs->rows_per_peer;
        for (int i = 0; i < rs->n_peers; ++i) {
            if (!rs->peers[i] || (reinterpret_cast<uintptr_t>(rs->peers[i]) & 15)) return CK_ERR_SHAPE;
            p.peer_src[i] = rs->peers[i];
        }
    } else {
        if (!rs->src || (reinterpret_cast<uintptr_t>(rs->src) & 15) || rs->src_rows <= 0 || rs->src_rows > (int64_t(1) << kPeerRowBits)) return CK_ERR_SHAPE;
        p.a_src = rs->src;
    }
    if ((int64_t(K) * int64_t(sizeof(T))) % 16 != 0) return CK_ERR_SHAPE;  // 16-byte pieces of whole rows
    if (rs->rows_out) {
        p.rows_out = rs->rows_out;
        return map_rows_out<T>(&p.tmOut, rs->rows_out, cap, K);
    }
    return CK_OK;
}

static bool act_is_gated(int act_kind) { return act_kind == CK_ACT_SWIGLU || act_kind == CK_ACT_GLU; }
static bool act_is_known(int act_kind) { return act_is_gated(act_kind) || act_kind == CK_ACT_GELU_TANH; }

template <typename T>
static int up_act_fwd_t(const void *xg, const void *wfc, const void *b_fc, const void *gate_w, const int32_t *row_map,
                        const int32_t *mtile_off, void *act, void *h, int E, int64_t cap, int H, int I, int act_kind,
                        int32_t *dev_status, cudaStream_t stream, const RowSource *rs = nullptr) {
    GemmParams p = {};
    p.cap = cap;
    int rc;
    if ((rc = set_a_operand<T>(p, xg, rs, cap, H)) != CK_OK) return rc;
    p.mtile_off = mtile_off; p.row_map = row_map; p.gate_w = gate_w; p.out0 = act; p.out1 = h; p.dev_status = dev_status;
    p.E = E; p.N = I; p.K = H; p.act_kind = act_kind; p.top_k = 1;
    p.bias = b_fc;
    if (act_is_gated(act_kind)) {
        // B tile = 128 rows of W_up | the matching 128 rows of W_gate
        if ((rc = map_w_kmajor<T>(&p.tmB, wfc, E, 2 * I, H, BN / 2)) != CK_OK) return rc;
        p.n_tiles = (I + BN / 2 - 1) / (BN / 2);
        p.bias_ld = 2 * I;
        return launch_gemm<T, MODE_UP_ACT, false>(p, (cap / BM) * p.n_tiles, stream);
    }
    if ((rc = map_w_kmajor<T>(&p.tmB, wfc, E, I, H, use_cta_pair() ? BN / 2 : BN)) != CK_OK) return rc;
    p.n_tiles = (I + BN - 1) / BN;
    p.bias_ld = I;
    return launch_gemm<T, MODE_UP_ACT1, false>(p, (cap / BM) * p.n_tiles, stream);
}

template <typename T>
static int down_combine_fwd_t(const void *act, const void *wproj, const void *b_proj, const void *gate_w, const int32_t *row_map,
                              const int32_t *mtile_off, float *out32, int E, int64_t cap, int H, int I, int top_k,
                              int32_t *dev_status, cudaStream_t stream) {
    GemmParams p = {};
    p.cap = cap;
    int rc;
    if ((rc = map_a_kmajor<T>(&p.tmA, act, cap, I)) != CK_OK) return rc;
    if ((rc = map_w_kmajor<T>(&p.tmB, wproj, E, H, I, use_cta_pair() ? BN / 2 : BN)) != CK_OK) return rc;
    p.mtile_off = mtile_off; p.row_map = row_map; p.out32 = out32; p.dev_status = dev_status;
    p.E = E; p.n_tiles = (H + BN - 1) / BN; p.N = H; p.K = I; p.top_k = top_k;
    p.bias = b_proj; p.bias_ld = H; p.gate_w = gate_w;
    return launch_gemm<T, MODE_SCATTER_ADD, false>(p, (cap / BM) * p.n_tiles, stream);
}

template <typename T>
static int dgrad_down_t(const void *dyg, const void *wproj, const void *h, const void *gate_w, const int32_t *row_map,
                        const int32_t *mtile_off, void *dh, float *dgates, float *dgates_part, int E, int64_t cap, int H,
                        int I, int act_kind, int32_t *dev_status, cudaStream_t stream, const RowSource *rs = nullptr) {
    GemmParams p = {};
    p.cap = cap;
    int rc;
    if ((rc = set_a_operand<T>(p, dyg, rs, cap, H)) != CK_OK) return rc;
    if ((rc = map_w_mnmajor<T>(&p.tmB, wproj, E, H, I)) != CK_OK) return rc;
    p.mtile_off = mtile_off; p.row_map = row_map; p.gate_w = gate_w; p.h_in = h; p.out0 = dh; p.dgates = dgates;
    p.dgates_part = dgates_part;
    p.dev_status = dev_status;
    p.E = E; p.n_tiles = (I + BN - 1) / BN; p.N = I; p.K = H; p.act_kind = act_kind; p.top_k = 1;
    if (act_is_gated(act_kind)) return launch_gemm<T, MODE_ACT_BWD, true>(p, (cap / BM) * p.n_tiles, stream);
    return launch_gemm<T, MODE_ACT1_BWD, true>(p, (cap / BM) * p.n_tiles, stream);
}

// dgates[row_map[p]] = sum over the parts, in part order, of part[i * cap + p]   (one thread per padded row)
__global__ void reduce_dgates_kernel(const float *__restrict__ part, int n_parts, int64_t cap, const int32_t *__restrict__ row_map,
                                     const int32_t *__restrict__ padded_off, int E, float *__restrict__ dgates) {
    int64_t rows = padded_off[E];
    if (rows > cap) rows = cap;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t r = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; r < rows; r += stride) {
        const int32_t dst = row_map[r];
        if (dst < 0) continue;
        float acc = 0.0f;
        for (int i = 0; i < n_parts; ++i) acc += part[int64_t(i) * cap + r];
        dgates[dst] = acc;
    }
}

template <typename T>
static int dgrad_up_t(const void *dh, const void *wfc, const int32_t *row_map, const int32_t *mtile_off, float *dx32,
                      int E, int64_t cap, int H, int I2, int top_k, int32_t *dev_status, cudaStream_t stream) {
    GemmParams p = {};
    p.cap = cap;
    int rc;
    if ((rc = map_a_kmajor<T>(&p.tmA, dh, cap, I2)) != CK_OK) return rc;
    if ((rc = map_w_mnmajor<T>(&p.tmB, wfc, E, I2, H)) != CK_OK) return rc;
    p.mtile_off = mtile_off; p.row_map = row_map; p.out32 = dx32; p.dev_status = dev_status;
    p.E = E; p.n_tiles = (H + BN - 1) / BN; p.N = H; p.K = I2; p.top_k = top_k;
    return launch_gemm<T, MODE_SCATTER_ADD, true>(p, (cap / BM) * p.n_tiles, stream);
}

// un-permuted [rows, cols] matrix addressed row by row as an MN-major wgrad operand: box {128 bytes of cols, 1}
template <typename T>
static int map_act_mn_gather(CUtensorMap *tm, const void *a, int64_t rows, int cols) {
    const uint64_t dims[2] = {uint64_t(cols), uint64_t(rows)};
    const uint32_t box[2] = {uint32_t(GemmTraits<T>::kMnBoxElems), 1};
    return encode_map<T>(tm, a, 2, dims, box, true);
}

template <typename T>
static int wgrad_t(const void *a, const void *b, const int32_t *padded_off, void *dw, int E, int64_t cap, int M, int N,
                   int32_t *dev_status, cudaStream_t stream, const int32_t *row_map = nullptr, int64_t a_rows = 0,
                   int a_fan = 0, int64_t b_rows = 0, int b_fan = 0) {
    GemmParams p = {};
    p.cap = cap;
    int rc;
    if (a_fan > 0) {
        if ((rc = map_act_mn_gather<T>(&p.tmA, a, a_rows, M)) != CK_OK) return rc;
    } else if ((rc = map_act_mnmajor<T>(&p.tmA, a, cap, M)) != CK_OK) return rc;
    if (b_fan > 0) {
        if ((rc = map_act_mn_gather<T>(&p.tmB, b, b_rows, N)) != CK_OK) return rc;
    } else if ((rc = map_act_mnmajor<T>(&p.tmB, b, cap, N)) != CK_OK) return rc;
    p.gather_fan = a_fan; p.gather_b_fan = b_fan; p.row_map = row_map;
    p.padded_off = padded_off; p.out0 = dw; p.dev_status = dev_status;
    p.E = E; p.m_tiles_w = (M + BM - 1) / BM; p.n_tiles = (N + BN - 1) / BN; p.M = M; p.N = N;
    // keep the smaller operand panel set L2 resident: iterate the shorter output dimension fastest
    p.n_fastest = (N <= M) ? 1 : 0;
    return launch_gemm<T, MODE_WGRAD, true>(p, int64_t(E) * p.m_tiles_w * p.n_tiles, stream);
}

template <typename T>
static int grouped_linear_t(const void *x, const void *w, const int32_t *mtile_off, const int32_t *row_map, void *y, int E,
                            int64_t cap, int N, int K, int trans_w, int32_t *dev_status, cudaStream_t stream,
                            const int32_t *dst_flat = nullptr, void *const *peer_out = nullptr, int n_peers = 0,
                            int64_t peer_rows = 0, const void *bias = nullptr, const void *gate_w = nullptr) {
    GemmParams p = {};
    p.cap = cap;
    p.bias = bias; p.bias_ld = N; p.gate_w = gate_w;
    int rc;
    if ((rc = map_a_kmajor<T>(&p.tmA, x, cap, K)) != CK_OK) return rc;
    p.mtile_off = mtile_off; p.row_map = row_map; p.out0 = y; p.dev_status = dev_status;
    if (n_peers > 0) {
        p.dst_flat = dst_flat; p.n_peers = n_peers; p.peer_rows = peer_rows;
        for (int i = 0; i < n_peers; ++i) p.peer_out[i] = peer_out[i];
        p.out0 = peer_out[0];  // only the base the row indices are taken against; nothing is stored through it
    }
    p.E = E; p.n_tiles = (N + BN - 1) / BN; p.N = N; p.K = K; p.top_k = 1;
    if (trans_w) {
        if ((rc = map_w_mnmajor<T>(&p.tmB, w, E, K, N)) != CK_OK) return rc;
        return launch_gemm<T, MODE_STORE, true>(p, (cap / BM) * p.n_tiles, stream);
    }
    if ((rc = map_w_kmajor<T>(&p.tmB, w, E, N, K, use_cta_pair() ? BN / 2 : BN)) != CK_OK) return rc;
    return launch_gemm<T, MODE_STORE, false>(p, (cap / BM) * p.n_tiles, stream);
}

// ---- gate projection + router tail ---------------------------------------------------------------------------
// logits[t, :] = x[t, :] @ gate_w^T (rounded to T), top-k / softmax / ids from the epilogue.  The tokens are one group of
// ceil(tokens / 128) m-tiles (no routing tables needed yet: this IS the step that produces the expert ids); rows past
// `tokens` in the last tile are zero-filled by TMA and never written.
template <typename T>
static int router_gate_t(const void *x, const void *gate_w, void *logits, void *weights, int32_t *ids, int64_t tokens, int H,
                         int E, int top_k, int32_t *dev_status, cudaStream_t stream) {
    GemmParams p = {};
    const int64_t m_tiles = (tokens + BM - 1) / BM;
    p.cap = m_tiles * BM;
    int rc;
    if ((rc = map_a_kmajor<T>(&p.tmA, x, tokens, H)) != CK_OK) return rc;
    if (use_cta_pair()) {
        p.b_rows_lead = E < BN / 2 ? E : BN / 2;
        p.b_rows_peer = E > BN / 2 ? E - BN / 2 : 0;
        if ((rc = map_w_kmajor<T>(&p.tmB, gate_w, 1, E, H, p.b_rows_lead)) != CK_OK) return rc;
        if (p.b_rows_peer > 0 && (rc = map_w_kmajor<T>(&p.tmOut, gate_w, 1, E, H, p.b_rows_peer)) != CK_OK) return rc;
    } else {
        p.b_rows_lead = E;
        if ((rc = map_w_kmajor<T>(&p.tmB, gate_w, 1, E, H, E)) != CK_OK) return rc;
    }
    p.mtile_off = nullptr; p.m_tiles_w = int(m_tiles);
    p.out0 = logits; p.out1 = weights; p.ids_out = ids; p.dev_status = dev_status;
    p.E = 1; p.n_tiles = 1; p.N = E; p.K = H; p.M = int(tokens); p.top_k = top_k;
    return launch_gemm<T, MODE_ROUTER, false>(p, m_tiles, stream);
}

// ---- bias gradients (layers with add_bias=True) -------------------------------------------------------------
// out[e, n] = sum over the padded rows p of expert e of scale(p) * rows[p, n], scale(p) = gate_w[row_map[p]] (1 without
// gate_w; pad rows are zero).  One block per (expert, 256-column slab): the eight warps take every eighth row, each lane
// eight consecutive columns, then the warps' sums are added through shared memory in a fixed order (reproducible).
template <typename T>
__global__ void __launch_bounds__(256) bias_grad_kernel(const T *__restrict__ rows, int64_t ld, int N, const int32_t *__restrict__ row_map,
                                                        const T *__restrict__ gate_w, const int32_t *__restrict__ padded_off,
                                                        T *__restrict__ out) {
    __shared__ float red[8][256];
    const int e = blockIdx.x;
    const int col0 = blockIdx.y * 256 + (threadIdx.x & 31) * 8;
    const int warp = threadIdx.x >> 5;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (col0 < N) {
        for (int64_t r = padded_off[e] + warp; r < padded_off[e + 1]; r += 8) {
            float scale = 1.0f;
            if (gate_w != nullptr) {
                const int32_t src = row_map[r];
                if (src < 0) continue;
                scale = DT<T>::up(gate_w[src]);
            }
            float v[8];
            if (col0 + 8 <= N) {
                load8<T>(rows + r * ld + col0, v);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = col0 + i < N ? DT<T>::up(rows[r * ld + col0 + i]) : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(scale, v[i], acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[warp][(threadIdx.x & 31) * 8 + i] = acc[i];
    __syncthreads();
    const int col = blockIdx.y * 256 + threadIdx.x;
    if (col < N) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
        out[int64_t(e) * N + col] = DT<T>::down(s);
    }
}

// part[p] = rows[p, :] . bias[e(p), :]   (one warp per padded row; the bias term of the router-weight gradient)
template <typename T>
__global__ void __launch_bounds__(256) bias_dots_kernel(const T *__restrict__ rows, int N, const T *__restrict__ bias,
                                                        const int32_t *__restrict__ padded_off, int E, float *__restrict__ part) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const int64_t total = padded_off[E];
    for (int64_t r = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < total; r += warps) {
        int lo = 0, hi = E;  // expert of row r: padded_off[e] <= r < padded_off[e + 1]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (padded_off[mid] <= r) lo = mid; else hi = mid;
        }
        const T *x = rows + r * int64_t(N);
        const T *b = bias + int64_t(lo) * N;
        float acc = 0.0f;
        for (int c = lane * 8; c < N; c += 256) {  // N is a multiple of 8
            float xv[8], bv[8];
            load8<T>(x + c, xv);
            load8<T>(b + c, bv);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc = fmaf(xv[i], bv[i], acc);
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
        if (lane == 0) part[r] = acc;
    }
}

template <typename T>
static int bias_grad_t(const void *rows, int64_t cap, int N, const int32_t *row_map, const void *gate_w, const int32_t *padded_off,
                       int E, void *out, cudaStream_t stream) {
    (void)cap;
    bias_grad_kernel<T><<<dim3(unsigned(E), unsigned((N + 255) / 256)), 256, 0, stream>>>((const T *)rows, N, N, row_map, (const T *)gate_w,
                                                                                           padded_off, (T *)out);
    CK_LAUNCH_CHECK("bias_grad_kernel");
    return CK_OK;
}
template <typename T>
static int bias_dots_t(const void *rows, int64_t cap, int N, const void *bias, const int32_t *padded_off, int E, float *part,
                       cudaStream_t stream) {
    int64_t blocks = ceil_div64(cap, 8);
    const int64_t limit = int64_t(num_sms()) * 8;
    if (blocks > limit) blocks = limit;
    bias_dots_kernel<T><<<unsigned(blocks), 256, 0, stream>>>((const T *)rows, N, (const T *)bias, padded_off, E, part);
    CK_LAUNCH_CHECK("bias_dots_kernel");
    return CK_OK;
}

// ---- self test of the bounded wait --------------------------------------------------------------------
// One CTA, no TMA, no TMEM, no cluster: two lanes wait on an mbarrier that nobody ever arrives at, with the same
// wait_barrier the GEMM roles use.  The first lane to run out of time raises the abort flag and CK_DEV_TIMEOUT; the
// other leaves through the flag (or its own limit).  The kernel then returns normally.
struct WaitTestCtl {
    uint64_t bar;
    volatile int abort_flag;
    uint64_t wait_limit_ns;
};

__global__ void __launch_bounds__(64) wait_timeout_test_kernel(uint64_t limit_ns, int32_t *result, int32_t *dev_status) {
    __shared__ WaitTestCtl ctl;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&ctl.bar), 1);
        ctl.abort_flag = 0;
        ctl.wait_limit_ns = limit_ns;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    const uint64_t t0 = ptx::globaltimer_ns();
    int ok = 1;
    if (threadIdx.x == 0) ok = wait_barrier(ptx::smem_u32(&ctl.bar), 0u, &ctl, dev_status) ? 1 : 0;
    if (threadIdx.x == 32) ok = wait_barrier<true>(ptx::smem_u32(&ctl.bar), 0u, &ctl, dev_status) ? 1 : 0;
    const uint64_t waited = ptx::globaltimer_ns() - t0;
    if (threadIdx.x == 0) { result[0] = ok; result[2] = int32_t(waited > 0x7fffffffull ? 0x7fffffffull : waited); }
    if (threadIdx.x == 32) result[1] = ok;
    __syncthreads();
    if (threadIdx.x == 0) result[3] = ctl.abort_flag;
}

}  // namespace ck

using namespace ck;

extern "C" int ck_test_wait_timeout(int64_t limit_ns, int32_t *result4, int32_t *dev_status, void *stream) {
    if (!result4 || !dev_status) return CK_ERR_SHAPE;
    if (limit_ns <= 0 || limit_ns > 100000000ll) return CK_ERR_RANGE;  // at most 100 ms: this entry never stalls a GPU
    wait_timeout_test_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(uint64_t(limit_ns), result4, dev_status);
    CK_LAUNCH_CHECK("wait_timeout_test_kernel");
    return CK_OK;
}

#ifdef CK_GEMM_PROFILE
// Profile builds only: copies the last launch's counters, [160 CTAs][16 slots] of uint64, to `host` (synchronises the device).
extern "C" __attribute__((visibility("default"))) int ck_gemm_profile_read(unsigned long long *host) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(host, g_prof, sizeof(g_prof));
    return e == cudaSuccess ? CK_OK : CK_ERR_CUDA;
}
#endif
extern "C" int ck_gemm_cta_pair(void) { return use_cta_pair() ? 1 : 0; }

extern "C" int ck_gemm_sm_budget(void) { return gemm_sms(); }

extern "C" int ck_set_gemm_sm_budget(int sms) {
    const int prev = gemm_sms();
    g_sm_budget = sms > 0 ? sms : 0;
    return prev;
}

extern "C" int ck_set_gemm_cta_pair(int enable) {
    const int prev = use_cta_pair() ? 1 : 0;
    g_cta_pair = enable ? 1 : 0;
    return prev;
}

#define CK_DISPATCH_DTYPE(dtype, CALL)                              \
    switch (dtype) {                                                \
        case CK_BF16: { using T = __nv_bfloat16; return CALL; }     \
        case CK_F16: { using T = __half; return CALL; }             \
        case CK_F32: { using T = float; return CALL; }              \
        default: return CK_ERR_UNSUPPORTED;                         \
    }

extern "C" int ck_moe_up_act_fwd(const void *xg, const void *wfc, const void *b_fc, const void *gate_w, const int32_t *row_map,
                                 const int32_t *mtile_off, void *act, void *h, int E, int64_t cap, int H, int I,
                                 int act_kind, int dtype, int32_t *dev_status, void *stream) {
    if (!xg || !wfc || !row_map || !mtile_off || !act || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (!act_is_known(act_kind)) return CK_ERR_UNSUPPORTED;
    CK_DISPATCH_DTYPE(dtype, (up_act_fwd_t<T>(xg, wfc, b_fc, gate_w, row_map, mtile_off, act, h, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_up_act_fwd_gather(const void *x, int64_t tokens, int top_k, const void *wfc, const void *b_fc, const void *gate_w,
                                        const int32_t *row_map, const int32_t *mtile_off, void *act, void *h, void *xg_out,
                                        int E, int64_t cap, int H, int I, int act_kind, int dtype, int32_t *dev_status,
                                        void *stream) {
    if (!x || tokens <= 0 || top_k <= 0 || !wfc || !row_map || !mtile_off || !act || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (!act_is_known(act_kind)) return CK_ERR_UNSUPPORTED;
    RowSource rs;
    rs.src = x; rs.src_rows = tokens; rs.fan = top_k; rs.rows_out = xg_out;
    CK_DISPATCH_DTYPE(dtype, (up_act_fwd_t<T>(nullptr, wfc, b_fc, gate_w, row_map, mtile_off, act, h, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream, &rs)));
}

extern "C" int ck_moe_up_act_fwd_gather_peer(const void *const *peer_src, int n_peers, int64_t rows_per_peer, int fan_out,
                                             const void *wfc, const void *gate_w, const int32_t *row_map,
                                             const int32_t *mtile_off, void *act, void *h, void *xg_out, int E, int64_t cap,
                                             int H, int I, int act_kind, int dtype, int32_t *dev_status, void *stream) {
    if (!peer_src || n_peers <= 0 || fan_out <= 0 || !wfc || !row_map || !mtile_off || !act || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (!act_is_known(act_kind)) return CK_ERR_UNSUPPORTED;
    RowSource rs;
    rs.peers = peer_src; rs.n_peers = n_peers; rs.rows_per_peer = rows_per_peer; rs.fan = fan_out; rs.rows_out = xg_out;
    CK_DISPATCH_DTYPE(dtype, (up_act_fwd_t<T>(nullptr, wfc, nullptr, gate_w, row_map, mtile_off, act, h, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream, &rs)));
}

extern "C" int ck_moe_down_combine_fwd(const void *act, const void *wproj, const void *b_proj, const void *gate_w,
                                       const int32_t *row_map, const int32_t *mtile_off, float *out32, int E, int64_t cap,
                                       int H, int I, int top_k, int dtype, int32_t *dev_status, void *stream) {
    if (!act || !wproj || !row_map || !mtile_off || !out32 || E <= 0 || E > kMaxSchedExperts || top_k <= 0 || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (down_combine_fwd_t<T>(act, wproj, b_proj, gate_w, row_map, mtile_off, out32, E, cap, H, I, top_k, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_dgrad_down(const void *dyg, const void *wproj, const void *h, const void *gate_w,
                                 const int32_t *row_map, const int32_t *mtile_off, void *dh, float *dgates,
                                 float *dgates_part, int E, int64_t cap, int H, int I, int act_kind, int dtype,
                                 int32_t *dev_status, void *stream) {
    if (!dyg || !wproj || !h || !row_map || !mtile_off || !dh || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (!act_is_known(act_kind)) return CK_ERR_UNSUPPORTED;
    CK_DISPATCH_DTYPE(dtype, (dgrad_down_t<T>(dyg, wproj, h, gate_w, row_map, mtile_off, dh, dgates, dgates_part, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_dgrad_down_gather(const void *dy, int64_t tokens, int top_k, const void *wproj, const void *h,
                                        const void *gate_w, const int32_t *row_map, const int32_t *mtile_off, void *dh,
                                        float *dgates, float *dgates_part, void *dyg_out, int E, int64_t cap, int H, int I,
                                        int act_kind, int dtype, int32_t *dev_status, void *stream) {
    if (!dy || tokens <= 0 || top_k <= 0 || !wproj || !h || !row_map || !mtile_off || !dh || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (!act_is_known(act_kind)) return CK_ERR_UNSUPPORTED;
    RowSource rs;
    rs.src = dy; rs.src_rows = tokens; rs.fan = top_k; rs.rows_out = dyg_out;
    CK_DISPATCH_DTYPE(dtype, (dgrad_down_t<T>(nullptr, wproj, h, gate_w, row_map, mtile_off, dh, dgates, dgates_part, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream, &rs)));
}

extern "C" int ck_moe_dgrad_down_gather_peer(const void *const *peer_src, int n_peers, int64_t rows_per_peer, int fan_out,
                                             const void *wproj, const void *h, const void *gate_w, const int32_t *row_map,
                                             const int32_t *mtile_off, void *dh, float *dgates, float *dgates_part,
                                             void *dyg_out, int E, int64_t cap, int H, int I, int act_kind, int dtype,
                                             int32_t *dev_status, void *stream) {
    if (!peer_src || n_peers <= 0 || fan_out <= 0 || !wproj || !h || !row_map || !mtile_off || !dh || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (!act_is_known(act_kind)) return CK_ERR_UNSUPPORTED;
    RowSource rs;
    rs.peers = peer_src; rs.n_peers = n_peers; rs.rows_per_peer = rows_per_peer; rs.fan = fan_out; rs.rows_out = dyg_out;
    CK_DISPATCH_DTYPE(dtype, (dgrad_down_t<T>(nullptr, wproj, h, gate_w, row_map, mtile_off, dh, dgates, dgates_part, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream, &rs)));
}

extern "C" int ck_moe_dgrad_down_parts(int I) {
    if (I <= 0) return 0;
    const int n_tiles = (I + BN - 1) / BN;
    return use_cta_pair() ? 2 * n_tiles : n_tiles;  // the CTA-pair kernel runs two epilogue groups per n-tile
}

extern "C" int ck_moe_reduce_dgates(const float *dgates_part, int n_parts, int64_t cap, const int32_t *row_map,
                                    const int32_t *padded_off, int E, float *dgates, void *stream) {
    if (!dgates_part || n_parts <= 0 || cap <= 0 || !row_map || !padded_off || E <= 0 || !dgates) return CK_ERR_SHAPE;
    int64_t blocks = ceil_div64(cap, 256);
    const int64_t limit = int64_t(num_sms()) * 8;
    if (blocks > limit) blocks = limit;
    reduce_dgates_kernel<<<unsigned(blocks), 256, 0, (cudaStream_t)stream>>>(dgates_part, n_parts, cap, row_map, padded_off, E, dgates);
    CK_LAUNCH_CHECK("reduce_dgates_kernel");
    return CK_OK;
}

extern "C" int ck_moe_wgrad_gather(const void *a, int64_t a_rows, int a_fan, const void *b, int64_t b_rows, int b_fan,
                                   const int32_t *row_map, const int32_t *padded_off, void *dw, int E, int64_t cap, int M,
                                   int N, int dtype, int32_t *dev_status, void *stream) {
    if (!a || !b || !row_map || !padded_off || !dw || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, M, N)) return CK_ERR_SHAPE;
    if (a_fan < 0 || b_fan < 0 || (a_fan > 0 && a_rows <= 0) || (b_fan > 0 && b_rows <= 0)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (wgrad_t<T>(a, b, padded_off, dw, E, cap, M, N, dev_status, (cudaStream_t)stream, row_map, a_rows, a_fan, b_rows, b_fan)));
}

extern "C" int ck_moe_dgrad_up(const void *dh, const void *wfc, const int32_t *row_map, const int32_t *mtile_off,
                               float *dx32, int E, int64_t cap, int H, int I2, int top_k, int dtype,
                               int32_t *dev_status, void *stream) {
    if (!dh || !wfc || !row_map || !mtile_off || !dx32 || E <= 0 || E > kMaxSchedExperts || top_k <= 0 || !dims_ok(cap, H, I2)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (dgrad_up_t<T>(dh, wfc, row_map, mtile_off, dx32, E, cap, H, I2, top_k, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_wgrad(const void *a, const void *b, const int32_t *padded_off, void *dw, int E, int64_t cap, int M,
                            int N, int dtype, int32_t *dev_status, void *stream) {
    if (!a || !b || !padded_off || !dw || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, M, N)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (wgrad_t<T>(a, b, padded_off, dw, E, cap, M, N, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_grouped_linear(const void *x, const void *w, const int32_t *mtile_off, void *y, int E, int64_t cap,
                                     int N, int K, int trans_w, int dtype, int32_t *dev_status, void *stream) {
    if (!x || !w || !mtile_off || !y || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, N, K)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (grouped_linear_t<T>(x, w, mtile_off, nullptr, y, E, cap, N, K, trans_w, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_grouped_linear_scatter(const void *x, const void *w, const void *bias, const void *gate_w,
                                             const int32_t *mtile_off, const int32_t *row_map, void *y, int E, int64_t cap,
                                             int N, int K, int trans_w, int dtype, int32_t *dev_status, void *stream) {
    if (!x || !w || !mtile_off || !row_map || !y || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, N, K)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (grouped_linear_t<T>(x, w, mtile_off, row_map, y, E, cap, N, K, trans_w, dev_status, (cudaStream_t)stream,
                                                  nullptr, nullptr, 0, 0, bias, gate_w)));
}

extern "C" int ck_router_gate_topk_softmax(const void *x, const void *gate_w, void *logits, void *weights, int32_t *ids,
                                           int64_t tokens, int H, int E, int top_k, int dtype, int32_t *dev_status, void *stream) {
    if (tokens < 0 || H <= 0 || H % 8 != 0 || E <= 0 || E % 8 != 0 || E > BN || top_k <= 0 || top_k > 8 || top_k > E) return CK_ERR_SHAPE;
    if (tokens > INT32_MAX - BM) return CK_ERR_SHAPE;
    if (tokens == 0) return CK_OK;
    if (!x || !gate_w || !logits || !weights || !ids) return CK_ERR_SHAPE;
    if (dtype == CK_F32) return CK_ERR_UNSUPPORTED;  // fp32 logits would come out of a TF32 product: not what top-k should see
    CK_DISPATCH_DTYPE(dtype, (router_gate_t<T>(x, gate_w, logits, weights, ids, tokens, H, E, top_k, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_bias_grad(const void *rows, int64_t cap, int N, const int32_t *row_map, const void *gate_w,
                                const int32_t *padded_off, int E, void *out, int dtype, void *stream) {
    if (!rows || cap <= 0 || N <= 0 || N % 8 != 0 || !padded_off || E <= 0 || !out || (gate_w && !row_map)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (bias_grad_t<T>(rows, cap, N, row_map, gate_w, padded_off, E, out, (cudaStream_t)stream)));
}

extern "C" int ck_moe_bias_dots(const void *rows, int64_t cap, int N, const void *bias, const int32_t *padded_off, int E,
                                float *part, int dtype, void *stream) {
    if (!rows || cap <= 0 || N <= 0 || N % 8 != 0 || !bias || !padded_off || E <= 0 || !part) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (bias_dots_t<T>(rows, cap, N, bias, padded_off, E, part, (cudaStream_t)stream)));
}

extern "C" int ck_moe_grouped_linear_scatter_peer(const void *x, const void *w, const int32_t *mtile_off,
                                                  const int32_t *row_map, const int32_t *dst_flat, void *const *peer_out,
                                                  int n_peers, int64_t rows_per_peer, int E, int64_t cap, int N, int K,
                                                  int trans_w, int dtype, int32_t *dev_status, void *stream) {
    if (!x || !w || !mtile_off || !row_map || !peer_out || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, N, K))
        return CK_ERR_SHAPE;
    if (n_peers <= 0 || n_peers > CK_MAX_PEERS || rows_per_peer <= 0) return CK_ERR_SHAPE;
    if (rows_per_peer > (int64_t(1) << kPeerRowBits) || rows_per_peer * n_peers > INT32_MAX) return CK_ERR_RANGE;
    for (int i = 0; i < n_peers; ++i)
        if (!peer_out[i] || (reinterpret_cast<uintptr_t>(peer_out[i]) & 15)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (grouped_linear_t<T>(x, w, mtile_off, row_map, nullptr, E, cap, N, K, trans_w, dev_status,
                                                  (cudaStream_t)stream, dst_flat, peer_out, n_peers, rows_per_peer)));
}
