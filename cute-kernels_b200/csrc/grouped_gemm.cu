// Grouped GEMMs of the MoE expert path on tcgen05 tensor cores.
//
// One persistent, warp-specialised kernel template covers the five GEMMs of a forward + backward
// pass.  Rows of every activation matrix live in the "padded grouped" layout produced by ck_route:
// the rows routed to expert e occupy [padded_off[e], padded_off[e+1]), a multiple of 128 rows, pad
// rows are zero.  A 128-row tile therefore belongs to exactly one expert and needs no row masks on
// the operand side.
//
//   CTA (192 threads, one per SM, 128x256 output tile, fp32 accumulators in TMEM, double buffered)
//     warp 0     : TMA producer  -- global -> 128B-swizzled shared memory, 4-stage mbarrier ring
//     warp 1     : MMA issuer    -- tcgen05.mma (cta_group::1, M=128, N=256, K=32 bytes per instruction)
//     warps 2..5 : epilogue      -- tcgen05.ld of the finished accumulator + the fused tail:
//                                   activation, SwiGLU backward, router-weight grad, scatter-add
//                                   combine, or a plain store (wgrad / generic grouped linear)
//
// Every mbarrier wait is bounded by wall-clock time; when one runs out the CTA raises
// CK_DEV_TIMEOUT in the caller's status word, lets in-flight copies land, frees TMEM and returns.
#include <cuda.h>
#include <stdlib.h>

#include "ck_common.cuh"
#include "sm100_ptx.cuh"

namespace ck {

enum { MODE_STORE = 0, MODE_UP_ACT = 1, MODE_SCATTER_ADD = 2, MODE_ACT_BWD = 3, MODE_WGRAD = 4 };

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
    const int32_t *mtile_off;   // [E+1] (all modes but WGRAD)
    const int32_t *padded_off;  // [E+1] (WGRAD)
    const int32_t *row_map;     // [cap]
    const void *gate_w;         // router weights, flat [T*k], dtype T (may be NULL)
    const void *h_in;           // ACT_BWD: saved [cap, 2I] pre-activation
    void *out0;                 // STORE/WGRAD: y | UP_ACT: act | ACT_BWD: dh
    void *out1;                 // UP_ACT: h (may be NULL)
    float *out32;               // SCATTER_ADD target [T, N]
    float *dgates;              // ACT_BWD: [T*k] fp32
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
    // STORE with peer destinations (n_peers > 0): row row_map[p] of the result belongs to global slot
    // g = dst_flat ? dst_flat[row_map[p]] : row_map[p] and is
    // stored at peer_out[g / peer_rows] + (g % peer_rows) * N (another GPU's memory over NVLink, or this GPU's own buffer)
    const int32_t *dst_flat;
    int64_t peer_rows;
    int n_peers;
    void *peer_out[CK_MAX_PEERS];
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
    int32_t sched[kMaxSchedExperts + 1];
};

constexpr size_t kGemmSmemBytes_noepi = 1024 /*alignment slack*/ + size_t(kStages) * (kAStageBytes + kBStageBytes) + sizeof(SmemCtl);

// bounded wait: false when the CTA is aborting or the time limit ran out
// BACKOFF: sleep between polls (epilogue warps: 32 polling lanes would otherwise compete for issue slots with the
// producer / MMA lanes that share their scheduler)
template <bool BACKOFF = false>
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, SmemCtl *ctl, int32_t *dev_status) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (BACKOFF) __nanosleep(100);
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (ctl->abort_flag) return false;
            if (ptx::globaltimer_ns() - t0 > kWaitLimitNs) {
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

// ---- fused tail of one 128 x 256 tile: executed by the four epilogue warps of a CTA --------------------
//
// tcgen05.ld hands every thread one accumulator ROW.  Writing rows straight from registers makes each
// warp-wide global access touch 32 different rows (32 LSU wavefronts of 16 bytes): on tiles with a short
// K loop the load/store unit, not the tensor pipe, then sets the pace.  The tail therefore computes in the
// row-per-thread domain and moves data between registers and global memory through a small per-warp
// shared-memory stage, so that every global access is a run of 64 or 128 contiguous bytes of one row.
constexpr int kStagePitchWords = 36;                           // 32 payload words + 4 pad: conflict-free v4 / v2 access
constexpr int kStageWarpBytes = 32 * kStagePitchWords * 4;     // 4608 B per epilogue warp
constexpr int kEpiWarps = 4;
constexpr int kEpiSmemBytes = kEpiWarps * (kStageWarpBytes + 32 * 4);  // stages + per-row info

struct EpiSmem {
    uint32_t *stage;  // [32][kStagePitchWords] words, private to the warp
    int32_t *rowinfo; // [32] per-row index (row_map entry), private to the warp
};

// thread `lane` (owner of tile row `lane` of this warp) writes / reads its WORDS consecutive words
template <int WORDS>
__device__ __forceinline__ void stage_put_row(uint32_t *stage, int lane, const uint32_t *w) {
    uint4 *dst = reinterpret_cast<uint4 *>(stage + lane * kStagePitchWords);
#pragma unroll
    for (int q = 0; q < WORDS / 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
}
template <int WORDS>
__device__ __forceinline__ void stage_get_row(const uint32_t *stage, int lane, uint32_t *w) {
    const uint4 *src = reinterpret_cast<const uint4 *>(stage + lane * kStagePitchWords);
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
template <typename T, typename RowPtr>
__device__ __forceinline__ void stage_write_rows(const uint32_t *stage, int lane, int col0, int ncols, RowPtr row_ptr) {
    using RP = RowPass<T>;
    const int sub = lane % RP::kLpr;
    const int col = col0 + sub * RP::kElemsPerLane;
#pragma unroll
    for (int it = 0; it < RP::kIters; ++it) {
        const int r = RP::row(it, lane);
        const uint2 v = *reinterpret_cast<const uint2 *>(stage + r * kStagePitchWords + 2 * sub);
        T *dst = row_ptr(r);
        if (dst != nullptr && col < ncols) __stcs(reinterpret_cast<uint2 *>(dst + col), v);  // written once: evict-first, keeps the operand panels in L2
    }
}
// global -> rows of the stage (zeros where the row is absent or the columns are out of range)
template <typename T, typename RowPtr>
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
        *reinterpret_cast<uint2 *>(stage + r * kStagePitchWords + 2 * sub) = v;
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
template <typename T>
__device__ __forceinline__ void rows_to_stage(uint32_t *stage, int lane, const uint2 *regs) {
    using RP = RowPass<T>;
    const int sub = lane % RP::kLpr;
#pragma unroll
    for (int it = 0; it < RP::kIters; ++it)
        *reinterpret_cast<uint2 *>(stage + RP::row(it, lane) * kStagePitchWords + 2 * sub) = regs[it];
}

template <typename T, int MODE>
__device__ __forceinline__ void epilogue_tile(const GemmParams &p, const TileCoord &c, uint32_t tbase, int row_in_tile,
                                              const EpiSmem &es) {
    const bool have_acc = c.k_iters > 0;
    const int lane = row_in_tile & 31;
    const int row0 = row_in_tile - lane;  // first tile row of this warp
    using RP = RowPass<T>;

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
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 32) {
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
            uint32_t w[RP::kWords];
            pack32<T>(v, w);
            stage_put_row<RP::kWords>(es.stage, lane, w);
            __syncwarp();
            stage_write_rows<T>(es.stage, lane, n0 + cc, p.N, row_ptr);
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
        for (int cc = 0; cc < BN / 2; cc += 32) {
            uint32_t ru[32], rg[32];
            ptx::tmem_ld32(tbase + cc, ru);
            ptx::tmem_ld32(tbase + BN / 2 + cc, rg);
            ptx::tmem_ld_wait();
            float va[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) va[i] = wgt * act_fwd<T>(p.act_kind, __uint_as_float(ru[i]), __uint_as_float(rg[i]));
            uint32_t w[RP::kWords];
            pack32<T>(va, w);
            stage_put_row<RP::kWords>(es.stage, lane, w);
            __syncwarp();
            stage_write_rows<T>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return act + r * ld_act; });
            __syncwarp();
            if (h) {
                float vf[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) vf[i] = __uint_as_float(ru[i]);
                pack32<T>(vf, w);
                stage_put_row<RP::kWords>(es.stage, lane, w);
                __syncwarp();
                stage_write_rows<T>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return h + r * ld_h; });
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 32; ++i) vf[i] = __uint_as_float(rg[i]);
                pack32<T>(vf, w);
                stage_put_row<RP::kWords>(es.stage, lane, w);
                __syncwarp();
                stage_write_rows<T>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return h + r * ld_h + p.N; });
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
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 32) {
            uint32_t r[32];
            ptx::tmem_ld32(tbase + cc, r);
            ptx::tmem_ld_wait();
            stage_put_row<32>(es.stage, lane, r);
            __syncwarp();
            const int col = n0 + cc + 4 * sub;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int rr = it * 4 + (lane >> 3);
                const int32_t tok = es.rowinfo[rr];
                const float4 v = *reinterpret_cast<const float4 *>(es.stage + rr * kStagePitchWords + 4 * sub);
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
        rows_prefetch<T>(pu, lane, n0, p.N, h_up);
        rows_prefetch<T>(pg, lane, n0, p.N, h_gate);
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 32) {
            if (n0 + cc >= p.N) break;  // whole chunk past the valid columns (uniform across the warp)
            uint32_t w[RP::kWords];
            float vu[32], vg[32];
            rows_to_stage<T>(es.stage, lane, pu);
            __syncwarp();
            stage_get_row<RP::kWords>(es.stage, lane, w);
            unpack32<T>(w, vu);
            __syncwarp();
            rows_to_stage<T>(es.stage, lane, pg);
            __syncwarp();
            stage_get_row<RP::kWords>(es.stage, lane, w);
            unpack32<T>(w, vg);
            __syncwarp();
            if (cc + 32 < BN && n0 + cc + 32 < p.N) {
                rows_prefetch<T>(pu, lane, n0 + cc + 32, p.N, h_up);
                rows_prefetch<T>(pg, lane, n0 + cc + 32, p.N, h_gate);
            }
            uint32_t r[32];
            ptx::tmem_ld32(tbase + cc, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float acc = __uint_as_float(r[i]);
                float a, du_m, dg_m;
                act_bwd<T>(p.act_kind, vu[i], vg[i], a, du_m, dg_m);
                dgate_w += a * acc;
                const float da = wgt * acc;
                vu[i] = da * du_m;
                vg[i] = da * dg_m;
            }
            pack32<T>(vu, w);
            stage_put_row<RP::kWords>(es.stage, lane, w);
            __syncwarp();
            stage_write_rows<T>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return dh + r * ld_h; });
            __syncwarp();
            pack32<T>(vg, w);
            stage_put_row<RP::kWords>(es.stage, lane, w);
            __syncwarp();
            stage_write_rows<T>(es.stage, lane, n0 + cc, p.N, [&](int r) -> T * { return dh + r * ld_h + p.N; });
            __syncwarp();
        }
        if (p.dgates && src >= 0) atomicAdd(p.dgates + src, dgate_w);
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
        for (int i = threadIdx.x; i <= p.E; i += kGemmThreads) ctl->sched[i] = src[i];
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
        } else if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                const TileCoord c = decode_tile<MODE, BK>(p, ctl, t);
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    if (!wait_barrier(ptx::smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.dev_status)) { ok = false; break; }
                    const uint32_t full = ptx::smem_u32(&ctl->full[stage]);
                    ptx::mbar_expect_tx(full, kAStageBytes + kBStageBytes);
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBStageBytes;
                    if constexpr (MODE == MODE_WGRAD) {
                        const int krow = c.k_row0 + kb * BK;
#pragma unroll
                        for (int j = 0; j < BM / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d(sa + j * TR::kMnBoxBytes, &p.tmA, full, c.m_tile * BM + j * TR::kMnBoxElems, krow);
#pragma unroll
                        for (int j = 0; j < BN / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d(sb + j * TR::kMnBoxBytes, &p.tmB, full, c.n_tile * BN + j * TR::kMnBoxElems, krow);
                    } else {
                        const int k0 = kb * BK;
                        ptx::tma_load_2d(sa, &p.tmA, full, k0, c.m_tile * BM);
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
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
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
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++it) {
                const TileCoord c = decode_tile<MODE, BK>(p, ctl, t);
                const int buf = it & 1;
                if (!wait_barrier(ptx::smem_u32(&ctl->tmem_empty[buf]), ((uint32_t(it) >> 1) & 1u) ^ 1u, ctl, p.dev_status)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(buf) * BN;
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    if (!wait_barrier(ptx::smem_u32(&ctl->full[stage]), phase, ctl, p.dev_status)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBStageBytes;
#pragma unroll
                    for (int k = 0; k < TR::kSteps; ++k) {
                        uint64_t adesc, bdesc;
                        if constexpr (A_MN) adesc = ptx::umma_desc_mnmajor<TR::kTf32>(sa + k * TR::UMMA_K * kRowBytes, TR::kMnBoxBytes);
                        else adesc = ptx::umma_desc_kmajor(sa + k * 32);
                        if constexpr (B_MN) bdesc = ptx::umma_desc_mnmajor<TR::kTf32>(sb + k * TR::UMMA_K * kRowBytes, TR::kMnBoxBytes);
                        else bdesc = ptx::umma_desc_kmajor(sb + k * 32);
                        ptx::umma_ss<TR::kTf32>(d_tmem, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(ptx::smem_u32(&ctl->empty[stage]));  // frees the stage when these MMAs retire
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit(ptx::smem_u32(&ctl->tmem_full[buf]));  // accumulator complete
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
            epilogue_tile<T, MODE>(p, c, tbase, row_in_tile, es);
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
#ifndef CK_PAIR_STAGES
#define CK_PAIR_STAGES 6
#endif
constexpr int kPairStages = CK_PAIR_STAGES;
constexpr int kBHalfStageBytes = kBStageBytes / 2;  // 16 KiB

struct SmemCtlPair {
    uint64_t full[kPairStages];
    uint64_t empty[kPairStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_ptr;
    volatile int abort_flag;
    int32_t sched[kMaxSchedExperts + 1];   // m-tile offsets (or padded row offsets for WGRAD)
    int32_t psched[kMaxSchedExperts + 1];  // pair-tile offsets per expert
};

constexpr size_t kGemmPairSmemBytes = 1024 + size_t(kPairStages) * (kAStageBytes + kBHalfStageBytes) + sizeof(SmemCtlPair) + kEpiSmemBytes;

template <int MODE, int BK>
__device__ __forceinline__ TileCoord decode_pair_tile(const GemmParams &p, const SmemCtlPair *ctl, int t, int rank) {
    TileCoord c;
    if constexpr (MODE == MODE_WGRAD) {
        const int mpairs = (p.m_tiles_w + 1) >> 1;
        const int per_e = mpairs * p.n_tiles;
        c.e = t / per_e;
        const int local = t - c.e * per_e;
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

// BACKOFF: sleep between polls (epilogue warps: 32 polling lanes would otherwise compete for issue slots with the
// producer / MMA lanes that share their scheduler)
template <bool BACKOFF = false>
__device__ __forceinline__ bool wait_barrier_pair(uint32_t bar, uint32_t parity, SmemCtlPair *ctl, int32_t *dev_status) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (BACKOFF) __nanosleep(100);
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (ctl->abort_flag) return false;
            if (ptx::globaltimer_ns() - t0 > kWaitLimitNs) {
                ctl->abort_flag = 1;
                if (dev_status) atomicOr(dev_status, CK_DEV_TIMEOUT);
                return false;
            }
        }
    }
}

template <typename T, int MODE, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    grouped_gemm_pair_kernel(const __grid_constant__ GemmParams p) {
    using TR = GemmTraits<T>;
    constexpr bool A_MN = (MODE == MODE_WGRAD);
    constexpr int BK = TR::BK;
    constexpr uint32_t kIdesc = make_idesc<T>(A_MN, B_MN, 2 * BM);
    constexpr uint32_t kStageTx = 2 * (kAStageBytes + kBHalfStageBytes);  // both CTAs' bytes land on the leader's barrier

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_u32 & 1023u)) & 1023u;
    uint8_t *smem = smem_raw + pad;
    const uint32_t smem_a = raw_u32 + pad;
    const uint32_t smem_b = smem_a + kPairStages * kAStageBytes;
    SmemCtlPair *ctl = reinterpret_cast<SmemCtlPair *>(smem + kPairStages * (kAStageBytes + kBHalfStageBytes));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rank = int(ptx::cluster_ctarank());  // 0 = leader
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&ctl->tmem_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&ctl->tmem_empty[b]), 8);  // 4 epilogue warps of each CTA
        }
        ctl->abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&p.tmA);
        ptx::prefetch_tensormap(&p.tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(&ctl->tmem_ptr), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    {
        const int32_t *src = (MODE == MODE_WGRAD) ? p.padded_off : p.mtile_off;
        for (int i = threadIdx.x; i <= p.E; i += kGemmThreads) ctl->sched[i] = src[i];
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

    if (warp == 0) {
        // ================= TMA producer (one per CTA: own A rows, own half of B) =================
        const bool gather_a = p.gather_fan > 0;
        const bool gather_b = (MODE == MODE_WGRAD) && p.gather_b_fan > 0;
        if (gather_a || gather_b) {
            int stage = 0;
            uint32_t phase = 0;
            int ok = 1;
            for (int t = pair_id; t < ntiles && ok; t += num_pairs) {
                const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, rank);
                int ridx[4] = {0, 0, 0, 0};
                if (MODE != MODE_WGRAD && gather_a) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int32_t src = p.row_map[int64_t(c.m_tile) * BM + 4 * lane + q];
                        ridx[q] = src >= 0 ? src / p.gather_fan : 0;
                    }
                }
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    if (lane == 0) {
                        ok = wait_barrier_pair(ptx::smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.dev_status) ? 1 : 0;
                        if (ok && rank == 0) ptx::mbar_expect_tx(ptx::smem_u32(&ctl->full[stage]), kStageTx);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    const uint32_t full = ptx::mapa_shared(ptx::smem_u32(&ctl->full[stage]), 0);  // the leader's barrier
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBHalfStageBytes;
                    const int nb0 = c.n_tile * BN + rank * (BN / 2);  // this CTA's half of the N range
                    if constexpr (MODE == MODE_WGRAD) {
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
                    } else {
                        const int k0 = kb * BK;
                        if (gather_a) ptx::tma_gather4_pair(sa + lane * 512, &p.tmA, full, k0, ridx[0], ridx[1], ridx[2], ridx[3]);
                        else if (lane == 0) ptx::tma_load_2d_pair(sa, &p.tmA, full, k0, c.m_tile * BM);
                        if (lane == 0) {
                            if constexpr (B_MN) {
#pragma unroll
                                for (int j = 0; j < (BN / 2) / TR::kMnBoxElems; ++j)
                                    ptx::tma_load_3d_pair(sb + j * TR::kMnBoxBytes, &p.tmB, full, nb0 + j * TR::kMnBoxElems, k0, c.e);
                            } else if constexpr (MODE == MODE_UP_ACT) {
                                // leader: 128 rows of W_up, peer: the matching 128 rows of W_gate
                                ptx::tma_load_3d_pair(sb, &p.tmB, full, k0, rank * p.N + c.n_tile * (BN / 2), c.e);
                            } else {
                                ptx::tma_load_3d_pair(sb, &p.tmB, full, k0, nb0, c.e);
                            }
                        }
                    }
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok && lane == 0) {
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        } else if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint64_t pol_a = ptx::l2_policy(p.l2_hint_a), pol_b = ptx::l2_policy(p.l2_hint_b);
            for (int t = pair_id; t < ntiles && ok; t += num_pairs) {
                const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, rank);
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    if (!wait_barrier_pair(ptx::smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.dev_status)) { ok = false; break; }
                    if (rank == 0) ptx::mbar_expect_tx(ptx::smem_u32(&ctl->full[stage]), kStageTx);
                    const uint32_t full = ptx::mapa_shared(ptx::smem_u32(&ctl->full[stage]), 0);  // the leader's barrier
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBHalfStageBytes;
                    const int nb0 = c.n_tile * BN + rank * (BN / 2);  // this CTA's half of the N range
                    if constexpr (MODE == MODE_WGRAD) {
                        const int krow = c.k_row0 + kb * BK;
#pragma unroll
                        for (int j = 0; j < BM / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d_pair_hint(sa + j * TR::kMnBoxBytes, &p.tmA, full, c.m_tile * BM + j * TR::kMnBoxElems, krow, pol_a);
#pragma unroll
                        for (int j = 0; j < (BN / 2) / TR::kMnBoxElems; ++j)
                            ptx::tma_load_2d_pair_hint(sb + j * TR::kMnBoxBytes, &p.tmB, full, nb0 + j * TR::kMnBoxElems, krow, pol_b);
                    } else {
                        const int k0 = kb * BK;
                        ptx::tma_load_2d_pair_hint(sa, &p.tmA, full, k0, c.m_tile * BM, pol_a);
                        if constexpr (B_MN) {
#pragma unroll
                            for (int j = 0; j < (BN / 2) / TR::kMnBoxElems; ++j)
                                ptx::tma_load_3d_pair_hint(sb + j * TR::kMnBoxBytes, &p.tmB, full, nb0 + j * TR::kMnBoxElems, k0, c.e, pol_b);
                        } else if constexpr (MODE == MODE_UP_ACT) {
                            // leader: 128 rows of W_up, peer: the matching 128 rows of W_gate
                            ptx::tma_load_3d_pair_hint(sb, &p.tmB, full, k0, rank * p.N + c.n_tile * (BN / 2), c.e, pol_b);
                        } else {
                            ptx::tma_load_3d_pair_hint(sb, &p.tmB, full, k0, nb0, c.e, pol_b);
                        }
                    }
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ================= MMA issuer: the leader CTA drives both tensor cores =================
        if (lane == 0 && rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int t = pair_id; t < ntiles && ok; t += num_pairs, ++it) {
                const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, 0);
                const int buf = it & 1;
                if (!wait_barrier_pair(ptx::smem_u32(&ctl->tmem_empty[buf]), ((uint32_t(it) >> 1) & 1u) ^ 1u, ctl, p.dev_status)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(buf) * BN;
                for (int kb = 0; kb < c.k_iters; ++kb) {
                    if (!wait_barrier_pair(ptx::smem_u32(&ctl->full[stage]), phase, ctl, p.dev_status)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t sa = smem_a + stage * kAStageBytes;
                    const uint32_t sb = smem_b + stage * kBHalfStageBytes;
#pragma unroll
                    for (int k = 0; k < TR::kSteps; ++k) {
                        uint64_t adesc, bdesc;
                        if constexpr (A_MN) adesc = ptx::umma_desc_mnmajor<TR::kTf32>(sa + k * TR::UMMA_K * kRowBytes, TR::kMnBoxBytes);
                        else adesc = ptx::umma_desc_kmajor(sa + k * 32);
                        if constexpr (B_MN) bdesc = ptx::umma_desc_mnmajor<TR::kTf32>(sb + k * TR::UMMA_K * kRowBytes, TR::kMnBoxBytes);
                        else bdesc = ptx::umma_desc_kmajor(sb + k * 32);
                        ptx::umma_ss_pair<TR::kTf32>(d_tmem, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit_pair(ptx::smem_u32(&ctl->empty[stage]), 3);  // frees the stage in both CTAs
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit_pair(ptx::smem_u32(&ctl->tmem_full[buf]), 3);  // accumulators of both CTAs complete
            }
            if (!ok) {
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        }
        __syncwarp();
    } else {
        // ================= epilogue: each CTA drains its own 128 rows =================
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        uint8_t *epi_base = reinterpret_cast<uint8_t *>(ctl) + ((sizeof(SmemCtlPair) + 15) & ~size_t(15));
        EpiSmem es;
        es.stage = reinterpret_cast<uint32_t *>(epi_base + quarter * kStageWarpBytes);
        es.rowinfo = reinterpret_cast<int32_t *>(epi_base + kEpiWarps * kStageWarpBytes + quarter * 128);
        const uint32_t leader_empty0 = ptx::mapa_shared(ptx::smem_u32(&ctl->tmem_empty[0]), 0);
        const uint32_t leader_empty1 = ptx::mapa_shared(ptx::smem_u32(&ctl->tmem_empty[1]), 0);
        int it = 0;
        bool ok = true;
        for (int t = pair_id; t < ntiles && ok; t += num_pairs, ++it) {
            const TileCoord c = decode_pair_tile<MODE, BK>(p, ctl, t, rank);
            const int buf = it & 1;
            if (!wait_barrier_pair<true>(ptx::smem_u32(&ctl->tmem_full[buf]), (uint32_t(it) >> 1) & 1u, ctl, p.dev_status)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t tbase = tmem_base + uint32_t(buf) * BN + (uint32_t(quarter * 32) << 16);
            if (c.valid) epilogue_tile<T, MODE>(p, c, tbase, row_in_tile, es);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(buf ? leader_empty1 : leader_empty0);
        }
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
        set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
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
        CK_CUDA_TRY(cudaFuncSetAttribute(kern2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmPairSmemBytes));
        int64_t pairs = num_sms() / 2;
        if (pairs > max_tiles) pairs = max_tiles;  // upper bound: a pair tile covers at least one single tile
        if (pairs < 1) return CK_OK;
        kern2<<<dim3((unsigned)(2 * pairs)), kGemmThreads, kGemmPairSmemBytes, stream>>>(p);
        CK_LAUNCH_CHECK("grouped_gemm_pair_kernel");
        return CK_OK;
    }
    auto kern = grouped_gemm_kernel<T, MODE, B_MN>;
    CK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmemBytes));
    int64_t grid = num_sms();
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

template <typename T>
static int up_act_fwd_t(const void *xg, const void *wfc, const void *gate_w, const int32_t *row_map,
                        const int32_t *mtile_off, void *act, void *h, int E, int64_t cap, int H, int I, int act_kind,
                        int32_t *dev_status, cudaStream_t stream, int64_t gather_rows = 0, int gather_fan = 0) {
    GemmParams p = {};
    p.cap = cap;
    int rc;
    if (gather_fan > 0) {
        if ((rc = map_a_gather<T>(&p.tmA, xg, gather_rows, H)) != CK_OK) return rc;
        p.gather_fan = gather_fan;
    } else if ((rc = map_a_kmajor<T>(&p.tmA, xg, cap, H)) != CK_OK) return rc;
    if ((rc = map_w_kmajor<T>(&p.tmB, wfc, E, 2 * I, H, BN / 2)) != CK_OK) return rc;
    p.mtile_off = mtile_off; p.row_map = row_map; p.gate_w = gate_w; p.out0 = act; p.out1 = h; p.dev_status = dev_status;
    p.E = E; p.n_tiles = (I + BN / 2 - 1) / (BN / 2); p.N = I; p.K = H; p.act_kind = act_kind; p.top_k = 1;
    return launch_gemm<T, MODE_UP_ACT, false>(p, (cap / BM) * p.n_tiles, stream);
}

template <typename T>
static int down_combine_fwd_t(const void *act, const void *wproj, const int32_t *row_map, const int32_t *mtile_off,
                              float *out32, int E, int64_t cap, int H, int I, int top_k, int32_t *dev_status,
                              cudaStream_t stream) {
    GemmParams p = {};
    p.cap = cap;
    int rc;
    if ((rc = map_a_kmajor<T>(&p.tmA, act, cap, I)) != CK_OK) return rc;
    if ((rc = map_w_kmajor<T>(&p.tmB, wproj, E, H, I, use_cta_pair() ? BN / 2 : BN)) != CK_OK) return rc;
    p.mtile_off = mtile_off; p.row_map = row_map; p.out32 = out32; p.dev_status = dev_status;
    p.E = E; p.n_tiles = (H + BN - 1) / BN; p.N = H; p.K = I; p.top_k = top_k;
    return launch_gemm<T, MODE_SCATTER_ADD, false>(p, (cap / BM) * p.n_tiles, stream);
}

template <typename T>
static int dgrad_down_t(const void *dyg, const void *wproj, const void *h, const void *gate_w, const int32_t *row_map,
                        const int32_t *mtile_off, void *dh, float *dgates, int E, int64_t cap, int H, int I, int act_kind,
                        int32_t *dev_status, cudaStream_t stream, int64_t gather_rows = 0, int gather_fan = 0) {
    GemmParams p = {};
    p.cap = cap;
    int rc;
    if (gather_fan > 0) {
        if ((rc = map_a_gather<T>(&p.tmA, dyg, gather_rows, H)) != CK_OK) return rc;
        p.gather_fan = gather_fan;
    } else if ((rc = map_a_kmajor<T>(&p.tmA, dyg, cap, H)) != CK_OK) return rc;
    if ((rc = map_w_mnmajor<T>(&p.tmB, wproj, E, H, I)) != CK_OK) return rc;
    p.mtile_off = mtile_off; p.row_map = row_map; p.gate_w = gate_w; p.h_in = h; p.out0 = dh; p.dgates = dgates;
    p.dev_status = dev_status;
    p.E = E; p.n_tiles = (I + BN - 1) / BN; p.N = I; p.K = H; p.act_kind = act_kind; p.top_k = 1;
    return launch_gemm<T, MODE_ACT_BWD, true>(p, (cap / BM) * p.n_tiles, stream);
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
                            int64_t peer_rows = 0) {
    GemmParams p = {};
    p.cap = cap;
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

}  // namespace ck

using namespace ck;

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

extern "C" int ck_moe_up_act_fwd(const void *xg, const void *wfc, const void *gate_w, const int32_t *row_map,
                                 const int32_t *mtile_off, void *act, void *h, int E, int64_t cap, int H, int I,
                                 int act_kind, int dtype, int32_t *dev_status, void *stream) {
    if (!xg || !wfc || !row_map || !mtile_off || !act || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (act_kind != CK_ACT_SWIGLU && act_kind != CK_ACT_GLU) return CK_ERR_UNSUPPORTED;
    CK_DISPATCH_DTYPE(dtype, (up_act_fwd_t<T>(xg, wfc, gate_w, row_map, mtile_off, act, h, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_up_act_fwd_gather(const void *x, int64_t tokens, int top_k, const void *wfc, const void *gate_w,
                                        const int32_t *row_map, const int32_t *mtile_off, void *act, void *h, int E,
                                        int64_t cap, int H, int I, int act_kind, int dtype, int32_t *dev_status,
                                        void *stream) {
    if (!x || tokens <= 0 || top_k <= 0 || !wfc || !row_map || !mtile_off || !act || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (act_kind != CK_ACT_SWIGLU && act_kind != CK_ACT_GLU) return CK_ERR_UNSUPPORTED;
    CK_DISPATCH_DTYPE(dtype, (up_act_fwd_t<T>(x, wfc, gate_w, row_map, mtile_off, act, h, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream, tokens, top_k)));
}

extern "C" int ck_moe_down_combine_fwd(const void *act, const void *wproj, const int32_t *row_map,
                                       const int32_t *mtile_off, float *out32, int E, int64_t cap, int H, int I,
                                       int top_k, int dtype, int32_t *dev_status, void *stream) {
    if (!act || !wproj || !row_map || !mtile_off || !out32 || E <= 0 || E > kMaxSchedExperts || top_k <= 0 || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (down_combine_fwd_t<T>(act, wproj, row_map, mtile_off, out32, E, cap, H, I, top_k, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_dgrad_down(const void *dyg, const void *wproj, const void *h, const void *gate_w,
                                 const int32_t *row_map, const int32_t *mtile_off, void *dh, float *dgates, int E,
                                 int64_t cap, int H, int I, int act_kind, int dtype, int32_t *dev_status, void *stream) {
    if (!dyg || !wproj || !h || !row_map || !mtile_off || !dh || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (act_kind != CK_ACT_SWIGLU && act_kind != CK_ACT_GLU) return CK_ERR_UNSUPPORTED;
    CK_DISPATCH_DTYPE(dtype, (dgrad_down_t<T>(dyg, wproj, h, gate_w, row_map, mtile_off, dh, dgates, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream)));
}

extern "C" int ck_moe_dgrad_down_gather(const void *dy, int64_t tokens, int top_k, const void *wproj, const void *h,
                                        const void *gate_w, const int32_t *row_map, const int32_t *mtile_off, void *dh,
                                        float *dgates, int E, int64_t cap, int H, int I, int act_kind, int dtype,
                                        int32_t *dev_status, void *stream) {
    if (!dy || tokens <= 0 || top_k <= 0 || !wproj || !h || !row_map || !mtile_off || !dh || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, H, I)) return CK_ERR_SHAPE;
    if (act_kind != CK_ACT_SWIGLU && act_kind != CK_ACT_GLU) return CK_ERR_UNSUPPORTED;
    CK_DISPATCH_DTYPE(dtype, (dgrad_down_t<T>(dy, wproj, h, gate_w, row_map, mtile_off, dh, dgates, E, cap, H, I, act_kind, dev_status, (cudaStream_t)stream, tokens, top_k)));
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

extern "C" int ck_moe_grouped_linear_scatter(const void *x, const void *w, const int32_t *mtile_off, const int32_t *row_map,
                                             void *y, int E, int64_t cap, int N, int K, int trans_w, int dtype,
                                             int32_t *dev_status, void *stream) {
    if (!x || !w || !mtile_off || !row_map || !y || E <= 0 || E > kMaxSchedExperts || !dims_ok(cap, N, K)) return CK_ERR_SHAPE;
    CK_DISPATCH_DTYPE(dtype, (grouped_linear_t<T>(x, w, mtile_off, row_map, y, E, cap, N, K, trans_w, dev_status, (cudaStream_t)stream)));
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
