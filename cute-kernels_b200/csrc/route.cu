// Routing kernels: continuous_count (histogram) and route (count + scan + stable scatter).
//
// Both are HBM-bound integer passes over the expert ids.  The histogram aggregates equal ids
// inside a warp with __match_any_sync / __popc so that a skewed (Zipf) id distribution costs one
// shared-memory update per distinct id per warp step instead of one contended atomic per element.
// The stable scatter gives every warp a contiguous slice of the ids; a slice's position in the
// output is (exclusive scan over experts) + (exclusive scan over earlier warps for that expert) +
// (running count inside the warp), which is exactly the order torch.sort(stable=True) produces.
#include <algorithm>
#include <mutex>
#include <type_traits>

#include "ck_common.cuh"

namespace ck {

constexpr int kRouteMaxSlices = 148 * 4;  // upper bound on id slices, one per thread block (fixed so workspace size is device independent)
constexpr int kRouteWarpsPerBlock = 8;
constexpr int kHistWarpsPerBlock = 4;  // histogram pass: 33 KiB of private histograms per block at 64 experts, so that all 592
                                       // slices are resident at once (8 warps: 3 blocks per SM, a second wave a third full)
constexpr int kLoads = 16;          // coalesced 32-id loads in flight per warp: 2 KiB (int32) of reads per warp step
constexpr int kStep = 32 * kLoads;  // ids per warp per unrolled step

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Peer mask of the lanes holding the same key, built from one ballot per key bit.  __match_any_sync
// gives the same mask but its cost grows with the number of distinct keys in the warp (about 26 of 32
// lanes differ for uniform ids over 64 experts); log2(range) ballots cost the same for every input.
// Lanes with key < 0 (out of range / past the end) get 0.
__device__ __forceinline__ unsigned match_key_bits(int key, int nbits) {
    unsigned m = __ballot_sync(0xffffffffu, key >= 0);
    for (int b = 0; b < nbits; ++b) {
        const bool bit = (key >> b) & 1;
        const unsigned bal = __ballot_sync(0xffffffffu, bit);
        m &= bit ? bal : ~bal;
    }
    return key >= 0 ? m : 0u;
}

template <int NBITS>
__device__ __forceinline__ unsigned match_key_fixed(int key) {
    unsigned m = __ballot_sync(0xffffffffu, key >= 0);
#pragma unroll
    for (int b = 0; b < NBITS; ++b) {
        const bool bit = (key >> b) & 1;
        const unsigned bal = __ballot_sync(0xffffffffu, bit);
        m &= bit ? bal : ~bal;
    }
    return key >= 0 ? m : 0u;
}

template <typename IdT>
__device__ __forceinline__ int load_key(const IdT *__restrict__ ids, int64_t idx, int64_t end, int range, bool &bad) {
    if (idx >= end) return -1;
    const IdT v = ids[idx];
    using U = typename std::make_unsigned<IdT>::type;
    if (U(v) < U(range)) return int(v);
    bad = true;
    return -1;
}

// One warp step: kLoads coalesced 32-id loads.  FULL = the whole step lies inside the range, no bounds checks.
// `p` already points at (step start + lane); ids outside [0, range) become -1 and set `bad`.
template <typename IdT, bool FULL>
__device__ __forceinline__ void load_step(const IdT *__restrict__ p, int remaining, int lane, int range, int (&key)[kLoads], bool &bad) {
    using U = typename std::make_unsigned<IdT>::type;
    IdT v[kLoads];
#pragma unroll
    for (int j = 0; j < kLoads; ++j) {
        if (FULL || 32 * j + lane < remaining) v[j] = p[32 * j];
        else v[j] = IdT(0);
    }
#pragma unroll
    for (int j = 0; j < kLoads; ++j) {
        const bool in = FULL || 32 * j + lane < remaining;
        const bool ok = U(v[j]) < U(range);
        key[j] = (in && ok) ? int(v[j]) : -1;
        bad |= in && !ok;
    }
}

// Whole step inside the range, ids mapped to [0, range]: `range` itself stands for "out of range" and indexes a spare
// histogram row, so the counting loop needs neither a predicate nor a flag per id.
template <typename IdT>
__device__ __forceinline__ void load_step_clamped(const IdT *__restrict__ p, int range, int (&key)[kLoads]) {
    using U = typename std::make_unsigned<IdT>::type;
    IdT v[kLoads];
#pragma unroll
    for (int j = 0; j < kLoads; ++j) v[j] = p[32 * j];
#pragma unroll
    for (int j = 0; j < kLoads; ++j) key[j] = int(min(U(v[j]), U(range)));
}

constexpr int kLanePrivateMax = 128;  // largest id range that gets a per-lane histogram (16 KiB per warp)

// ------------------------------------------------------------------------------------------------
// continuous_count: counts[v] += #ids == v.  counts is zeroed by the host wrapper beforehand.
// Small ranges (the MoE case) count into per-lane histograms laid out [value][lane]: bank == lane, so
// the read-modify-write needs neither atomics nor conflict replays; larger ranges aggregate equal ids in
// the warp first and issue one shared-memory atomic per distinct id.
// ------------------------------------------------------------------------------------------------
template <typename IdT, bool LANE_PRIVATE>
__global__ void __launch_bounds__(512) count_kernel(const IdT *__restrict__ ids, int64_t n, int size, int nbits,
                                                   uint32_t *__restrict__ counts) {
    extern __shared__ uint32_t hist[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int64_t warp_id = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const int64_t nchunks = (n + kStep - 1) / kStep;
    bool bad = false;

    if constexpr (LANE_PRIVATE) {
        const int wpb = blockDim.x >> 5;
        uint32_t *wh = hist + wib * (size + 1) * 32;  // [size + 1][32] per warp; the last row collects out-of-range ids
        uint32_t *bh = hist + wpb * (size + 1) * 32;  // [size] block totals
        for (int i = lane; i < (size + 1) * 32; i += 32) wh[i] = 0;
        for (int i = threadIdx.x; i < size; i += blockDim.x) bh[i] = 0;
        __syncthreads();
        uint32_t *mine = wh + lane;
        // two steps in flight per warp: the loads of step c + nwarps are issued before step c is counted
        int cur[kLoads], nxt[kLoads];
        auto fetch = [&](int64_t c, int (&key)[kLoads]) {
            const int64_t b = c * kStep;
            if (b + kStep <= n) {
                load_step_clamped<IdT>(ids + b + lane, size, key);
            } else {  // the ragged last step: positions past the end go to the spare row too
                load_step<IdT, false>(ids + b + lane, int(n - b), lane, size, key, bad);
#pragma unroll
                for (int j = 0; j < kLoads; ++j) key[j] = key[j] < 0 ? size : key[j];
            }
        };
        if (warp_id < nchunks) fetch(warp_id, cur);
        for (int64_t c = warp_id; c < nchunks; c += nwarps) {
            const bool more = c + nwarps < nchunks;
            if (more) fetch(c + nwarps, nxt);
#pragma unroll
            for (int j = 0; j < kLoads; ++j) atomicAdd(mine + cur[j] * 32, 1u);  // private slot: a fire-and-forget shared-memory add
            if (more) {
#pragma unroll
                for (int j = 0; j < kLoads; ++j) cur[j] = nxt[j];
            }
        }
        __syncwarp();
        // lanes -> warp -> block -> one global atomic per value per block (same-sector atomics serialise in L2,
        // so the number of global atomics, not the histogram itself, would otherwise set the run time)
        // lane l sums the 32 private slots of values l, l + 32, ...; the rotated slot order keeps the 32 lanes on 32 banks
        for (int v = lane; v < size; v += 32) {
            uint32_t c = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) c += wh[v * 32 + ((lane + j) & 31)];
            if (c) atomicAdd(&bh[v], c);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < size; i += blockDim.x) {
            const int v = (i + blockIdx.x * 8) % size;  // blocks start on different 32-byte sectors
            const uint32_t c = bh[v];
            if (c) atomicAdd(&counts[v], c);
        }
    } else {
        for (int i = threadIdx.x; i < size; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int64_t c = warp_id; c < nchunks; c += nwarps) {
            const int64_t b = c * kStep + lane;
            int key[kLoads];
#pragma unroll
            for (int j = 0; j < kLoads; ++j) key[j] = load_key(ids, b + 32 * j, n, size, bad);
#pragma unroll
            for (int j = 0; j < kLoads; ++j) {
                const unsigned m = match_key_bits(key[j], nbits);
                if (key[j] >= 0 && lane == __ffs(m) - 1) atomicAdd(&hist[key[j]], __popc(m));
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < size; i += blockDim.x) {
            const uint32_t v = hist[i];
            if (v) atomicAdd(&counts[i], v);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// route pass 1: per-warp histogram of a contiguous slice of ids -> whist[w][E]
// ------------------------------------------------------------------------------------------------
template <typename IdT, bool LANE_PRIVATE>
__global__ void __launch_bounds__(kHistWarpsPerBlock * 32)
    route_hist_kernel(const IdT *__restrict__ ids, int64_t n, int E, int64_t slice, int32_t *__restrict__ whist,
                      int32_t *dev_status) {
    // one thread block per slice; its warps take the 512-id steps of the slice round-robin
    extern __shared__ int32_t smem_i[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int64_t begin = int64_t(blockIdx.x) * slice;
    const int len = int(min(begin + slice, n) - begin);
    const IdT *__restrict__ my_ids = ids + begin + lane;
    int32_t *bh = smem_i;  // [E] block histogram
    for (int e = threadIdx.x; e < E; e += blockDim.x) bh[e] = 0;
    bool bad = false;

    if constexpr (LANE_PRIVATE) {
        int32_t *wh = smem_i + E + wib * (E + 1) * 32;  // [E + 1][32] per warp, bank == lane; row E collects what is not counted
        for (int i = lane; i < (E + 1) * 32; i += 32) wh[i] = 0;
        __syncthreads();
        int32_t *mine = wh + lane;
        constexpr int kStride = kHistWarpsPerBlock * kStep;
        int cur[kLoads], nxt[kLoads];
        int spare_ok = 0;  // entries this lane sent to row E that are not range errors (positions past the slice end)
        auto fetch = [&](int off, int (&key)[kLoads]) {
            if (off + kStep <= len) {
                load_step_clamped<IdT>(my_ids + off, E, key);  // range errors land in row E and are found there afterwards
            } else {
                load_step<IdT, false>(my_ids + off, len - off, lane, E, key, bad);  // flags its own range errors
#pragma unroll
                for (int j = 0; j < kLoads; ++j) {
                    spare_ok += key[j] < 0;
                    key[j] = key[j] < 0 ? E : key[j];
                }
            }
        };
        if (wib * kStep < len) fetch(wib * kStep, cur);
        for (int off = wib * kStep; off < len; off += kStride) {  // next step's loads fly while this one is counted
            const bool more = off + kStride < len;
            if (more) fetch(off + kStride, nxt);
#pragma unroll
            for (int j = 0; j < kLoads; ++j) atomicAdd(mine + cur[j] * 32, 1);  // private slot, no dependency chain
            if (more) {
#pragma unroll
                for (int j = 0; j < kLoads; ++j) cur[j] = nxt[j];
            }
        }
        __syncwarp();
        bad |= mine[E * 32] != spare_ok;
        // lane l sums the 32 private slots of experts l, l + 32, ...; the rotated slot order keeps the 32 lanes on 32 banks
        for (int e = lane; e < E; e += 32) {
            int c = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) c += wh[e * 32 + ((lane + j) & 31)];
            if (c) atomicAdd(&bh[e], c);
        }
    } else {
        __syncthreads();
        for (int off = wib * kStep; off < len; off += kHistWarpsPerBlock * kStep) {
            int key[kLoads];
            if (off + kStep <= len) load_step<IdT, true>(my_ids + off, kStep, lane, E, key, bad);
            else load_step<IdT, false>(my_ids + off, len - off, lane, E, key, bad);
#pragma unroll
            for (int j = 0; j < kLoads; ++j)
                if (key[j] >= 0) atomicAdd(&bh[key[j]], 1);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) whist[int64_t(blockIdx.x) * E + e] = bh[e];
    if (__any_sync(0xffffffffu, bad) && lane == 0 && dev_status) atomicOr(dev_status, CK_DEV_RANGE);
}

// block-wide exclusive scan of one int per thread (blockDim.x == 1024); returns the exclusive
// prefix, writes the block total to *total.
__device__ __forceinline__ int block_excl_scan_1024(int v, int *total, int *warp_sums /*[32]*/) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += t;
    }
    if (lane == 31) warp_sums[wid] = incl;
    __syncthreads();
    if (wid == 0) {
        int s = warp_sums[lane];
        int si = s;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, si, d);
            if (lane >= d) si += t;
        }
        warp_sums[lane] = si - s;  // exclusive prefix of warp sums
        if (lane == 31) *total = si;
    }
    __syncthreads();
    const int res = warp_sums[wid] + incl - v;
    __syncthreads();  // warp_sums / total may be reused by the caller
    return res;
}

// ------------------------------------------------------------------------------------------------
// route pass 2: one block per expert scans whist[:, e] over the slices (in place: whist[w][e]
// becomes the number of ids == e in earlier slices); the last block to finish scans the E counts
// into the exclusive / end / padded offsets.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
    route_scan_kernel(int32_t *__restrict__ whist, int W, int E, uint32_t *__restrict__ counts,
                      int32_t *__restrict__ excl_off, int32_t *__restrict__ end_off,
                      int32_t *__restrict__ padded_off, int32_t *__restrict__ mtile_off, int *ticket) {
    __shared__ int warp_sums[32];
    __shared__ int total_s;
    __shared__ int is_last;
    const int e = blockIdx.x;
    // W <= kRouteMaxSlices: kScanItems consecutive slices per thread, all loads issued before one block scan
    constexpr int kScanItems = (kRouteMaxSlices + 1023) / 1024;
    int v[kScanItems];
    int tsum = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        const int w = threadIdx.x * kScanItems + i;
        v[i] = (w < W) ? whist[int64_t(w) * E + e] : 0;
    }
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) tsum += v[i];
    int run = block_excl_scan_1024(tsum, &total_s, warp_sums);
    const int carry = total_s;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        const int w = threadIdx.x * kScanItems + i;
        if (w < W) whist[int64_t(w) * E + e] = run;
        run += v[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        counts[e] = uint32_t(carry);
        __threadfence();
        const int t = atomicAdd(ticket, 1);
        is_last = (t == E - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // E <= 1024: one expert per thread
    const int c = (threadIdx.x < E) ? int(__ldcg(&counts[threadIdx.x])) : 0;
    const int ex = block_excl_scan_1024(c, &total_s, warp_sums);
    if (threadIdx.x < E) {
        excl_off[threadIdx.x] = ex;
        end_off[threadIdx.x] = ex + c;
    }
    if (padded_off) {
        const int tiles = (c + CK_TILE_M - 1) / CK_TILE_M;
        const int tex = block_excl_scan_1024(tiles, &total_s, warp_sums);
        if (threadIdx.x < E) {
            mtile_off[threadIdx.x] = tex;
            padded_off[threadIdx.x] = tex * CK_TILE_M;
        }
        if (threadIdx.x == 0) {
            mtile_off[E] = total_s;
            padded_off[E] = total_s * CK_TILE_M;
        }
    }
    if (threadIdx.x == 0) *ticket = 0;
}

// ------------------------------------------------------------------------------------------------
// route pass 3: stable scatter.  Each warp walks its slice in order; an id's output position is
// excl_off[e] + whist[w][e] + (ids == e seen so far in this slice).
// ------------------------------------------------------------------------------------------------
// route pass 3: stable scatter, one thread block per slice, tiles of 8 x 512 ids.
//
// Inside a tile every id gets (expert, rank among the tile's ids of that expert); the tile is counting-sorted
// into shared memory and written out expert run by expert run, so global stores cover whole 32-byte sectors
// (an id-at-a-time scatter made every store a partial-sector read-modify-write in L2 and ran at a seventh of
// this speed).  The rank inside a warp round comes from a peer mask built in shared memory: every lane ORs its
// bit into a per-expert word, after a warp barrier the word holds exactly the lanes with that expert id.  Two
// mask buffers alternate so the clearing store of one round never races the ORs of the next.
constexpr int kTile = kRouteWarpsPerBlock * kStep;  // 4096 ids

template <typename IdT, bool HAS_SEXP, bool HAS_ROWMAP>
__global__ void __launch_bounds__(kRouteWarpsPerBlock * 32, 4)  // 4 blocks per SM: all 592 slices resident at once
    route_scatter_kernel(const IdT *__restrict__ ids, int64_t n, int E, int64_t slice,
                         const int32_t *__restrict__ whist, const int32_t *__restrict__ excl_off,
                         const int32_t *__restrict__ padded_off, int32_t *__restrict__ sorted_idx,
                         int32_t *__restrict__ sorted_expert, int32_t *__restrict__ row_map) {
    extern __shared__ int32_t smem_i[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    // shared-memory carve-up (ints)
    int32_t *gbase = smem_i;                         // [E] next global position per expert
    int32_t *delta = gbase + E;                      // [E] padded_off - excl_off
    int32_t *tstart = delta + E;                     // [E + 1] start of each expert's run inside the staged tile
    int32_t *wcnt = tstart + E + 1;                  // [warps][E] per-warp counts, then per-warp prefixes
    unsigned *wmask = reinterpret_cast<unsigned *>(wcnt + kRouteWarpsPerBlock * E);  // [warps][2][E]
    int32_t *stage_idx = reinterpret_cast<int32_t *>(wmask + 2 * kRouteWarpsPerBlock * E);  // [kTile]
    uint16_t *stage_e = reinterpret_cast<uint16_t *>(stage_idx + kTile);                    // [kTile]

    const int64_t begin = int64_t(blockIdx.x) * slice;
    const int len = int(min(begin + slice, n) - begin);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int ex = excl_off[e];
        gbase[e] = ex + whist[int64_t(blockIdx.x) * E + e];
        delta[e] = HAS_ROWMAP ? padded_off[e] - ex : 0;
    }
    for (int i = threadIdx.x; i < kRouteWarpsPerBlock * E; i += blockDim.x) wcnt[i] = 0;
    for (int i = threadIdx.x; i < 2 * kRouteWarpsPerBlock * E; i += blockDim.x) wmask[i] = 0u;
    __syncthreads();

    const unsigned lt = lanemask_lt();
    const unsigned bit = 1u << lane;
    int32_t *mycnt = wcnt + wib * E;
    unsigned *mk = wmask + wib * 2 * E;
    unsigned *mk_other = mk + E;
    bool bad = false;

    for (int tile = 0; tile < len; tile += kTile) {
        const int off = tile + wib * kStep;  // this warp's 512 ids of the tile
        int key[kLoads];
        if (off + kStep <= len) load_step<IdT, true>(ids + begin + off + lane, kStep, lane, E, key, bad);
        else if (off < len) load_step<IdT, false>(ids + begin + off + lane, len - off, lane, E, key, bad);
        else {
#pragma unroll
            for (int j = 0; j < kLoads; ++j) key[j] = -1;
        }
        // rank of every id among the ids of its expert inside this warp's 512
        int loc[kLoads];
#pragma unroll
        for (int j = 0; j < kLoads; ++j) {
            const int k = key[j];
            const bool valid = k >= 0;
            if (valid) atomicOr(mk + k, bit);
            __syncwarp();
            unsigned m = 0u;
            int b = 0;
            if (valid) {
                m = mk[k];
                b = mycnt[k];
            }
            __syncwarp();
            if (valid && (m & lt) == 0u) {  // lowest lane of the group advances the count and resets the mask
                mycnt[k] = b + __popc(m);
                mk[k] = 0u;
            }
            loc[j] = b + __popc(m & lt);
            unsigned *t = mk; mk = mk_other; mk_other = t;
        }
        __syncthreads();
        // per expert: counts of the 8 warps -> exclusive prefixes; tile totals -> run starts
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            int run = 0;
#pragma unroll
            for (int w = 0; w < kRouteWarpsPerBlock; ++w) {
                const int c = wcnt[w * E + e];
                wcnt[w * E + e] = run;
                run += c;
            }
            tstart[e + 1] = run;  // totals for now
        }
        __syncthreads();
        if (wib == 0) {  // exclusive scan of the totals over the experts (E <= 1024: 32 per lane at most)
            int carry = 0;
            for (int base = 0; base < E; base += 32) {
                const int e = base + lane;
                const int v = e < E ? tstart[e + 1] : 0;
                int incl = v;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, incl, d);
                    if (lane >= d) incl += t;
                }
                if (e < E) tstart[e + 1] = carry + incl;
                carry += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) tstart[0] = 0;
        }
        __syncthreads();
        // counting sort of the tile into shared memory
#pragma unroll
        for (int j = 0; j < kLoads; ++j) {
            const int k = key[j];
            if (k >= 0) {
                const int p = tstart[k] + mycnt[k] + loc[j];
                stage_idx[p] = int32_t(begin) + off + 32 * j + lane;  // n < 2^31 is checked by the host wrapper
                stage_e[p] = uint16_t(k);
            }
        }
        __syncthreads();
        // write the tile out: consecutive threads -> consecutive positions of one expert's run
        const int staged = tstart[E];
        for (int p = threadIdx.x; p < staged; p += blockDim.x) {
            const int k = stage_e[p];
            const int32_t src = stage_idx[p];
            const int pos = gbase[k] + (p - tstart[k]);
            sorted_idx[pos] = src;
            if (HAS_SEXP) sorted_expert[pos] = k;
            if (HAS_ROWMAP) row_map[pos + delta[k]] = src;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            gbase[e] += tstart[e + 1] - tstart[e];
#pragma unroll
            for (int w = 0; w < kRouteWarpsPerBlock; ++w) wcnt[w * E + e] = 0;
        }
        __syncthreads();
    }
}

static void route_plan(int64_t n, int64_t *slice, int *W) {
    if (n <= 0) {
        *slice = kStep;
        *W = 0;
        return;
    }
    int64_t s = ceil_div64(n, kRouteMaxSlices);
    s = ceil_div64(s, kTile) * kTile;  // whole tiles: every warp of a block takes one 512-id step per tile
    *slice = s;
    *W = int(ceil_div64(n, s));
}

}  // namespace ck

using namespace ck;

extern "C" int ck_continuous_count(const void *ids, int ids_is_i64, int64_t n, int size, uint32_t *counts,
                                   void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (size <= 0 || n < 0 || counts == nullptr) return CK_ERR_SHAPE;
    if (size > CK_COUNT_MAX_SIZE) return CK_ERR_RANGE;
    if (n > 0 && ids == nullptr) return CK_ERR_SHAPE;
    CK_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(uint32_t) * size, stream));
    if (n == 0) return CK_OK;
    const bool lane_private = size <= kLanePrivateMax;
    const int nbits = size > 1 ? 32 - __builtin_clz(unsigned(size - 1)) : 0;
    int wpb = 16;  // warps per block; one block per SM keeps the count of global atomics at num_sms * size
    if (lane_private) wpb = std::max(1, std::min(16, int((200 * 1024) / (size_t(size + 1) * 128))));
    const int threads = wpb * 32;
    const size_t smem = lane_private ? sizeof(uint32_t) * (size_t(size + 1) * 32 * wpb + size) : sizeof(uint32_t) * size;
    const int64_t nchunks = ceil_div64(n, kStep);
    int64_t grid = ceil_div64(nchunks, wpb);
    const int64_t cap = int64_t(num_sms()) * (lane_private ? 1 : 2);
    if (grid > cap) grid = cap;
#define CK_LAUNCH_COUNT(IDT, LP)                                                                                          \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            CK_CUDA_TRY(cudaFuncSetAttribute(count_kernel<IDT, LP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        count_kernel<IDT, LP><<<dim3((unsigned)grid), threads, smem, stream>>>((const IDT *)ids, n, size, nbits, counts);    \
    } while (0)
    if (ids_is_i64) {
        if (lane_private) CK_LAUNCH_COUNT(int64_t, true); else CK_LAUNCH_COUNT(int64_t, false);
    } else {
        if (lane_private) CK_LAUNCH_COUNT(int32_t, true); else CK_LAUNCH_COUNT(int32_t, false);
    }
#undef CK_LAUNCH_COUNT
    CK_LAUNCH_CHECK("count_kernel");
    return CK_OK;
}

extern "C" int64_t ck_route_workspace_bytes(int64_t n, int E) {
    if (n < 0 || E <= 0 || E > CK_ROUTE_MAX_EXPERTS) return CK_ERR_SHAPE;
    int64_t slice;
    int W;
    route_plan(n, &slice, &W);
    return 256 + int64_t(W > 0 ? W : 1) * E * int64_t(sizeof(int32_t));
}

extern "C" int64_t ck_route_padded_capacity(int64_t n, int E) {
    if (n < 0 || E <= 0) return CK_ERR_SHAPE;
    return (n / CK_TILE_M + E) * CK_TILE_M;
}

extern "C" int ck_route(const void *ids, int ids_is_i64, int64_t n, int E, uint32_t *counts, int32_t *excl_off,
                        int32_t *end_off, int32_t *sorted_idx, int32_t *sorted_expert, int32_t *padded_off,
                        int32_t *mtile_off, int32_t *row_map, void *workspace, int64_t workspace_bytes,
                        int32_t *dev_status, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (E <= 0 || E > CK_ROUTE_MAX_EXPERTS || n < 0) return CK_ERR_SHAPE;
    if (n > int64_t(INT32_MAX) - int64_t(E) * CK_TILE_M) return CK_ERR_SHAPE;
    if (!counts || !excl_off || !end_off || (n > 0 && (!ids || !sorted_idx))) return CK_ERR_SHAPE;
    const int meta = (padded_off != nullptr) + (mtile_off != nullptr) + (row_map != nullptr);
    if (meta != 0 && meta != 3) return CK_ERR_SHAPE;
    const int64_t need = ck_route_workspace_bytes(n, E);
    if (!workspace || workspace_bytes < need) return CK_ERR_WORKSPACE;

    int64_t slice;
    int W;
    route_plan(n, &slice, &W);
    int *ticket = (int *)workspace;
    int32_t *whist = (int32_t *)((char *)workspace + 256);
    CK_CUDA_TRY(cudaMemsetAsync(ticket, 0, 256, stream));
    if (row_map) CK_CUDA_TRY(cudaMemsetAsync(row_map, 0xFF, sizeof(int32_t) * ck_route_padded_capacity(n, E), stream));

    const int threads = kRouteWarpsPerBlock * 32;
    const int blocks = W;  // one thread block per slice
    if (W > 0) {
        const bool lane_private = E <= kLanePrivateMax;
        const size_t smem = sizeof(int32_t) * (size_t(E) + (lane_private ? size_t(kHistWarpsPerBlock) * (E + 1) * 32 : 0));
#define CK_LAUNCH_HIST(IDT, LP)                                                                                          \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            CK_CUDA_TRY(cudaFuncSetAttribute(route_hist_kernel<IDT, LP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        route_hist_kernel<IDT, LP><<<blocks, kHistWarpsPerBlock * 32, smem, stream>>>((const IDT *)ids, n, E, slice, whist, dev_status); \
    } while (0)
        if (ids_is_i64) {
            if (lane_private) CK_LAUNCH_HIST(int64_t, true); else CK_LAUNCH_HIST(int64_t, false);
        } else {
            if (lane_private) CK_LAUNCH_HIST(int32_t, true); else CK_LAUNCH_HIST(int32_t, false);
        }
#undef CK_LAUNCH_HIST
        CK_LAUNCH_CHECK("route_hist_kernel");
    }
    route_scan_kernel<<<E, 1024, 0, stream>>>(whist, W, E, counts, excl_off, end_off, padded_off, mtile_off, ticket);
    CK_LAUNCH_CHECK("route_scan_kernel");
    if (W > 0) {
        const size_t smem = sizeof(int32_t) * (size_t(27) * E + 1 + kTile + kTile / 2);  // gbase, delta, tstart, wcnt[8], wmask[16], staged ids + experts
        const bool sexp = sorted_expert != nullptr, rmap = row_map != nullptr;
#define CK_LAUNCH_SCATTER(IDT, SE, RM)                                                                                     \
    do {                                                                                                                   \
        if (smem > 48 * 1024)                                                                                              \
            CK_CUDA_TRY(cudaFuncSetAttribute(route_scatter_kernel<IDT, SE, RM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        route_scatter_kernel<IDT, SE, RM><<<blocks, threads, smem, stream>>>((const IDT *)ids, n, E, slice, whist, excl_off, \
                                                                            padded_off, sorted_idx, sorted_expert, row_map); \
    } while (0)
#define CK_SCATTER_FLAGS(IDT)                                   \
    do {                                                        \
        if (sexp && rmap) CK_LAUNCH_SCATTER(IDT, true, true);   \
        else if (sexp) CK_LAUNCH_SCATTER(IDT, true, false);     \
        else if (rmap) CK_LAUNCH_SCATTER(IDT, false, true);     \
        else CK_LAUNCH_SCATTER(IDT, false, false);              \
    } while (0)
        if (ids_is_i64) CK_SCATTER_FLAGS(int64_t); else CK_SCATTER_FLAGS(int32_t);
#undef CK_SCATTER_FLAGS
#undef CK_LAUNCH_SCATTER
        CK_LAUNCH_CHECK("route_scatter_kernel");
    }
    return CK_OK;
}

// ------------------------------------------------------------------------------------------------
// ck_route_static: the routing pass for callers that cannot bring a workspace.
//
// Some hosts of this library have no way to allocate device memory at the moment they need the routing
// tables: a serving loop whose memory pool is sealed after start-up, a plug-in living inside an engine
// that owns every byte of the device and hands out only the input and output buffers, a real-time step
// that must not run into the device-wide synchronisation cudaMalloc / cudaFree imply.  For them the
// per-slice histograms and the ticket counter live in the fixed array below instead of a caller-owned
// workspace.  The array is part of the loaded module: every GPU that loads the library holds these
// CK_ROUTE_STATIC_SCRATCH_BYTES until the process exits, whether or not this entry point is ever called.
//
// The array's name is only a host-side handle; the device address comes from cudaGetSymbolAddress, asked
// once per device with that device current (the first call on a device does this set-up, so make that
// first call outside any stream capture).  Nothing here calls cudaMalloc, cudaFree or an allocating
// library routine.  All calls share the one array and it keeps whatever the previous call left: the
// ticket counter is cleared on every call, the histogram slots in use are fully rewritten before they
// are read.  Two calls whose kernels overlap on the same GPU (different streams, or different host
// threads) race on the array; serialise them.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_route_static_scratch[CK_ROUTE_STATIC_SCRATCH_BYTES];

static int route_static_scratch_ptr(void **out) {
    static std::mutex mu;
    static void *ptrs[64];  // per device, nullptr = not looked up yet
    int dev = -1;
    CK_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return CK_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void *p = nullptr;
        CK_CUDA_TRY(cudaGetSymbolAddress(&p, g_route_static_scratch));
        if (p == nullptr) return CK_ERR_CUDA;
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return CK_OK;
}

extern "C" int64_t ck_route_static_max_bytes(void) { return CK_ROUTE_STATIC_SCRATCH_BYTES; }

extern "C" int ck_route_static(const void *ids, int ids_is_i64, int64_t n, int E, uint32_t *counts, int32_t *excl_off,
                               int32_t *end_off, int32_t *sorted_idx, int32_t *sorted_expert, int32_t *padded_off,
                               int32_t *mtile_off, int32_t *row_map, int32_t *dev_status, void *stream_) {
    const int64_t need = ck_route_workspace_bytes(n, E);
    if (need < 0) return CK_ERR_SHAPE;
    if (need > CK_ROUTE_STATIC_SCRATCH_BYTES) return CK_ERR_RANGE;  // n * E beyond the built-in scratch
    void *scratch = nullptr;
    const int rc = route_static_scratch_ptr(&scratch);
    if (rc != CK_OK) return rc;
    return ck_route(ids, ids_is_i64, n, E, counts, excl_off, end_off, sorted_idx, sorted_expert, padded_off, mtile_off,
                    row_map, scratch, CK_ROUTE_STATIC_SCRATCH_BYTES, dev_status, stream_);
}
