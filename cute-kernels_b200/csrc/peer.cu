// Expert-parallel dispatch over peer memory: the rows a rank's experts need are read straight out of the
// other ranks' token buffers (NVLink loads), instead of being packed, sent through an all-to-all and
// re-gathered.  The reference has no multi-GPU path; per rank these kernels are its `group`
// (kernels/scattermoe/triton_implementation/ops.py:108-140) with the source row living on another GPU.
//
// Addressing: every rank exposes a buffer of `rows_per_peer` slots; a routed row is named by its global
// flat slot g = rank * rows_per_peer + f (f = token * k + j on the owning rank).  `peer[r]` is rank r's
// buffer as mapped into this process (the local rank's own buffer included).
//
// None of these kernels waits on another GPU: ordering between ranks comes from stream-ordered
// collectives issued by the host between the phases.
#include "ck_common.cuh"

namespace ck {

struct PeerTable {
    void *p[CK_MAX_PEERS];
};

constexpr int kPeerThreads = 128;
constexpr int kPeerUnroll = 8;

// dst[p, :] = peer[g / S][(g % S) / fan_out, :] with g = src_flat ? src_flat[row_map[p]] : row_map[p]; zeros where
// row_map[p] < 0.
// Every block owns one contiguous run of padded rows, so at any moment the grid reads from all parts of the
// sorted order at once.  The sorted order is source-rank major inside an expert: a grid-stride sweep would have
// every GPU of the node pulling from the same source rank at the same time and queue on that rank's links.
template <typename T>
__global__ void __launch_bounds__(kPeerThreads)
    gather_rows_peer_kernel(const PeerTable peers, int n_peers, int64_t S, T *__restrict__ dst,
                            const int32_t *__restrict__ row_map, const int32_t *__restrict__ padded_off,
                            const int32_t *__restrict__ src_flat, int E, int64_t cap, int fan_out, int64_t vpr,
                            int64_t row_begin, int64_t row_end, int32_t *dev_status) {
    constexpr int VEC = Vec16<T>::N;
    int64_t rows = padded_off[E];
    if (rows > cap) rows = cap;
    if (rows > row_end) rows = row_end;
    if (rows <= row_begin) return;
    const int64_t rows_per_block = ceil_div64(rows - row_begin, gridDim.x);
    const int64_t row0 = row_begin + int64_t(blockIdx.x) * rows_per_block;
    const int64_t row1 = min(row0 + rows_per_block, rows);
    const int lane = threadIdx.x & 31;
    bool bad = false;
    // one warp per row of the block's run: the slot is decoded once per row, the lanes stream the row
    for (int64_t p = row0 + (threadIdx.x >> 5); p < row1; p += kPeerThreads / 32) {
        const int32_t s = row_map[p];
        const int4 *sr = nullptr;
        if (s >= 0) {
            const int64_t g = src_flat ? int64_t(src_flat[s]) : int64_t(s);
            const int64_t r = g / S;
            if (g >= 0 && r < n_peers)
                sr = reinterpret_cast<const int4 *>(reinterpret_cast<const T *>(peers.p[r]) + ((g - r * S) / fan_out) * (vpr * VEC));
            else
                bad = true;
        }
        int4 *d = reinterpret_cast<int4 *>(dst + p * (vpr * VEC));
        for (int64_t c0 = lane; c0 < vpr; c0 += 32 * kPeerUnroll) {
            int4 x[kPeerUnroll];
#pragma unroll
            for (int j = 0; j < kPeerUnroll; ++j) {
                const int64_t c = c0 + 32 * j;
                x[j] = make_int4(0, 0, 0, 0);
                if (sr && c < vpr) x[j] = sr[c];  // plain load: the source may be another GPU's memory
            }
#pragma unroll
            for (int j = 0; j < kPeerUnroll; ++j) {
                const int64_t c = c0 + 32 * j;
                if (c < vpr) d[c] = x[j];
            }
        }
    }
    if (bad && dev_status) atomicOr(dev_status, CK_DEV_RANGE);
}

// dst[j] = peer[g / S][g % S], g = flat[j]  (U = 2- or 4-byte scalar)
template <typename U>
__global__ void __launch_bounds__(kPeerThreads)
    peer_gather_scalars_kernel(const PeerTable peers, int n_peers, int64_t S, const int32_t *__restrict__ flat, int64_t n,
                               U *__restrict__ dst, int32_t *dev_status) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t j = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride) {
        const int64_t g = flat[j];
        const int64_t r = g / S;
        if (g >= 0 && r < n_peers) dst[j] = reinterpret_cast<const U *>(peers.p[r])[g - r * S];
        else if (dev_status) atomicOr(dev_status, CK_DEV_RANGE);
    }
}

// peer[g / S][g % S] = by_slot ? vals[g] : vals[j], g = flat[j]; entries with g < 0 (pad rows) are skipped.
// Every slot has exactly one writer across all ranks.
template <typename U>
__global__ void __launch_bounds__(kPeerThreads)
    peer_scatter_scalars_kernel(const U *__restrict__ vals, const int32_t *__restrict__ flat, int64_t n, int by_slot,
                                const PeerTable peers, int n_peers, int64_t S, int32_t *dev_status) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t j = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride) {
        const int64_t g = flat[j];
        if (g < 0) continue;
        const int64_t r = g / S;
        if (r < n_peers) reinterpret_cast<U *>(peers.p[r])[g - r * S] = vals[by_slot ? g : j];
        else if (dev_status) atomicOr(dev_status, CK_DEV_RANGE);
    }
    __threadfence_system();  // the stores must have landed on the peer before this rank's next collective
}

static int fill_table(PeerTable &t, const void *const *ptrs, int n_peers) {
    if (!ptrs || n_peers <= 0 || n_peers > CK_MAX_PEERS) return CK_ERR_SHAPE;
    for (int i = 0; i < CK_MAX_PEERS; ++i) t.p[i] = i < n_peers ? const_cast<void *>(ptrs[i]) : nullptr;
    for (int i = 0; i < n_peers; ++i)
        if (!t.p[i] || (reinterpret_cast<uintptr_t>(t.p[i]) & 15)) return CK_ERR_SHAPE;
    return CK_OK;
}

static inline unsigned peer_grid(int64_t items) {
    int64_t blocks = ceil_div64(items, kPeerThreads);
    const int64_t cap = int64_t(num_sms()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return unsigned(blocks);
}

template <typename T>
static int gather_rows_peer_t(const PeerTable &t, int n_peers, int64_t S, void *dst, const int32_t *row_map,
                              const int32_t *padded_off, const int32_t *src_flat, int E, int64_t cap, int fan_out,
                              int64_t cols, int64_t row_begin, int64_t row_end, int32_t *dev_status, cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    if (cols % VEC != 0 || (reinterpret_cast<uintptr_t>(dst) & 15)) return CK_ERR_SHAPE;
    const int64_t vpr = cols / VEC;
    const int64_t span = (row_end < cap ? row_end : cap) - row_begin;
    gather_rows_peer_kernel<T><<<peer_grid(ceil_div64(span * vpr, kPeerUnroll)), kPeerThreads, 0, stream>>>(
        t, n_peers, S, (T *)dst, row_map, padded_off, src_flat, E, cap, fan_out, vpr, row_begin, row_end, dev_status);
    CK_LAUNCH_CHECK("gather_rows_peer_kernel");
    return CK_OK;
}

}  // namespace ck

using namespace ck;

extern "C" int ck_moe_gather_rows_peer(const void *const *peer_src, int n_peers, int64_t rows_per_peer, void *dst,
                                       const int32_t *row_map, const int32_t *padded_off, const int32_t *src_flat, int E,
                                       int64_t cap, int fan_out, int64_t cols, int64_t row_begin, int64_t row_end,
                                       int dtype, int32_t *dev_status, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!dst || !row_map || !padded_off || E <= 0 || cap < 0 || fan_out <= 0 || cols <= 0 || rows_per_peer <= 0)
        return CK_ERR_SHAPE;
    if (rows_per_peer * n_peers > INT32_MAX) return CK_ERR_RANGE;
    PeerTable t;
    const int rc = fill_table(t, peer_src, n_peers);
    if (rc != CK_OK) return rc;
    if (row_begin < 0 || row_end < row_begin) return CK_ERR_SHAPE;
    if (cap == 0 || row_begin >= cap || row_end == row_begin) return CK_OK;
    switch (dtype) {
        case CK_F32: return gather_rows_peer_t<float>(t, n_peers, rows_per_peer, dst, row_map, padded_off, src_flat, E, cap, fan_out, cols, row_begin, row_end, dev_status, stream);
        case CK_F16: return gather_rows_peer_t<__half>(t, n_peers, rows_per_peer, dst, row_map, padded_off, src_flat, E, cap, fan_out, cols, row_begin, row_end, dev_status, stream);
        case CK_BF16: return gather_rows_peer_t<__nv_bfloat16>(t, n_peers, rows_per_peer, dst, row_map, padded_off, src_flat, E, cap, fan_out, cols, row_begin, row_end, dev_status, stream);
        default: return CK_ERR_UNSUPPORTED;
    }
}

extern "C" int ck_peer_gather_scalars(const void *const *peer_src, int n_peers, int64_t rows_per_peer,
                                      const int32_t *flat, int64_t n, void *dst, int elem_bytes, int32_t *dev_status,
                                      void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n < 0 || rows_per_peer <= 0 || (elem_bytes != 2 && elem_bytes != 4)) return CK_ERR_SHAPE;
    if (rows_per_peer * n_peers > INT32_MAX) return CK_ERR_RANGE;
    PeerTable t;
    const int rc = fill_table(t, peer_src, n_peers);
    if (rc != CK_OK) return rc;
    if (n == 0) return CK_OK;
    if (!flat || !dst) return CK_ERR_SHAPE;
    if (elem_bytes == 2)
        peer_gather_scalars_kernel<uint16_t><<<peer_grid(n), kPeerThreads, 0, stream>>>(t, n_peers, rows_per_peer, flat, n, (uint16_t *)dst, dev_status);
    else
        peer_gather_scalars_kernel<uint32_t><<<peer_grid(n), kPeerThreads, 0, stream>>>(t, n_peers, rows_per_peer, flat, n, (uint32_t *)dst, dev_status);
    CK_LAUNCH_CHECK("peer_gather_scalars_kernel");
    return CK_OK;
}

extern "C" int ck_peer_scatter_scalars(const void *vals, const int32_t *flat, int64_t n, int by_slot, void *const *peer_dst,
                                       int n_peers, int64_t rows_per_peer, int elem_bytes, int32_t *dev_status,
                                       void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n < 0 || rows_per_peer <= 0 || (elem_bytes != 2 && elem_bytes != 4)) return CK_ERR_SHAPE;
    if (rows_per_peer * n_peers > INT32_MAX) return CK_ERR_RANGE;
    PeerTable t;
    const int rc = fill_table(t, (const void *const *)peer_dst, n_peers);
    if (rc != CK_OK) return rc;
    if (n == 0) return CK_OK;
    if (!flat || !vals) return CK_ERR_SHAPE;
    if (elem_bytes == 2)
        peer_scatter_scalars_kernel<uint16_t><<<peer_grid(n), kPeerThreads, 0, stream>>>((const uint16_t *)vals, flat, n, by_slot, t, n_peers, rows_per_peer, dev_status);
    else
        peer_scatter_scalars_kernel<uint32_t><<<peer_grid(n), kPeerThreads, 0, stream>>>((const uint32_t *)vals, flat, n, by_slot, t, n_peers, rows_per_peer, dev_status);
    CK_LAUNCH_CHECK("peer_scatter_scalars_kernel");
    return CK_OK;
}
