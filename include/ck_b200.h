/*
 * ck_b200.h -- C ABI of the B200 (sm_100a) MoE expert path.
 *
 * One ahead-of-time built shared library (libck_b200.so) replaces the JIT-built pybind modules and
 * the Triton launches of the reference for this path.  Every entry point
 *   - takes plain device pointers, sizes and a cudaStream_t passed as void*,
 *   - never allocates or frees device memory (outputs and workspaces are caller-owned),
 *   - launches on the given stream and returns without synchronising,
 *   - returns a ck_status (0 = ok, negative = error) for everything the host can check,
 *   - reports device-side findings (out-of-range expert id, a bounded wait that ran out) by
 *     OR-ing a CK_DEV_* bit into the caller's `dev_status` word (device memory, may be NULL).
 *
 * Citations name files of the reference project (cute_kernels/...).
 */
#ifndef CK_B200_H
#define CK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CK_API __attribute__((visibility("default")))
#else
#define CK_API
#endif

/* ---- status ------------------------------------------------------------------------------ */
enum {
    CK_OK = 0,
    CK_ERR_SHAPE = -1,       /* a size / stride / alignment the kernel cannot take            */
    CK_ERR_RANGE = -2,       /* value out of the accepted range (e.g. size > CK_COUNT_MAX_SIZE)*/
    CK_ERR_TIMEOUT = -3,     /* reserved for hosts that translate CK_DEV_TIMEOUT               */
    CK_ERR_CUDA = -4,        /* a CUDA runtime / driver call failed (see ck_last_cuda_error)   */
    CK_ERR_UNSUPPORTED = -5, /* dtype / mode not built                                         */
    CK_ERR_WORKSPACE = -6    /* workspace pointer NULL or too small                            */
};

/* bits OR-ed into *dev_status by kernels */
enum {
    CK_DEV_RANGE = 1,   /* an expert id outside [0, E) was seen (the element was skipped)        */
    CK_DEV_TIMEOUT = 2, /* a bounded mbarrier wait ran out; the kernel backed out, output invalid */
    CK_DEV_META = 4     /* tile metadata inconsistent with the launch (capacity too small)        */
};

/* element types of activations / weights */
enum { CK_F32 = 0, CK_F16 = 1, CK_BF16 = 2 };

/* fused activation of the up projection */
enum {
    CK_ACT_SWIGLU = 0, /* up * silu(gate)     (swiglu_packed: [up | gate] along the last dim)   */
    CK_ACT_GLU = 1,    /* up * sigmoid(gate)  (torch.nn.GLU on the same packing)                 */
    CK_ACT_GELU_TANH = 2 /* un-gated: gelu(pre) with the tanh approximation (torch.nn.GELU(approximate="tanh"),
                          * the reference tests' is_glu=False activation, tests/test_commons.py:85-86): Wfc is
                          * [E, I, H], and h / dh are [cap, I] instead of [cap, 2I]                           */
};

#define CK_COUNT_MAX_SIZE 16384 /* same bound as kernels/continuous_count/cuda_implementation/forward.cu:12 */
#define CK_ROUTE_MAX_EXPERTS 1024
#define CK_TILE_M 128 /* rows of one grouped-GEMM tile; expert segments are padded to this */

CK_API const char *ck_status_string(int status);
CK_API const char *ck_last_cuda_error(void);
CK_API int ck_abi_version(void);

/* ---- continuous_count --------------------------------------------------------------------
 * Replaces continuous_count_cuda (kernels/continuous_count/cuda_implementation/ops.cpp:7-15,
 * forward.cu:110-178): counts[v] = #{i : ids[i] == v} for v in [0, size); values outside the
 * range are ignored, as kernels/continuous_count/__init__.py:15-16 promises.
 * ids: int32 or int64 device array of n elements (any alignment of the element type).
 * counts: uint32[size], fully overwritten.  size <= CK_COUNT_MAX_SIZE. */
CK_API int ck_continuous_count(const void *ids, int ids_is_i64, int64_t n, int size, uint32_t *counts,
                        void *stream);

/* ---- routing: count + scan + stable scatter ----------------------------------------------
 * Replaces the three torch calls of MoE_Triton._compute_experts
 * (kernels/scattermoe/triton_implementation/__init__.py:82-83: sort(), bincount(), cumsum())
 * and MoE_Torch._compute_expert_assignment (kernels/scattermoe/torch_implementation.py:171-193).
 *
 *   counts[e]      = bincount(ids, minlength=E)
 *   excl_off[e]    = sum_{e'<e} counts[e']            (exclusive scan)
 *   end_off[e]     = excl_off[e] + counts[e]          (the reference's expert_offsets)
 *   sorted_idx[j]  = torch.sort(ids, stable=True).indices[j]   (int32)
 *   sorted_expert[j] = ids[sorted_idx[j]]             (optional, may be NULL)
 *
 * Optional grouped-GEMM metadata (all three NULL, or all three non-NULL): expert segments padded
 * to CK_TILE_M rows so that one GEMM tile never spans two experts.
 *   padded_off[E+1] : start row of each expert in the padded layout; padded_off[E] = total rows
 *   mtile_off[E+1]  : padded_off / CK_TILE_M
 *   row_map[cap]    : row_map[padded_off[e] + r] = sorted_idx[excl_off[e] + r]; -1 on pad rows.
 *                     cap = ck_route_padded_capacity(n, E).
 * n <= 2^31 - 1 - E*CK_TILE_M; E <= CK_ROUTE_MAX_EXPERTS.  Out-of-range ids are skipped and flagged
 * with CK_DEV_RANGE (the outputs then describe the in-range ids only). */
CK_API int64_t ck_route_workspace_bytes(int64_t n, int E);
CK_API int64_t ck_route_padded_capacity(int64_t n, int E);
CK_API int ck_route(const void *ids, int ids_is_i64, int64_t n, int E, uint32_t *counts, int32_t *excl_off,
             int32_t *end_off, int32_t *sorted_idx, int32_t *sorted_expert, int32_t *padded_off,
             int32_t *mtile_off, int32_t *row_map, void *workspace, int64_t workspace_bytes,
             int32_t *dev_status, void *stream);

/* ck_route without a caller workspace.  No counterpart in the reference (its routing goes through torch
 * ops that allocate freely); added for hosts that cannot allocate device memory where they call this:
 * a sealed memory pool, an engine that owns the device and passes only inputs and outputs, a step that
 * must not meet the device-wide synchronisation of cudaMalloc / cudaFree.  The scratch is a fixed
 * CK_ROUTE_STATIC_SCRATCH_BYTES array inside the library, held by every GPU that loads it until exit.
 * Same outputs, bit for bit, as ck_route.  Limits: ck_route_workspace_bytes(n, E) must not exceed
 * CK_ROUTE_STATIC_SCRATCH_BYTES (any n at E <= 256; n <= 1,212,416 ids at E = 512; n <= 606,208 at E = 1024), otherwise
 * CK_ERR_RANGE and nothing is launched.  The first call on a device looks up the array's device address
 * (make it outside stream capture) and keeps it for the life of the process: the cached address does not survive
 * cudaDeviceReset.  Calls share the array: do not let two of them overlap on one GPU. */
#define CK_ROUTE_STATIC_SCRATCH_BYTES (256 + 148 * 32 * 32 * 4)
CK_API int64_t ck_route_static_max_bytes(void);
CK_API int ck_route_static(const void *ids, int ids_is_i64, int64_t n, int E, uint32_t *counts,
                           int32_t *excl_off, int32_t *end_off, int32_t *sorted_idx, int32_t *sorted_expert,
                           int32_t *padded_off, int32_t *mtile_off, int32_t *row_map, int32_t *dev_status,
                           void *stream);

/* ---- SwiGLU ------------------------------------------------------------------------------
 * Replace swiglu_forward_cuda / swiglu_backward_cuda
 * (kernels/swiglu/cuda_implementation/ops.cpp:7-22, forward.cu:31-93, backward.cu:44-128) and
 * the strided Triton kernels used by swiglu_packed_cute (kernels/swiglu/__init__.py:114-138).
 *   out = up * gate * sigmoid(gate)                      (fp32 math, round-to-nearest downcast)
 *   dgate = dy * up * (s + gate*s*(1-s)), dup = dy * gate * s,   s = sigmoid(gate)
 * sigmoid clamps its argument to +-88.3762626647949 (include/activations.h:9-22).
 * Tensors are rows x cols with a row stride in elements (contiguous: rows=1, cols=numel).
 * The packed form passes up = x, gate = x + cols, stride = 2*cols. */
CK_API int ck_swiglu_fwd(const void *gate, const void *up, void *out, int64_t rows, int64_t cols,
                  int64_t in_stride, int64_t out_stride, int dtype, void *stream);
CK_API int ck_swiglu_bwd(const void *gate, const void *up, const void *dy, void *dgate, void *dup,
                  int64_t rows, int64_t cols, int64_t in_stride, int64_t dy_stride,
                  int64_t grad_stride, int dtype, void *stream);

/* ---- grouped rows: gather / cast ----------------------------------------------------------
 * ck_moe_gather_rows replaces `group` (kernels/scattermoe/triton_implementation/ops.py:108-140,
 * kernels.py:225-280) for the padded layout: dst[p, :] = src[row_map[p] / fan_out, :] for
 * p < padded_off[E], zeros on pad rows (row_map[p] < 0).  cap rows are scanned. */
CK_API int ck_moe_gather_rows(const void *src, void *dst, const int32_t *row_map, const int32_t *padded_off,
                       int E, int64_t cap, int fan_out, int64_t cols, int dtype, void *stream);
/* dst[i] = (T) src[i] for fp32 staging buffers of the fused combine */
CK_API int ck_cast_from_f32(const float *src, void *dst, int64_t n, int dtype, void *stream);

/* ---- grouped GEMMs (tcgen05 / TMEM / TMA) -------------------------------------------------
 * Together these replace scatter2scatter, group_bwd_W and the bmm / sum combines of
 * _ScatteredExperts (kernels/scattermoe/triton_implementation/ops.py:31-105,143-292,
 * kernels.py:12-222).  Notation: Rp = padded_off[E] rows (capacity `cap` allocated), H hidden,
 * I intermediate, T tokens, k top-k.  All matrices row-major, 16-byte aligned, leading dimensions
 * equal to the logical widths.  H % 8 == 0 and I % 8 == 0.
 * Every entry that takes mtile_off processes the m-tiles [mtile_off[e], mtile_off[e+1]) of expert e; mtile_off[0]
 * may be above 0 and the array may be a clamped copy (min(max(mtile_off, lo), hi)): the call then covers only the
 * padded rows [128 lo, 128 hi), which lets a caller run one window while another is still being filled.
 * `tmap_cache` is reserved (pass NULL). */

/* up projection + fused activation:  h[p, :] = xg[p, :] @ Wfc[e]^T + b_fc[e]  ([up | gate], 2I wide),
 * act[p, :] = w[p] * up * silu(gate), with w[p] = gate_w[row_map[p]] (1 if gate_w is NULL).
 * Wfc: [E, 2I, H] (c_fc.weight); b_fc: [E, 2I] (c_fc.bias, Experts_Torch torch_implementation.py:20-22,41-44) or
 * NULL.  h may be NULL (inference: gate/up never reach HBM).  With act_kind == CK_ACT_GELU_TANH the layer is un-gated:
 * Wfc [E, I, H], b_fc [E, I], h[p, :] = the I pre-activations, act = w * gelu(h). */
CK_API int ck_moe_up_act_fwd(const void *xg, const void *wfc, const void *b_fc, const void *gate_w, const int32_t *row_map,
                      const int32_t *mtile_off, void *act, void *h, int E, int64_t cap, int H, int I,
                      int act_kind, int dtype, int32_t *dev_status, void *stream);

/* the same with the gather fused into the kernel -- scatter2scatter with x_grouped=False (kernels.py:63-66): the
 * routed rows are read from the un-permuted token matrix x [tokens, H] (token of padded row p = row_map[p] / top_k)
 * by the GEMM's own producer and never have to exist as a grouped matrix first.  CTA-pair kernels (the default): two
 * producer warps per CTA copy 16-byte pieces of the rows into the 128-byte-swizzled stages with cp.async; when
 * xg_out is not NULL the first n-tile of every m-tile also stores its stages back out as the grouped copy xg_out
 * [cap, H] (zero pad rows included) that ck_moe_wgrad contracts over later.  Single-CTA kernels
 * (ck_set_gemm_cta_pair(0)): TMA gather4, xg_out must be NULL (CK_ERR_UNSUPPORTED otherwise). */
CK_API int ck_moe_up_act_fwd_gather(const void *x, int64_t tokens, int top_k, const void *wfc, const void *b_fc, const void *gate_w,
                                    const int32_t *row_map, const int32_t *mtile_off, void *act, void *h,
                                    void *xg_out, int E, int64_t cap, int H, int I, int act_kind, int dtype,
                                    int32_t *dev_status, void *stream);

/* down projection + fused gather-back and top-k combine:
 * out32[row_map[p] / k, :] += act[p, :] @ Wproj[e]^T + w[p] * b_proj[e]   (fp32 red.add into a zeroed [T, H] buffer).
 * Wproj: [E, H, I] (c_proj.weight); b_proj: [E, H] (c_proj.bias) or NULL; gate_w as in the up projection (the
 * activations already carry w[p], the bias term needs it here; NULL: w = 1). */
CK_API int ck_moe_down_combine_fwd(const void *act, const void *wproj, const void *b_proj, const void *gate_w,
                            const int32_t *row_map, const int32_t *mtile_off, float *out32, int E, int64_t cap,
                            int H, int I, int top_k, int dtype, int32_t *dev_status, void *stream);

/* dgrad of the down projection fused with the activation backward and the router-weight grad:
 *   g[p, :]   = dyg[p, :] @ Wproj[e]                      (dyg = gathered, un-weighted grad_out)
 *   dh[p, :]  = activation_backward(h[p, :], w[p] * g[p, :])      ([dup | dgate], 2I wide)
 *   router-weight grad of row p: sum_n a[p, n] * g[p, n],  a = up * silu(gate) recomputed from h.  Two forms:
 *     dgates_part != NULL: every (n-tile, epilogue group) stores its partial sum into
 *       dgates_part[part * cap + p] (fp32 [ck_moe_dgrad_down_parts(I), cap], plain stores, no initialisation
 *       needed); ck_moe_reduce_dgates then adds the parts in a fixed order into dgates[row_map[p]] -- bit-reproducible;
 *     dgates_part == NULL: atomicAdd into dgates[row_map[p]] (caller zeroes dgates; summation order varies).
 *   Both pointers NULL: the router-weight grad is not produced.
 * (the reference obtains d_gates from a bmm over the saved un-combined expert outputs, ops.py:209-214) */
CK_API int ck_moe_dgrad_down(const void *dyg, const void *wproj, const void *h, const void *gate_w,
                      const int32_t *row_map, const int32_t *mtile_off, void *dh, float *dgates,
                      float *dgates_part, int E, int64_t cap, int H, int I, int act_kind, int dtype,
                      int32_t *dev_status, void *stream);
CK_API int ck_moe_dgrad_down_parts(int I);
CK_API int ck_moe_reduce_dgates(const float *dgates_part, int n_parts, int64_t cap, const int32_t *row_map,
                                const int32_t *padded_off, int E, float *dgates, void *stream);

/* ck_moe_dgrad_down with the grad rows read from the un-permuted dy [tokens, H] by the kernel's own producer
 * (token of padded row p = row_map[p] / top_k) instead of a pre-gathered dyg; dyg_out as xg_out of
 * ck_moe_up_act_fwd_gather (the grouped copy the weight gradient of the down projection contracts over). */
CK_API int ck_moe_dgrad_down_gather(const void *dy, int64_t tokens, int top_k, const void *wproj, const void *h,
                                    const void *gate_w, const int32_t *row_map, const int32_t *mtile_off, void *dh,
                                    float *dgates, float *dgates_part, void *dyg_out, int E, int64_t cap, int H,
                                    int I, int act_kind, int dtype, int32_t *dev_status, void *stream);

/* dgrad of the up projection fused with the k-way sum:
 *   dx32[row_map[p] / k, :] += dh[p, :] @ Wfc[e]          (fp32 red.add into a zeroed [T, H])  */
CK_API int ck_moe_dgrad_up(const void *dh, const void *wfc, const int32_t *row_map, const int32_t *mtile_off,
                    float *dx32, int E, int64_t cap, int H, int I2, int top_k, int dtype,
                    int32_t *dev_status, void *stream);

/* wgrad: dW[e] = A_e^T @ B_e over the padded rows of expert e (pad rows must be zero in A or B and
 * finite in both).  A: [cap, M], B: [cap, N], dW: [E, M, N], fully overwritten (zeros for experts
 * without rows, so the caller needs no memset -- ops.py:252 zero-fills instead). */
CK_API int ck_moe_wgrad(const void *a, const void *b, const int32_t *padded_off, void *dw, int E, int64_t cap,
                 int M, int N, int dtype, int32_t *dev_status, void *stream);

/* ck_moe_wgrad with either operand gathered by TMA from an un-permuted matrix: with a_fan > 0, A is
 * [a_rows, M] and row p of the padded layout reads A[row_map[p] / a_fan, :] (likewise B with b_fan / b_rows);
 * a fan of 0 means that operand is already in the padded layout ([cap, M] / [cap, N]).  The operand that is not
 * gathered must be zero on pad rows.  Replaces group() + group_bwd_W (ops.py:228-260). */
CK_API int ck_moe_wgrad_gather(const void *a, int64_t a_rows, int a_fan, const void *b, int64_t b_rows, int b_fan,
                               const int32_t *row_map, const int32_t *padded_off, void *dw, int E, int64_t cap, int M,
                               int N, int dtype, int32_t *dev_status, void *stream);

/* plain grouped linear on padded rows (used when the activation is an arbitrary callable and for
 * expert-parallel shards whose rows travel back before the combine):
 *   trans_w == 0: y[p, :] = x[p, :] @ W[e]^T,  W: [E, N, K]     (forward)
 *   trans_w == 1: y[p, :] = x[p, :] @ W[e],    W: [E, K, N]     (dgrad)                        */
CK_API int ck_moe_grouped_linear(const void *x, const void *w, const int32_t *mtile_off, void *y, int E,
                          int64_t cap, int N, int K, int trans_w, int dtype, int32_t *dev_status,
                          void *stream);

/* Kernel flavour of the grouped GEMMs: 1 (default) = CTA pairs (tcgen05 cta_group::2, 256 x 256 tile per pair,
 * half of the weight tile per CTA), 0 = one CTA per 128 x 256 tile.  Returns the previous setting.  The initial
 * value comes from the environment variable CK_GEMM_CTA_PAIR.  Takes the place of the reference's per-call
 * cutotune knobs (cute_kernels/cutotune/): there is no runtime search, only this switch. */
CK_API int ck_set_gemm_cta_pair(int enable);
CK_API int ck_gemm_cta_pair(void); /* the current setting */
/* SMs the persistent grouped-GEMM grids may occupy: `sms` <= 0 or >= the device's SM count means all of them (the default;
 * CK_GEMM_SMS in the environment sets the initial value).  A smaller budget leaves SMs free so that kernels launched on
 * other streams (row pulls over NVLink, collectives) run beside a GEMM instead of in its tail.  Process-wide, like
 * ck_set_gemm_cta_pair; returns the previous budget.  No counterpart in the reference (its GEMMs are not persistent). */
CK_API int ck_set_gemm_sm_budget(int sms);
CK_API int ck_gemm_sm_budget(void); /* SMs in use by the next launch on the current device */

/* same as ck_moe_grouped_linear (plus an optional bias [E, N], scaled by gate_w[row_map[p]] when gate_w is given),
 * but row p of the result is stored at y[row_map[p], :] (pad rows dropped):
 * scatter2scatter with y_grouped=False and FAN_OUT=1 (ops.py:31-78) -- used by expert-parallel shards, where
 * every routed row is produced exactly once and travels back before the combine. */
CK_API int ck_moe_grouped_linear_scatter(const void *x, const void *w, const void *bias, const void *gate_w,
                                         const int32_t *mtile_off, const int32_t *row_map, void *y, int E, int64_t cap,
                                         int N, int K, int trans_w, int dtype, int32_t *dev_status, void *stream);

/* Bias gradients of a layer with add_bias=True (autograd of Experts_Torch's F.linear bias, torch_implementation.py:41-44).
 * ck_moe_bias_grad: out[e, n] = sum over the padded rows p of expert e of s(p) * rows[p, n], s(p) = gate_w[row_map[p]]
 *   (1 when gate_w is NULL); rows [cap, N], out [E, N] in `dtype`, summed in a fixed order.  d c_fc.bias = this over dh,
 *   d c_proj.bias = this over the gathered grad rows with the router weights.
 * ck_moe_bias_dots: part[p] = rows[p, :] . bias[e(p), :] (fp32 [cap]): the bias term of the router-weight gradient,
 *   laid out like one more part of the dgates_part buffer of ck_moe_dgrad_down. */
CK_API int ck_moe_bias_grad(const void *rows, int64_t cap, int N, const int32_t *row_map, const void *gate_w,
                            const int32_t *padded_off, int E, void *out, int dtype, void *stream);
CK_API int ck_moe_bias_dots(const void *rows, int64_t cap, int N, const void *bias, const int32_t *padded_off, int E,
                            float *part, int dtype, void *stream);

/* ---- row permutations around the expert-parallel exchange ---------------------------------------
 * ck_moe_gather_rows_scaled: dst[j, :] = c * src[idx[j] / fan_out, :], c = coeff ? coeff[idx[j]] : 1, zeros
 *   where idx[j] < 0 -- `group` with its optional coefficient (ops.py:108-140, kernels.py:225-280).
 * ck_moe_combine_rows: out[t, :] = sum_{j<k} (w ? w[t*k+j] : 1) * src[pos ? pos[t*k+j] : t*k+j, :] -- the bmm(gates, out)
 *   combine (ops.py:170-174) and the sum(-2) of the input grad (ops.py:276), deterministic, fp32 accumulate.
 * ck_moe_row_dots: dots[f] = <a[pos[f], :], b[f / k, :]> -- d_gates = bmm(output_expanded, grad_out) (ops.py:214).
 * cols must be a multiple of 16 bytes of elements; pointers 16-byte aligned. */
CK_API int ck_moe_gather_rows_scaled(const void *src, void *dst, const int32_t *idx, const void *coeff,
                                     int64_t n_rows, int fan_out, int64_t cols, int dtype, void *stream);
CK_API int ck_moe_combine_rows(const void *src, const int32_t *pos, const void *w, void *out, int64_t tokens,
                               int k, int64_t cols, int dtype, void *stream);
CK_API int ck_moe_row_dots(const void *a, const int32_t *pos, const void *b, void *dots, int64_t n, int k,
                           int64_t cols, int dtype, void *stream);

/* ---- RMSNorm / fused residual-add + RMSNorm ----------------------------------------------------------
 * Replace rmsnorm_cute and fused_residual_add_rmsnorm_cute (kernels/rmsnorm/__init__.py:12-77,
 * kernels/fused_residual_add_rmsnorm/__init__.py:15-132: Triton forward / backward kernels) with the math of
 * rmsnorm_torch / fused_residual_add_rmsnorm_torch (the torch_implementation.py next to each).  Rows of H
 * contiguous elements, `rows` of them; weight [H] or NULL; all statistics in fp32.
 * ck_rmsnorm_fwd:  a = residual ? x * multiplier + residual : x  (stored to added_out when given, else not kept);
 *   r = rsqrt(mean(a^2) + eps), stored to inv_rms_out [rows] fp32 when given; out = a * r * weight.
 * ck_rmsnorm_bwd:  `a` is what the forward normalised (x, or added_out); g = dy * weight;
 *   da = r * g - a * r^3 * mean(g * a) (+ d_added when given: the gradient arriving through the residual stream);
 *   d_residual = da (when given), dx = da * multiplier; d_weight [H] (in `dtype`, fully overwritten) = sum over rows of
 *   dy * a * r: every block of the backward kernel stores its share as one row of dw_partial
 *   (fp32 [ck_rmsnorm_bwd_parts(rows, H), H], caller-owned, needs no initialisation) and a second kernel adds the rows
 *   in a fixed order -- reproducible, where the reference accumulates with tl.atomic_add.  d_weight NULL: no weight
 *   gradient, dw_partial unused.  inv_rms NULL: r is recomputed from `a` (memory_efficient=True upstream).
 * Pass multiplier = 1 where the reference passes None. */
CK_API int ck_rmsnorm_fwd(const void *x, const void *residual, const void *weight, void *out, void *added_out,
                          float *inv_rms_out, int64_t rows, int64_t H, float eps, float multiplier, int dtype,
                          void *stream);
CK_API int64_t ck_rmsnorm_bwd_parts(int64_t rows, int64_t H);
CK_API int ck_rmsnorm_bwd(const void *a, const void *weight, const void *dy, const void *d_added, const float *inv_rms,
                          void *dx, void *d_residual, float *dw_partial, void *d_weight, int64_t rows, int64_t H,
                          float eps, float multiplier, int dtype, void *stream);

/* ---- router tail --------------------------------------------------------------------------------
 * ck_router_topk_softmax: for each token, the k largest of its E gate logits (descending; ties to the lower
 *   expert index), weights = softmax over those k logits computed in fp32 and rounded to `dtype`, ids as int32
 *   [tokens, k] -- MoE_Torch._compute_routing_weights after the gate projection
 *   (kernels/scattermoe/torch_implementation.py:122-135 with _get_topk :195-201), one launch instead of
 *   topk + softmax + type_as, and ids already in the form ck_route reads.  E <= 256, k <= 32 else CK_ERR_RANGE.
 * ck_router_topk_softmax_bwd: d_logits [tokens, E] = scatter of the softmax backward
 *   w_j * (dw_j - sum_i w_i dw_i) at ids, zeros elsewhere (what autograd derives for the same three torch ops).
 *   An id outside [0, E) is skipped and sets CK_DEV_RANGE in *dev_status (may be NULL).
 * NaN logits count as the greatest value (torch.topk's order), so every row yields k distinct ids in [0, E). */
CK_API int ck_router_topk_softmax(const void *logits, void *weights, int32_t *ids, int64_t tokens, int E, int k,
                                  int dtype, void *stream);
CK_API int ck_router_topk_softmax_bwd(const void *weights, const void *d_weights, const int32_t *ids,
                                      void *d_logits, int64_t tokens, int E, int k, int dtype, int32_t *dev_status,
                                      void *stream);

/* ck_router_gate_topk_softmax: the gate projection and the router tail in ONE tcgen05 launch.
 *   logits[t, :] = x[t, :] @ gate_w^T  (x [tokens, H], gate_w [E, H], fp32 accumulation, rounded to `dtype`: what
 *   F.linear returns), written out because the module returns them, and -- from the same accumulator row, in the GEMM
 *   epilogue -- weights [tokens, k] and ids [tokens, k] exactly as ck_router_topk_softmax computes them from those rounded
 *   logits.  Replaces self.gate(x) + topk + softmax + type_as (torch_implementation.py:122-135,195-201): the [tokens, E]
 *   logits are not re-read and no int64 ids exist.  H % 8 == 0, E % 8 == 0, E <= 256, k <= 8 and k <= E, 16-bit dtypes
 *   (CK_ERR_UNSUPPORTED for fp32: its logits would come out of a TF32 product); other shapes take the two-step path.
 *   The backward is ck_router_topk_softmax_bwd followed by the two library GEMMs of a linear layer. */
CK_API int ck_router_gate_topk_softmax(const void *x, const void *gate_w, void *logits, void *weights, int32_t *ids,
                                       int64_t tokens, int H, int E, int top_k, int dtype, int32_t *dev_status,
                                       void *stream);

/* ---- expert parallelism over peer memory ------------------------------------------------------------
 * No reference counterpart (the reference is single-GPU); per rank these are its `group` (ops.py:108-140) and
 * `scatter2scatter` with y_grouped=False (ops.py:31-78) with the other side of the permutation living on another
 * GPU.  Every rank exposes buffers of `rows_per_peer` slots; a routed row is named by its global flat slot
 * g = rank * rows_per_peer + f, f = token * k + j on the owning rank.  `peer_*` are HOST arrays of `n_peers`
 * device pointers (rank r's buffer as mapped into this process; entry [own rank] is the local buffer), all
 * 16-byte aligned, n_peers <= CK_MAX_PEERS, n_peers * rows_per_peer < 2^31.  The kernels never wait on another
 * GPU; the host orders the phases with stream-ordered collectives.
 * ck_moe_gather_rows_peer: dst[p, :] = peer_src[g / S][(g % S) / fan_out, :], g = src_flat[row_map[p]] (row_map[p]
 *   itself when src_flat is NULL: the ids of all ranks were routed as one array), zeros where row_map[p] < 0,
 *   for p in [row_begin, min(row_end, padded_off[E])): a window of the padded rows, so that a caller can pull one
 *   part while a GEMM already runs on another.
 * ck_moe_grouped_linear_scatter_peer: ck_moe_grouped_linear_scatter whose row row_map[p] is stored at
 *   peer_out[g / S] + (g % S) * N, g = dst_flat[row_map[p]] or row_map[p] when dst_flat is NULL
 *   (rows_per_peer <= 2^26).
 * ck_peer_gather_scalars: dst[j] = peer_src[g / S][g % S], g = flat[j].
 * ck_peer_scatter_scalars: peer_dst[g / S][g % S] = by_slot ? vals[g] : vals[j], g = flat[j], entries with g < 0
 *   skipped.  Both for 2- or 4-byte scalars (router weights and their gradients).
 * A slot outside [0, n_peers * S) is skipped and sets CK_DEV_RANGE in *dev_status. */
#define CK_MAX_PEERS 16
CK_API int ck_moe_gather_rows_peer(const void *const *peer_src, int n_peers, int64_t rows_per_peer, void *dst,
                                   const int32_t *row_map, const int32_t *padded_off, const int32_t *src_flat, int E,
                                   int64_t cap, int fan_out, int64_t cols, int64_t row_begin, int64_t row_end,
                                   int dtype, int32_t *dev_status, void *stream);
/* ck_moe_up_act_fwd_gather / ck_moe_dgrad_down_gather with the rows living on the ranks that own them: padded row p
 * reads row (g % S) / fan_out of peer_src[g / S], g = row_map[p] a global flat slot (the routing pass ran over all
 * ranks' slots).  The producer warps of the GEMM issue the NVLink loads (cp.async, 16 bytes per lane) tile by tile
 * while the tensor cores work on earlier stages; no TMA touches peer memory.  rows_out (xg_out / dyg_out) keeps the
 * pulled rows on this GPU for the weight-gradient GEMMs, so every row crosses NVLink once.  CTA-pair kernels only. */
CK_API int ck_moe_up_act_fwd_gather_peer(const void *const *peer_src, int n_peers, int64_t rows_per_peer, int fan_out,
                                         const void *wfc, const void *gate_w, const int32_t *row_map,
                                         const int32_t *mtile_off, void *act, void *h, void *xg_out, int E, int64_t cap,
                                         int H, int I, int act_kind, int dtype, int32_t *dev_status, void *stream);
CK_API int ck_moe_dgrad_down_gather_peer(const void *const *peer_src, int n_peers, int64_t rows_per_peer, int fan_out,
                                         const void *wproj, const void *h, const void *gate_w, const int32_t *row_map,
                                         const int32_t *mtile_off, void *dh, float *dgates, float *dgates_part,
                                         void *dyg_out, int E, int64_t cap, int H, int I, int act_kind, int dtype,
                                         int32_t *dev_status, void *stream);
CK_API int ck_moe_grouped_linear_scatter_peer(const void *x, const void *w, const int32_t *mtile_off,
                                              const int32_t *row_map, const int32_t *dst_flat, void *const *peer_out,
                                              int n_peers, int64_t rows_per_peer, int E, int64_t cap, int N, int K,
                                              int trans_w, int dtype, int32_t *dev_status, void *stream);
CK_API int ck_peer_gather_scalars(const void *const *peer_src, int n_peers, int64_t rows_per_peer,
                                  const int32_t *flat, int64_t n, void *dst, int elem_bytes, int32_t *dev_status,
                                  void *stream);
CK_API int ck_peer_scatter_scalars(const void *vals, const int32_t *flat, int64_t n, int by_slot,
                                   void *const *peer_dst, int n_peers, int64_t rows_per_peer, int elem_bytes,
                                   int32_t *dev_status, void *stream);

/* ---- self test of the bounded device waits -----------------------------------------------------------
 * No reference counterpart (the reference's kernels have no device-side waits).  Every mbarrier wait of the grouped
 * GEMMs polls with a wall-clock limit; when it runs out the CTA sets CK_DEV_TIMEOUT in *dev_status, leaves its
 * loops, frees TMEM and returns.  ck_test_wait_timeout runs that same wait routine in a one-CTA kernel on a barrier
 * nobody arrives at, with `limit_ns` (1 .. 100,000,000; else CK_ERR_RANGE) as the limit, so the abort path can be
 * exercised without a broken pipeline.  result4[0], [1]: what the two waiting lanes returned (0 = gave up),
 * result4[2]: nanoseconds the first lane waited (saturating), result4[3]: the CTA's abort flag.  The launch ends by
 * itself after about `limit_ns`; the context stays usable. */
CK_API int ck_test_wait_timeout(int64_t limit_ns, int32_t *result4, int32_t *dev_status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CK_B200_H */
