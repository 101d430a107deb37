/*
 * ixb - C ABI of the B200 (sm_100a) kernel library behind the inductor_x_b200 backend.
 *
 * Every entry point is extern "C", takes plain device pointers, sizes and a CUDA stream
 * handle (passed as void*), enqueues work on that stream and returns without
 * synchronising.  Return value: 0 (IXB_OK) or an ixb_status code; nothing throws or
 * aborts.  The caller owns every buffer; the library allocates no device memory.
 * Re-entrant: the only global state is a per-device attribute cache filled once.
 *
 * This boundary takes the place of the launcher the reference builds around each
 * compiled Triton kernel, `launcher(*args, grid=grid, stream=stream)` called as
 * `bin[grid](...)` (inductor_x/npu_triton_heuristics.py:239-253), and of the vendor
 * fused-attention call (inductor_x/npu_fusion_attention_graph.py:31).  Each declaration
 * names the reference code it stands in for.
 */
#ifndef IXB_H_
#define IXB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IXB_ABI_VERSION 1

typedef void* ixb_stream; /* cudaStream_t */

typedef enum ixb_status {
  IXB_OK = 0,
  IXB_ERR_ARG = 1,         /* null pointer, negative size, unknown enum value */
  IXB_ERR_DTYPE = 2,       /* dtype not supported by this entry point */
  IXB_ERR_ALIGN = 3,       /* pointer or stride not aligned as documented */
  IXB_ERR_SHAPE = 4,       /* extent outside what the kernel family supports */
  IXB_ERR_UNSUPPORTED = 5, /* no instantiated kernel for this configuration */
  IXB_ERR_SCRATCH = 6,     /* caller-provided scratch too small or missing */
  IXB_ERR_CUDA = 7,        /* CUDA runtime error; see ixb_last_cuda_error() */
  IXB_ERR_INDEX = 8        /* reported by ixb_check_index_status */
} ixb_status;

typedef enum ixb_dtype {
  IXB_F32 = 0,
  IXB_F16 = 1,
  IXB_BF16 = 2,
  IXB_I64 = 3,
  IXB_I32 = 4,
  IXB_U8 = 5
} ixb_dtype;

/* Reduction kinds: the set the reference's kernel emitter handles
 * (inductor_x/codegen/triton.py:1103-1262). */
typedef enum ixb_reduce {
  IXB_SUM = 0,
  IXB_MEAN = 1,
  IXB_AMAX = 2,
  IXB_AMIN = 3,
  IXB_ARGMAX = 4,
  IXB_ARGMIN = 5,
  IXB_VAR_MEAN = 6
} ixb_reduce;

/* Kernel families = the template each fused node group is instantiated from; they
 * correspond to the decorators the reference emits, pointwise_npu_index /
 * reduction_npu_index / persistent_reduction_npu_index
 * (inductor_x/npu_triton_heuristics.py:545-611). */
typedef enum ixb_family {
  IXB_FAM_POINTWISE = 0,
  IXB_FAM_ROW = 1,       /* reduced axis is stride-1 and held on chip */
  IXB_FAM_OUTER = 2,     /* reduced axis is not stride-1 */
  IXB_FAM_SHORT_ROW = 3, /* stride-1 reduced axis of <= 512 bytes, permuted store */
  IXB_FAM_GATHER = 4
} ixb_family;

/* Device facts the launch chooser works from; replaces num_vector_core / npu_block of
 * inductor_x/config.py:15-28 and the byte table of inductor_x/codegen/triton_utils.py:6-27. */
typedef struct ixb_devinfo {
  int32_t sm_count;
  int32_t cc_major;
  int32_t cc_minor;
  int32_t max_threads_per_sm;
  int64_t l2_bytes;
  int64_t smem_per_block_optin;
  int64_t global_mem_bytes;
  int32_t vector_bytes; /* 16: width of one coalesced access per thread */
  int32_t reserved;
} ixb_devinfo;

/* A launch configuration.  Zero-initialised = "let the library choose". */
typedef struct ixb_cfg {
  int32_t team;    /* threads cooperating on one row (ROW family): 32..1024 */
  int32_t vpt;     /* 128-bit vectors per thread and row: 1, 2, 4 or 8 */
  int32_t grid;    /* CTAs; 0 = persistent grid sized from occupancy */
  int32_t rsplit;  /* OUTER family: segments of the reduced axis (needs scratch if > 1) */
  int32_t threads; /* CTA size where the family allows a choice */
  int32_t unroll;  /* independent loads in flight per thread */
  int32_t reserved[2];
} ixb_cfg;

/* What the chooser needs to know about a problem. */
typedef struct ixb_problem {
  int32_t family;    /* ixb_family */
  int32_t dtype;     /* ixb_dtype of the dominant input */
  int64_t outer;     /* rows (ROW), outer extent (OUTER), gathered rows (GATHER) */
  int64_t reduce;    /* reduced extent (ROW: row length; OUTER: R) */
  int64_t inner;     /* stride-1 kept extent (OUTER), row bytes (GATHER) */
  int32_t row_inputs;/* ROW: number of row-shaped inputs streamed per row */
  int32_t aligned;   /* 1 if every base pointer and row pitch is 16-byte aligned */
} ixb_problem;

/* ---- library ------------------------------------------------------------------- */
int ixb_abi_version(void);
const char* ixb_strerror(int status);
/* Message of the last CUDA runtime error seen by the calling thread ("" if none). */
const char* ixb_last_cuda_error(void);
/* Attributes of CUDA device `device` (-1 = current). */
int ixb_device_info(int device, ixb_devinfo* out);

/* Launch-config and split-factor chooser.  Stands in for SplitTiling.select_split_axis /
 * select_tiling_axis / decide_nblocks_xblock (inductor_x/codegen/split_tiling.py:46-182),
 * TileGenerator (inductor_x/codegen/tile_generator.py:10-136), triton_config_npu_index
 * and grid (inductor_x/npu_triton_heuristics.py:444-544).  Pure host arithmetic. */
int ixb_choose_config(const ixb_problem* problem, const ixb_devinfo* dev, ixb_cfg* out);

/* ---- ROW family: fused graphs with the reduced axis held in registers ------------ */

/* out[r] = sum_c gelu_erf(x[r,c]*w[c] + b[c]); fp32.  One kernel for what the reference
 * runs as mul+add, an extern gelu and a sum (inductor_x/lowering.py:185-215,251-268). */
int ixb_affine_gelu_rowsum_f32(const float* x, const float* w, const float* b, float* out,
                               int64_t rows, int64_t cols, const ixb_cfg* cfg, ixb_stream stream);

/* y = layer_norm(softmax(x,-1)*g + x, gamma, beta, eps) over the last axis; dtype F16,
 * BF16 or F32 for all tensors, fp32 arithmetic.  Replaces the looped multi-pass reduction
 * kernels of inductor_x/codegen/triton.py:1208-1253 and the two-pass var_mean lowering
 * (inductor_x/lowering.py:217-233,270-325). */
int ixb_softmax_layernorm(int dtype, const void* x, const void* g, const void* gamma,
                          const void* beta, void* y, int64_t rows, int64_t cols, float eps,
                          const ixb_cfg* cfg, ixb_stream stream);

/* RMSNorm: h = x (+ res); y = h * rsqrt(mean(h*h) + eps) * w.  res and h_out may be null.
 * (mean lowering: inductor_x/lowering.py:217-233.) */
int ixb_rmsnorm(int dtype, const void* x, const void* res, const void* w, void* y, void* h_out,
                int64_t rows, int64_t cols, float eps, const ixb_cfg* cfg, ixb_stream stream);

/* Reduce the last (stride-1) axis of contiguous x[rows, cols].
 * kind SUM/MEAN/AMAX/AMIN: out[rows] in x's dtype (fp32 accumulation, unlike the
 * reference's sum_ which always returns fp32, inductor_x/lowering.py:204-215).
 * ARGMAX/ARGMIN: out is int64[rows].  VAR_MEAN: out = var[rows], out2 = mean[rows],
 * `correction` as in torch.var_mean.  (inductor_x/codegen/triton.py:1163-1253.) */
int ixb_row_reduce(int dtype, int kind, const void* x, void* out, void* out2, int64_t rows,
                   int64_t cols, float correction, const ixb_cfg* cfg, ixb_stream stream);

/* ---- OUTER family ------------------------------------------------------------------ */

/* Bytes of fp32 scratch ixb_outer_reduce needs for this problem with this rsplit
 * (0 when rsplit <= 1). */
size_t ixb_outer_reduce_scratch_bytes(int64_t outer, int64_t inner, int rsplit);

/* out[o, i] = reduce_r x[o, r, i] for contiguous x[outer, R, inner]; kind SUM/MEAN/AMAX/
 * AMIN.  With cfg->rsplit > 1 the reduced axis is cut into segments whose partials go to
 * `scratch` and are folded by a second launch - the deterministic counterpart of the
 * reference's atomic_add outer split (inductor_x/codegen/split_tiling.py:159-165,
 * inductor_x/codegen/triton.py:904-905,1003-1031). */
int ixb_outer_reduce(int dtype, int kind, const void* x, void* out, int64_t outer, int64_t R,
                     int64_t inner, void* scratch, size_t scratch_bytes, const ixb_cfg* cfg,
                     ixb_stream stream);

/* Capacity of the built-in scratch used by ixb_outer_reduce_static. */
#define IXB_STATIC_SCRATCH_BYTES (4u * 1024u * 1024u)

/* No counterpart in the reference: an addition for callers that cannot allocate.
 * Same result as ixb_outer_reduce with cfg->rsplit = rsplit, but the fp32 partials of
 * the split go to a fixed IXB_STATIC_SCRATCH_BYTES array that is part of the library
 * image (each GPU that loads the library holds those 4 MiB until the process exits), so
 * neither the caller nor the library allocates anything.  It is meant for code that runs
 * where a device allocation is off the table: a wrapper whose buffers were all planned
 * and reserved ahead of time, a serving loop in which cudaMalloc would stall every
 * stream of the device, or a process whose GPU memory is already owned by a caching
 * allocator so that a raw allocation may simply fail.
 *   - outer * inner * rsplit * 4 must not exceed IXB_STATIC_SCRATCH_BYTES, otherwise
 *     IXB_ERR_SCRATCH is returned and nothing is launched; x must be 16-byte aligned
 *     and inner a multiple of 16 bytes (IXB_ERR_ALIGN otherwise); rsplit >= 1.
 *   - The first call on each device looks up the array's device address (with that
 *     device current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array.  Every launch overwrites the partials
 *     it later reads, so nothing needs clearing between calls, but two calls whose
 *     kernels overlap on the GPU (different streams, no ordering) race on it: keep
 *     calls on one stream or order them with events. */
int ixb_outer_reduce_static(int dtype, int kind, const void* x, void* out, int64_t outer,
                            int64_t R, int64_t inner, int rsplit, ixb_stream stream);

/* ---- SHORT_ROW family ------------------------------------------------------------- */

/* x contiguous [A,B,C,L]; the stride-1 axis L (L*elsize a power-of-two multiple of 16 up
 * to 512 bytes) is reduced and the result stored at out[a*sa + b*sb + c*sc] (strides in
 * elements).  sb == 1 is the transposed store the reference emits through `_prime` index
 * variables and a tile permute (inductor_x/codegen/triton.py:856-914,1303-1332). */
int ixb_short_row_reduce(int dtype, int kind, const void* x, void* out, int64_t A, int64_t B,
                         int64_t C, int64_t L, int64_t sa, int64_t sb, int64_t sc,
                         ixb_stream stream);

/* ---- GATHER family ------------------------------------------------------------------ */

/* out[m, :] = table[idx[m], :], rows of row_bytes bytes, table row pitch
 * table_pitch_bytes; idx_dtype IXB_I64 or IXB_I32.  Bit-exact for any element type.
 * wrap_negative != 0 adds n_rows to negative indices.  `status` is null or two device
 * ints zeroed by the caller: an out-of-range index sets status[0]=1, status[1]=position,
 * and zero-fills that row (contract of the reference's indirect loads,
 * inductor_x/codegen/triton.py:1666-1710; the reference itself routes index_select to an
 * extern kernel, inductor_x/lowering.py:89-144,185-198). */
int ixb_index_select_rows(const void* table, const void* idx, void* out, int64_t n_rows,
                          int64_t m, int64_t row_bytes, int64_t table_pitch_bytes, int idx_dtype,
                          int wrap_negative, int32_t* status, ixb_stream stream);

/* ---- fused attention ----------------------------------------------------------------- */

/* out = softmax(q k^T * scale [+ causal mask]) v for q[B,H,Sq,D], k/v[B,H,Sk,D], D = 128,
 * dtype F16 or BF16, fp32 accumulation; lse[B,H,Sq] (fp32, natural log of the softmax
 * denominator times exp of the row maximum, i.e. logsumexp of the scaled scores) may be
 * NULL.  *_strides = element strides of the (batch, head, sequence) axes; the D axis must
 * be contiguous and every stride a multiple of 8 elements, so both the reference's BNSD
 * layout and a transposed BSND view are taken without a copy.  causal != 0 masks key j
 * for query i when j > i + (Sk - Sq) and requires Sk >= Sq.  `status` is NULL or a device
 * word zeroed by the caller; it is set to 1 if an internal wait gave up (results are then
 * undefined).  Stands in for the vendor call torch_npu.npu_fusion_attention behind
 * npu_graph::npu_fa (inductor_x/npu_fusion_attention_graph.py:20-35); note that entry
 * takes the softmax multiplier itself, whereas the reference passes inv_scale and inverts
 * it inside the op (inductor_x/npu_fusion_attention_graph.py:22-29,162). */
int ixb_fa_fwd(int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
               int32_t B, int32_t H, int32_t Sq, int32_t Sk, int32_t D, const int64_t* q_strides,
               const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
               float scale, int causal, int32_t* status, ixb_stream stream);

/* Gradients of ixb_fa_fwd: dq[B,H,Sq,D], dk/dv[B,H,Sk,D] from q, k, v, the forward's
 * output `o` and log-sum-exp `lse` [B,H,Sq] (fp32, contiguous) and the incoming gradient
 * `dout` [B,H,Sq,D]; same dtype, stride and alignment rules as ixb_fa_fwd for all eight
 * tensors, same meaning of `scale`, `causal` and `status`.  `delta` is caller-provided
 * scratch of B*H*Sq floats (it receives rowsum(dout * o)); nothing is allocated and no
 * atomics are used, so the result is deterministic.  Stands in for the vendor call
 * torch_npu.npu_fusion_attention_grad behind npu_graph::npu_fa_backward
 * (inductor_x/npu_fusion_attention_graph.py:38-42). */
int ixb_fa_bwd(int dtype, const void* q, const void* k, const void* v, const void* o,
               const void* dout, const float* lse, void* dq, void* dk, void* dv, float* delta,
               int32_t B, int32_t H, int32_t Sq, int32_t Sk, int32_t D, const int64_t* q_strides,
               const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
               const int64_t* do_strides, const int64_t* dq_strides, const int64_t* dk_strides,
               const int64_t* dv_strides, float scale, int causal, int32_t* status,
               ixb_stream stream);

/* ---- context-parallel attention merge ---------------------------------------------------- */

/* Fold the partial attention result of one ring step into the running one, (max, sum) form:
 *   m = max(pm, cm); ps = psum*exp(pm-m); cs = csum*exp(cm-m); l = ps+cs;
 *   out_attn = prev_attn*(ps/l) + cur_attn*(cs/l); out_max = m; out_sum = l
 * attn tensors [S, B, N*D] contiguous, dtype F32/F16/BF16 (fp32 math); statistics
 * [B, N, S, 8] fp32 whose N axis has the given element stride (so a slice along S of a longer
 * buffer can be passed), updated entry by entry; the attention weights use entry 0.
 * D*elsize must be a multiple of 16 and all pointers 16-byte aligned.  Replaces the
 * hand-written kernel tl_fn_forward_update
 * (test/npu_indexing/written/attn_cp_triton_kernel_3d.py:15-82; eager form
 * test/npu_indexing/attn_cp_test.py:36-59). */
int ixb_cp_forward_update(int dtype, const void* prev_attn, const float* prev_max,
                          const float* prev_sum, const void* cur_attn, const float* cur_max,
                          const float* cur_sum, void* out_attn, float* out_max, float* out_sum,
                          int32_t S, int32_t B, int32_t N, int32_t D, int64_t prev_stat_nstride,
                          int64_t cur_stat_nstride, int64_t out_stat_nstride, ixb_stream stream);

/* Log-sum-exp form, in place on the running result:
 *   lse = log(exp(p)+exp(c)); prev_attn = exp(p-lse)*prev_attn + exp(c-lse)*cur_attn; prev_lse = lse
 * attn [B, N, S, D] fp32 and lse [B, N, S] fp32, each with an element stride for its N axis;
 * D a multiple of 4, attn pointers and strides 16-byte aligned.  Replaces
 * tl_fn_forward_update_la (test/npu_indexing/written/attn_cp_triton_kernel_3d_la.py:11-55). */
int ixb_cp_forward_update_lse(float* prev_attn, float* prev_lse, const float* cur_attn,
                              const float* cur_lse, int32_t B, int32_t N, int32_t S, int32_t D,
                              int64_t prev_attn_nstride, int64_t prev_lse_nstride,
                              int64_t cur_attn_nstride, int64_t cur_lse_nstride, ixb_stream stream);

/* acc += cur over numel contiguous elements (fp32 add, rounded to the storage type): the
 * gradient accumulation of the ring backward (backward_update,
 * test/npu_indexing/written/test_attn_cp.py:267-287).  numel*elsize a multiple of 16. */
int ixb_cp_accumulate(int dtype, void* acc, const void* cur, int64_t numel, ixb_stream stream);

/* ---- generated modules ------------------------------------------------------------------
 * Every module the code generator builds (one per fused node group, compiled with nvcc for
 * sm_100a and cached as a shared object) exports the same two C symbols; they are what the
 * reference's launcher closure `launcher(*args, grid, stream)`
 * (inductor_x/npu_triton_heuristics.py:239-253) becomes.  They are not symbols of libixb.so,
 * so they are given here as function-pointer types for a host that loads such a module itself:
 *
 *   launch : ptrs = the tensor arguments in call order (device pointers), ints = the size
 *            arguments in call order followed by the kept extent (and, for a row kernel with a
 *            run-time reduced extent, that extent), stream = cudaStream_t.  Returns 0 or a
 *            cudaError_t value; enqueues and returns.
 *   bounds : only in modules generated with bounds checks (debug builds): copies out and
 *            clears {number of out-of-range data-dependent indices, one offending value};
 *            synchronises the device.  Returns 0 or a cudaError_t value. */
typedef int (*ixb_gen_launch_fn)(void** ptrs, const long long* ints, void* stream);
typedef int (*ixb_gen_bounds_fn)(unsigned long long* out);
#define IXB_GEN_LAUNCH_SYMBOL "ixb_gen_launch"
#define IXB_GEN_BOUNDS_SYMBOL "ixb_gen_bounds"

#ifdef __cplusplus
}
#endif
#endif /* IXB_H_ */
