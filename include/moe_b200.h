/*
 * moe_b200.h -- C ABI of libmoe_b200.so: the MoE hot path of triton_kernels as hand-written
 * CUDA for sm_100a (B200).
 *
 * Conventions
 *   - Every entry point returns 0 on success and a non-zero MOE_ERR_* code otherwise; it never
 *     throws and never traps.  moe_last_error() returns a per-thread message for the last failure.
 *   - All pointers are DEVICE pointers unless the name ends in _host.  Nothing here allocates
 *     device memory: outputs and scratch are owned by the caller (the Python shim allocates them
 *     through torch).  Work is enqueued on `stream` (a cudaStream_t passed as void*), without
 *     host synchronisation, so calls can be captured in a CUDA graph.
 *   - "Reference" citations are paths inside triton-lang/triton, python/triton_kernels/triton_kernels/.
 */
#ifndef MOE_B200_H
#define MOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MOE_F32 = 0, MOE_F16 = 1, MOE_BF16 = 2, MOE_F8E4M3 = 3 /* activations of the block-scaled GEMM only */ };
enum { MOE_OK = 0, MOE_ERR_ARG = 1, MOE_ERR_CUDA = 2, MOE_ERR_UNSUPPORTED = 3, MOE_ERR_DEVICE_STATUS = 4 };
enum { MOE_ROUND_UP = 0, MOE_ROUND_DOWN = 1 };
enum { MOE_ACT_NONE = 0, MOE_ACT_SWIGLU = 1 };
/* weight kinds understood by moe_grouped_gemm */
enum { MOE_W_DENSE = 0,          /* w[e,k,n] in the activation dtype, arbitrary element strides */
       MOE_W_MX4_CANONICAL = 1,  /* e2m1x2 bytes packed along K (K contiguous) + e8m0 scales, byte strides */
       MOE_W_MX4_B200 = 2,       /* tile-contiguous values + scales made by moe_weight_layout_to_b200 */
       MOE_W_MX4_B200MX = 3      /* tiles for the block-scaled MMA made by moe_weight_layout_to_b200mx */ };
#define MOE_MAX_PEERS 16
enum { MOE_GEMM_AUTO = 0, MOE_GEMM_SIMT = 1, MOE_GEMM_TCGEN05 = 2, MOE_GEMM_TCGEN05_PAIR = 3, MOE_GEMM_STREAM = 4,
       MOE_GEMM_MX = 5,          /* block-scaled kernel; bf16 tokens in the form it picks by block size */
       MOE_GEMM_MX_F8 = 6,       /* ... bf16 tokens as two e4m3 terms (kind::mxf8f6f4) */
       MOE_GEMM_MX_F4 = 7 };     /* ... bf16 tokens as four e2m1 terms (kind::mxf4), blocks of at most 32 rows */

const char* moe_last_error(void);
int moe_abi_version(void);
/* Kernels this library has launched in the calling process so far (every launch site counts itself).  Callers
 * use differences of it, e.g. to count the launches of one step. */
uint64_t moe_launch_count(void);

/* Device facts used by the host-side heuristics (replaces target_info.py:73-74 num_sms()). */
typedef struct {
  int sm_count;
  int cc_major, cc_minor;
  size_t smem_per_block_optin;
  size_t l2_bytes;
  size_t total_mem;
} MoeDeviceInfo;
int moe_device_info(int device, MoeDeviceInfo* out_host);

/* ---- MXFP4 quantiser / dequantiser -------------------------------------------------------------
 * Replaces numerics_details/mxfp.py:25-88 (downcast_to_mxfp -> _downcast_to_mxfp kernel,
 * mxfp_details/_downcast_to_mxfp.py:149-215) and mxfp.py:90-176 (upcast_from_mxfp ->
 * mxfp_details/_upcast_from_mxfp.py:109-220) for e2m1 values with e8m0 scales per 32 elements.
 * The source is viewed as [batch, outer, quant] with element strides; quant % 32 == 0.
 * q is [batch, outer, quant/2] bytes and scale [batch, outer, quant/32] bytes, both dense.       */
int moe_downcast_mxfp4(const void* x, int src_dtype, int64_t batch, int64_t outer, int64_t quant,
                       int64_t sx_batch, int64_t sx_outer, int64_t sx_quant,
                       uint8_t* q, uint8_t* scale, int rounding_mode, void* stream);
/* out is viewed as [batch, outer, quant] with element strides; q/scale dense as above. */
int moe_upcast_mxfp4(const uint8_t* q, const uint8_t* scale, void* out, int dst_dtype,
                     int64_t batch, int64_t outer, int64_t quant,
                     int64_t so_batch, int64_t so_outer, int64_t so_quant, void* stream);

/* ---- routing -----------------------------------------------------------------------------------
 * moe_topk_fwd replaces topk.py:25-73 (topk_forward -> topk_details/_topk_forward.py:91-150):
 * per row the k largest logits (ties -> smaller index), sorted descending, optional fp32 softmax
 * over the selected k, and the row of the expert bitmatrix.  indx is int16 [T,k]; bitmatrix word
 * (t, w) lives at bitmatrix[t*bm_stride_row + w*bm_stride_word].  Rows >= *n_rows_dev (or >= T if
 * NULL) are left untouched.  With use_provided_indx, indx is an input.                             */
int moe_topk_fwd(const void* logits, int dtype, int64_t T, int E, int k, int apply_softmax,
                 int64_t ld_logits, void* vals, int64_t ld_vals, int16_t* indx, int64_t ld_indx,
                 uint32_t* bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word,
                 const int32_t* n_rows_dev, int use_provided_indx, void* stream);

/* Replaces tensor_details/bitmatrix.py:110-150 (make_bitmatrix_metadata: sum_bitmatrix_rows +
 * stage1 + stage2): histogram col_sum[E], col_sorted_indx[T*k], row_sorted_indx[T*k] (stable
 * counting sort of the flat (token,slot) entries by expert; -1 padded).
 * workspace: moe_bitmatrix_metadata_workspace(T, E, k) bytes of device scratch.                    */
size_t moe_bitmatrix_metadata_workspace(int64_t T, int E, int k);
int moe_bitmatrix_metadata(const int16_t* indx, int64_t ld_indx, int64_t T, int E, int k,
                           const int32_t* n_rows_dev, int32_t* col_sum, int32_t* col_sorted,
                           int32_t* row_sorted, void* workspace, size_t workspace_bytes, void* stream);

/* The whole routing step of a layer in three launches (one for up to 256 tokens): moe_topk_fwd +
 * moe_bitmatrix_metadata + moe_ragged_metadata (topk.py:106-141 -> tensor.py:202-209 -> ragged_tensor.py:183-210 of the
 * reference, what its test helper `routing` composes, tests/test_distributed.py:203-210) with the expert histogram taken
 * in the top-k pass and the ragged metadata built beside the scan of the histograms.  Every one of the T rows is valid (no device-side row
 * bound, no provided indices); n_expts <= 256, otherwise MOE_ERR_UNSUPPORTED and the caller uses the separate entry
 * points.  Outputs as for those entry points; workspace of moe_route_workspace(T, n_expts, k) bytes.               */
size_t moe_route_workspace(int64_t T, int E, int k);
int moe_route(const void* logits, int dtype, int64_t T, int E, int k, int apply_softmax, int64_t ld_logits,
              void* vals, int64_t ld_vals, int16_t* indx, int64_t ld_indx,
              uint32_t* bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word,
              int32_t* col_sum, int32_t* col_sorted, int32_t* row_sorted,
              int32_t* slice_offs, int32_t* block_offs, int64_t ld_block_offs,
              int32_t* block_sched, int64_t ld_sched, int64_t n_sched,
              void* workspace, size_t workspace_bytes, void* stream);

/* The router product and the top-k selection in one kernel: logits = x @ Wg + bg on the tensor cores, then what
 * moe_topk_fwd does, in the epilogue (the reference runs `matmul(x, wg, bg)` and `topk` apart:
 * triton_kernels bench/bench_mlp.py:70, topk.py:25-141).
 *   x [T, K] bf16, row pitch ld_x; wg_t = Wg transposed, [E, K] bf16 with K contiguous, row pitch ld_wg (a [K, E] tensor
 *   whose stride along K is 1); bias [E] fp32 or bf16, may be NULL; E <= 256; k in {1, 2, 4, 8, 16}; K, ld_x, ld_wg
 *   multiples of 8 -- otherwise MOE_ERR_UNSUPPORTED and the caller runs the two steps apart.
 *   round_bf16: round every logit to bf16 before the selection (what a bf16 router output does in the two-step form).
 *   logits_out: NULL, or [T, E] fp32 that receives the logits the selection saw.
 *   vals [T, k] fp32 or bf16, indx, bitmatrix: as for moe_topk_fwd.
 * With few tokens K is cut into slices over the SMs and the partial logits meet in `workspace`
 * (moe_router_topk_workspace_bytes, 16-byte aligned): it must be ALL ZERO when the call starts and the call leaves it
 * all zero again, so one cudaMemset after allocating it serves every later call on the same stream (calls that share a
 * workspace must not overlap; clear it again after a call that reported a device status).  The fp32 sums of the slices
 * are formed in no fixed order.  A bounded wait that expires writes 801..804 to *status.                            */
size_t moe_router_topk_workspace_bytes(int64_t T, int64_t K, int E);
int moe_router_topk(const void* x, int64_t T, int64_t K, int64_t ld_x, const void* wg_t, int64_t ld_wg,
                    const void* bias, int bias_dtype, int E, int k, int apply_softmax, int round_bf16,
                    float* logits_out, int64_t ld_logits, void* vals, int vals_dtype, int64_t ld_vals,
                    int16_t* indx, int64_t ld_indx, uint32_t* bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word,
                    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* No counterpart in the reference.  The same computation as moe_bitmatrix_metadata for callers that cannot
 * supply a workspace because they cannot allocate device memory when they call: a serving process that gave
 * all device memory to its own pools at start-up, or a latency-critical section where cudaMalloc, which
 * synchronises the device, is not acceptable.  The scratch is a fixed 1 MiB array inside the library
 * (moe_bitmatrix_metadata_noalloc_capacity() bytes, held by every GPU that loads the library until the
 * process exits); inputs and outputs are still the caller's.  It serves problems with
 * (ceil(T / 256) * E + E) * 4 <= capacity, e.g. T = 65536 tokens with E = 128 experts, or 8192 tokens with
 * E = 4096, and returns MOE_ERR_ARG with a message for anything larger.  It calls no cudaMalloc / cudaFree or
 * other allocating routine.  The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current); make that first call before any stream capture begins.
 * All calls share the one array, and it keeps whatever the previous call left (nothing in it needs to start
 * at zero): two calls whose kernels may overlap on the GPU -- different streams, no ordering between them --
 * race on it and give wrong results; order them on one stream or with events.                           */
size_t moe_bitmatrix_metadata_noalloc_capacity(void);
int moe_bitmatrix_metadata_noalloc(const int16_t* indx, int64_t ld_indx, int64_t T, int E, int k,
                                   const int32_t* n_rows_dev, int32_t* col_sum, int32_t* col_sorted,
                                   int32_t* row_sorted, void* stream);

/* Replaces tensor_details/ragged_tensor.py:183-210 (make_ragged_tensor_metadata: memset + compute
 * kernels).  block_offs is [4][ld_block_offs] (block sizes 16,32,64,128), block_sched is
 * [4][ld_sched] with n_sched valid columns each (= max_n_blocks), padded with -1.                  */
int moe_ragged_metadata(const int32_t* slice_sizes, int E, int32_t* slice_offs, int32_t* block_offs,
                        int64_t ld_block_offs, int32_t* block_sched, int64_t ld_sched, int64_t n_sched,
                        void* stream);
/* Replaces ragged_tensor.py:348-381 (remap_ragged_tensor_metadata). */
int moe_ragged_metadata_remap(const int32_t* slice_sizes, const int32_t* slice_offs, const int32_t* block_offs,
                              int64_t ld_block_offs, const int32_t* block_sched, int64_t ld_sched, int64_t n_sched,
                              const int32_t* slice_map, int E, int32_t* out_slice_sizes, int32_t* out_slice_offs,
                              int32_t* out_block_offs, int32_t* out_block_sched, void* stream);

/* ---- SwiGLU and combine ------------------------------------------------------------------------
 * Replaces swiglu.py:85-86 (swiglu -> swiglu_details/_swiglu.py:73-120): a is [M, 2*N] with gate
 * and linear columns interleaved, out is [M, N].  n_rows_dev (nullable) bounds M on the device.    */
int moe_swiglu(const void* a, int64_t ld_a, void* out, int64_t ld_out, int dtype, int64_t M, int64_t N,
               float alpha, float limit, int has_limit, const int32_t* n_rows_dev, void* stream);
/* Replaces reduce.py:1143-1165 (reduce -> _reduce_forward, reduce.py:505-650) without mx/flex
 * features: y[s0,s1] = sum_r mask * scale * x[r,s0,s1], fp32 accumulation.  Strides are in
 * elements, in the order (reduced, s0, s1); mask (any of 1/2/4/8-byte integers, 0 = skip) and
 * scale (fp32) may be NULL and may broadcast through zero strides.                                 */
int moe_reduce(const void* x, int dtype, int64_t R, int64_t S0, int64_t S1,
               int64_t sx_r, int64_t sx_0, int64_t sx_1,
               const void* mask, int mask_elem_bytes, int64_t sm_r, int64_t sm_0, int64_t sm_1,
               const float* scale, int64_t ss_r, int64_t ss_0, int64_t ss_1,
               void* y, int y_dtype, int64_t sy_0, int64_t sy_1, void* stream);

/* ---- weight layout -----------------------------------------------------------------------------
 * One-time re-layout of canonical MXFP4 weights (the output of moe_downcast_mxfp4 on w[E,K,N] along
 * K: values [E][N][K/2], scales [E][N][K/32]) into the tile-contiguous layout the tensor-core kernel
 * streams with bulk copies: tiles of 128 n x 128 k, ordered [E][n_tile][k_tile]; a value tile is
 * [4 scale groups][128 rows][16 bytes] with the nibbles of every 32-bit word reordered
 * (k0,k2,k4,k6,k1,k3,k5,k7), a scale tile is 128 rows x 4 bytes; K and N are zero-padded to multiples of 128.  Plays the role of
 * convert_layout(..., BlackwellMX4ValueShuffledLayout / BlackwellMXScaleLayout)
 * (tensor_details/layout_details/blackwell_value_shuffled.py:203-261, blackwell_scale.py:505-533).
 * Either half (values or scales) may be skipped by passing NULL for both its input and output.    */
size_t moe_weight_b200_value_bytes(int E, int K, int N);
size_t moe_weight_b200_scale_bytes(int E, int K, int N);
int moe_weight_layout_to_b200(const uint8_t* q, int64_t q_stride_e, int64_t q_stride_n,
                              const uint8_t* scale, int64_t s_stride_e, int64_t s_stride_k, int64_t s_stride_n,
                              int E, int K, int N, uint8_t* out_values, uint8_t* out_scales, void* stream);
int moe_weight_layout_from_b200(const uint8_t* values, const uint8_t* scales, int E, int K, int N,
                                uint8_t* q /* [E][N][K/2] */, uint8_t* scale /* [E][N][K/32] */, void* stream);
/* The layout the block-scaled kernel (tcgen05.mma.kind::mxf8f6f4) streams, same sizes as above
 * (moe_weight_b200_value_bytes / _scale_bytes): tiles ordered [E][k_tile][n_block]; a value tile is 128 rows x 64
 * bytes of plain packed e2m1 (the TMA unit expands it to the byte-per-element operand in shared memory), a scale
 * tile is the 128 x 4 packed block [r % 32][r / 32][group] that tcgen05.cp moves into tensor memory -- the tile of
 * BlackwellMXScaleLayout (tensor_details/layout_details/blackwell_scale.py:165-175).  out_values must be 32-byte
 * aligned.  Arguments as for moe_weight_layout_to_b200 / _from_b200.                                          */
int moe_weight_layout_to_b200mx(const uint8_t* q, int64_t q_stride_e, int64_t q_stride_n,
                                const uint8_t* scale, int64_t s_stride_e, int64_t s_stride_k, int64_t s_stride_n,
                                int E, int K, int N, uint8_t* out_values, uint8_t* out_scales, void* stream);
int moe_weight_layout_from_b200mx(const uint8_t* values, const uint8_t* scales, int E, int K, int N,
                                  uint8_t* q /* [E][N][K/2] */, uint8_t* scale /* [E][N][K/32] */, void* stream);

/* ---- ragged grouped GEMM -------------------------------------------------------------------------
 * Replaces matmul.py:245-766 (matmul -> matmul_details/_p_matmul.py:62 / _matmul.py:43):
 *   y[rows(e)] = act((x[gather(rows(e))] @ dequant(w[e]) + bias[e] * betas) * out_alpha) * gammas
 * fp32 accumulation; rows(e) = [slice_offs[e], slice_offs[e] + slice_sizes[e]).  The epilogue order
 * is that of _p_matmul.py:610-628.  Two kernels: a tcgen05 kernel (bf16 activations x
 * MOE_W_MX4_B200 weights, TMEM accumulators) and a general SIMT kernel (any supported dtype/kind). */
typedef struct {
  /* activations: [rows_x, K], K contiguous, row stride in elements */
  const void* x; int x_dtype; int64_t ld_x; int64_t rows_x;
  /* weights */
  int w_kind;
  const void* w;
  int64_t w_stride_e, w_stride_k, w_stride_n;     /* dense: elements. canonical MX4: bytes (k ignored) */
  const uint8_t* w_scale;                          /* canonical / B200 scales */
  int64_t ws_stride_e, ws_stride_k, ws_stride_n;   /* canonical scales: bytes */
  int E, K, N;
  /* ragged structure; slice_sizes == NULL means one slice holding all M rows (E must be 1) */
  const int32_t* slice_sizes; const int32_t* slice_offs;
  const int32_t* block_offs_16;                    /* block_offs_data, row for block size 16 */
  const int32_t* block_sched_16;                   /* block_schedule_data, row for block size 16 */
  int64_t ld_block_offs, ld_block_sched;           /* row pitch: row b serves block size 16 << b */
  int64_t M;                                       /* rows of the (gathered) problem = upper bound on sum(slice_sizes) */
  /* epilogue */
  const void* bias; int bias_dtype; int64_t ld_bias; /* [E, N] */
  const int32_t* gather_indx;                      /* [M] source rows of x, -1 = zero row */
  const int32_t* scatter_indx;                     /* [M] destination rows of y, -1 = drop */
  const float* betas; const float* gammas;         /* [M], expert-sorted order */
  float out_alpha; int has_out_alpha;
  int activation; float act_alpha; float act_limit; int act_has_limit;
  void* y; int y_dtype; int64_t ld_y;              /* [M or len(scatter), N / (2 if swiglu)] */
  /* tuning */
  int kernel;                                      /* MOE_GEMM_* */
  int tile_m;                                      /* token rows per tile of the tcgen05 kernel: 0 auto, 128, 256 */
  int tile_n;                                      /* weight rows per tile: 0 auto, 128, 256 (256 needs tile_m 256) */
  int32_t* status;                                 /* device word, set non-zero when a bounded wait expires */
  void* y_peers[MOE_MAX_PEERS];                    /* optional: output rows live on n_y_peers devices.  Output row index r */
  int n_y_peers;                                   /* (m, or scatter_indx[m]) is row r % y_rows_per_peer of the buffer */
  int64_t y_rows_per_peer;                         /* y_peers[r / y_rows_per_peer] (peer-mapped memory, same ld_y and dtype);
                                                      the epilogue stores there directly.  n_y_peers = 0: everything goes to y. */
  void* gather_scratch;                            /* optional device buffer of gather_scratch_bytes >= M * K * 2: with it, */
  int64_t gather_scratch_bytes;                    /* large gathered problems first copy the gathered rows there (one pass
                                                      over x) and the tensor-core kernel then streams consecutive rows by
                                                      TMA instead of gathering 16 bytes at a time.  NULL: gather in-kernel. */
  /* block-scaled kernel (w_kind MOE_W_MX4_B200MX; matmul.py:130-132, 311-336 of the reference: a_mx_scale / fp8
     activations against MXFP4 weights).  x_dtype MOE_F8E4M3 takes e4m3 rows as they are, with x_scale (e8m0,
     [rows_x, K / 32], row pitch ld_x_scale bytes) for MXFP8 or NULL for unit scales; x_dtype MOE_BF16 is split inside
     the library into two e4m3 terms (kind::mxf8f6f4) or, for token blocks of 16 rows, four e2m1 terms (kind::mxf4);
     MOE_GEMM_MX_F8 / MOE_GEMM_MX_F4 pin the form.  mx_workspace holds the re-laid-out token blocks:
     moe_gemm_mx_workspace_bytes(args) bytes, 1024-byte aligned.  For this kernel tile_m is the token block
     (0 auto, 16, 32, 64, 128) and tile_n 128 / 384 pins one / three weight blocks per CTA tile.                 */
  const uint8_t* x_scale; int64_t ld_x_scale;
  void* mx_workspace; int64_t mx_workspace_bytes;
  int idle_sms;                                    /* persistent kernels leave this many SMs without a CTA
                                                      (matmul.py:239-243 matmul_set_idle_sms of the reference) */
} MoeGemmArgs;
int moe_grouped_gemm(const MoeGemmArgs* args_host, void* stream);
size_t moe_gemm_mx_workspace_bytes(const MoeGemmArgs* args_host);

/* Tensor-pipe roof of one MMA kind on this device, for the benchmark's roofline: one CTA per SM issues `iters` x 4
 * back-to-back tcgen05.mma (M 128, N 256) over operand tiles resident in shared memory.  kind 0: bf16 (kind::f16),
 * 1: e4m3 x e4m3 (kind::f8f6f4), 2: padded e2m1 x e4m3 with e8m0 block scales (kind::mxf8f6f4), 3: packed e2m1 x e2m1
 * with block scales (kind::mxf4).  The caller times the call with events; *flop_out receives the FLOPs it issued.
 * `status` (optional device word) is set if the final wait expires.  Stands in for the peak tables the reference
 * quotes (roofline.py; tutorials/gluon/11-tcgen05-mma-scaled.py:1530-1535).                                       */
int moe_tensor_roof(int kind, int iters, double* flop_out_host, int32_t* status, void* stream);

/* ---- expert-parallel row movement ------------------------------------------------------------------
 * Local halves of convert_dp_to_ep / convert_ep_to_dp (distributed.py:176-211, 256-283).  Two forms of the
 * exchange use them: kernels that pull rows straight from peer-mapped buffers of the other ranks
 * (moe_gather_rows_peers, moe_gather_reduce_rows_peers, ordered by moe_peer_barrier), and an NCCL all-to-all
 * issued by the host shim, for which these kernels pack rows into per-destination contiguous,
 * expert-sorted order and unpack them.                                                              */
/* Exchange keys: keys[p] = (home rank of the token at expert-sorted position p) * world + (rank owning its
 * expert), -1 for padding.  col_sorted is the global col_sorted_indx [n], expt_indx the global [T, k] int16
 * expert ids (flat), owner[e] the rank of expert e, entries_per_rank = T_local * k.  Sorting the positions by
 * this key (moe_bitmatrix_metadata with E = world^2, k = 1) yields the order rows travel in.           */
int moe_ep_keys(const int32_t* col_sorted, const int16_t* expt_indx, const int32_t* owner, int64_t n,
                int entries_per_rank, int world, int16_t* keys, void* stream);
/* Index of the pull dispatch: for every expert-sorted position p, src_row[p] = col_sorted[p] / k (the global token row)
 * when the position's expert is local (local_expt[e] >= 0, one row of expt_map), else -2; gammas[p] = vals[col_sorted[p]]
 * (0 for padding).  vals / expt_indx are the flat [T_global * k] routing outputs.                          */
int moe_ep_pull_index(const int32_t* col_sorted, const int16_t* expt_indx, const float* vals, const int32_t* local_expt,
                      int64_t n, int k, int32_t* src_row, float* gammas, void* stream);
/* Index of the pull combine: out[i] = owner[expt_indx[lo + i]] * rows_per_peer + row_sorted[lo + i] for the n_local flat
 * (token, slot) entries of this rank's tokens, -1 where the entry was dropped (row_sorted < 0): the row of the owners'
 * output buffers that moe_gather_reduce_rows_peers reads.  Replaces the index arithmetic of distributed.py:256-283. */
int moe_ep_combine_index(const int32_t* row_sorted, const int16_t* expt_indx, const int32_t* owner, int64_t lo,
                         int64_t n_local, int64_t rows_per_peer, int32_t* out, void* stream);
int moe_gather_rows(const void* src, int64_t ld_src, const int32_t* row_indx, int64_t n_rows_out, int64_t row_bytes,
                    void* dst, int64_t ld_dst, void* stream);
/* moe_gather_rows over rows that live on several devices: global row g = row_indx[r] is row g % rows_per_peer of
 * src_peers[g / rows_per_peer] (a host array of n_peers <= MOE_MAX_PEERS device pointers, peer-mapped memory
 * included; same pitch ld_src bytes); g = -1 writes zeros, g = -2 leaves the output row untouched.  The pull half of the expert-parallel dispatch
 * (distributed.py:176-211 does the same exchange with peer stores).                                            */
int moe_gather_rows_peers(const void* const* src_peers, int n_peers, int64_t rows_per_peer, int64_t ld_src,
                          const int32_t* row_indx, int64_t n_rows_out, int64_t row_bytes, void* dst, int64_t ld_dst,
                          void* stream);
/* y[t, :] = sum over j < k of src[row_indx[t * k + j], :] (negative index: skipped); bf16 rows, fp32 sum.  The
 * k-way combine (reduce.py:1143-1165 with dim = 1) read through an index, used after the combine exchange.   */
int moe_gather_reduce_rows(const void* src, int64_t ld_src, const int32_t* row_indx, int64_t T, int k, int64_t d,
                           void* y, int64_t ld_y, void* stream);
/* Barrier among the ranks of an expert-parallel group without a collective call: sig_peers[r] is rank r's signal
 * buffer of n_peers 32-bit words (peer-mapped, zero before the first barrier), `epoch` a zeroed 32-bit word of this
 * rank's own device memory that the kernel increments.  Work enqueued before the call on every rank is complete and
 * visible before work enqueued after it on any rank starts.  The wait is bounded (2 s); on expiry `status` (optional
 * device word) is set to 901 and the kernel returns.  Replaces the NCCL barriers around the reference's peer-store
 * exchanges (distributed.py:118-126 `symm_mem_pool` barriers).                                               */
int moe_peer_barrier(void* const* sig_peers, int n_peers, int rank, uint32_t* epoch, int32_t* status, void* stream);
/* All-gather of one small slice per rank by plain loads: dst[r * slice_bytes ...] = src_peers[r][0 .. slice_bytes). */
int moe_allgather_peers(const void* const* src_peers, int n_peers, int64_t slice_bytes, void* dst, void* stream);
/* moe_gather_reduce_rows over rows that live on several devices (global row g = row g % rows_per_peer of
 * src_peers[g / rows_per_peer], pitch ld_src elements): the pull half of the expert-parallel combine fused with the
 * k-way sum (distributed.py:256-283 followed by reduce.py:1143-1165 in the reference).                          */
int moe_gather_reduce_rows_peers(const void* const* src_peers, int n_peers, int64_t rows_per_peer, int64_t ld_src,
                                 const int32_t* row_indx, int64_t T, int k, int64_t d, void* y, int64_t ld_y, void* stream);
int moe_scatter_rows(const void* src, int64_t ld_src, const int32_t* row_indx, int64_t n_rows_in, int64_t row_bytes,
                     void* dst, int64_t ld_dst, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H */
