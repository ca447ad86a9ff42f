// moe_grouped_gemm: argument validation and kernel selection for the ragged grouped GEMM.
#include "gemm_common.cuh"

int moe_gemm_simt_launch(const GemmParams& p, int x_dtype, int y_dtype, int w_kind, int64_t grid_m, cudaStream_t st);
int moe_gemm_tc_launch(const GemmParams& p, const MoeGemmArgs& a, cudaStream_t st);
bool moe_gemm_tc_supported(const MoeGemmArgs& a, const char** why);
int moe_gemm_tc_pair_launch(const GemmParams& p, const MoeGemmArgs& a, cudaStream_t st);
bool moe_gemm_tc_pair_supported(const MoeGemmArgs& a, const char** why);
int moe_gemm_stream_launch(const GemmParams& p, const MoeGemmArgs& a, cudaStream_t st);
bool moe_gemm_stream_supported(const MoeGemmArgs& a, const char** why);
int moe_gemm_mx_launch(const GemmParams& p, const MoeGemmArgs& a, cudaStream_t st);
bool moe_gemm_mx_supported(const MoeGemmArgs& a, const char** why);

// upper bound on the number of row blocks (triton_kernels tensor_details/ragged_tensor.py:73-77)
static int64_t n_blocks_bound(int64_t n_slices, int64_t n_rows, int64_t block) {
  if (n_rows <= n_slices) return n_rows;
  int64_t a = n_slices - n_rows - 1;                 // negative
  int64_t fl = -((-a + block - 1) / block);          // floor division
  return n_slices - 1 - fl;
}

extern "C" __attribute__((visibility("default"))) int moe_grouped_gemm(const MoeGemmArgs* a, void* stream) {
  MOE_CHECK_ARG(a != nullptr, "moe_grouped_gemm: args is NULL");
  MOE_CHECK_ARG(a->E > 0 && a->K >= 0 && a->N >= 0 && a->M >= 0, "moe_grouped_gemm: bad extents E=%d K=%d N=%d M=%lld",
                a->E, a->K, a->N, (long long)a->M);
  if (a->M == 0 || a->N == 0) return MOE_OK;
  MOE_CHECK_ARG(a->x && a->w && (a->y || a->n_y_peers > 0), "moe_grouped_gemm: NULL x / w / y");
  MOE_CHECK_ARG(a->w_kind == MOE_W_DENSE || a->w_scale, "moe_grouped_gemm: MXFP4 weights need w_scale");
  MOE_CHECK_ARG(a->w_kind == MOE_W_DENSE || a->K % 32 == 0, "moe_grouped_gemm: MXFP4 weights need K %% 32 == 0 (K=%d)", a->K);
  MOE_CHECK_ARG(a->activation == MOE_ACT_NONE || (a->activation == MOE_ACT_SWIGLU && a->N % 2 == 0),
                "moe_grouped_gemm: SwiGLU needs an even N");
  if (a->slice_sizes) {
    MOE_CHECK_ARG(a->slice_offs && a->block_offs_16 && a->block_sched_16, "moe_grouped_gemm: ragged metadata incomplete");
  } else {
    MOE_CHECK_ARG(a->E == 1, "moe_grouped_gemm: without ragged metadata there must be one weight matrix");
  }
  cudaStream_t st = (cudaStream_t)stream;

  GemmParams p;
  p.x = a->x; p.ld_x = a->ld_x; p.rows_x = a->rows_x;
  p.w = a->w; p.w_stride_e = a->w_stride_e; p.w_stride_k = a->w_stride_k; p.w_stride_n = a->w_stride_n;
  p.w_scale = a->w_scale; p.ws_stride_e = a->ws_stride_e; p.ws_stride_k = a->ws_stride_k; p.ws_stride_n = a->ws_stride_n;
  p.E = a->E; p.K = a->K; p.N = a->N;
  p.slice_sizes = a->slice_sizes; p.slice_offs = a->slice_offs;
  p.block_offs = nullptr; p.block_sched = nullptr;
  p.M = a->M;
  p.bias = a->bias; p.bias_dtype = a->bias_dtype; p.ld_bias = a->ld_bias;
  p.gather_indx = a->gather_indx; p.scatter_indx = a->scatter_indx;
  p.betas = a->betas; p.gammas = a->gammas;
  p.out_alpha = a->out_alpha; p.has_out_alpha = a->has_out_alpha;
  p.activation = a->activation; p.act_alpha = a->act_alpha; p.act_limit = a->act_limit; p.act_has_limit = a->act_has_limit;
  p.y = a->y; p.ld_y = a->ld_y;
  p.status = a->status;
  MOE_CHECK_ARG(a->n_y_peers >= 0 && a->n_y_peers <= MOE_MAX_PEERS, "moe_grouped_gemm: n_y_peers must be 0..%d", MOE_MAX_PEERS);
  p.n_y_peers = a->n_y_peers; p.y_rows_per_peer = a->y_rows_per_peer;
  for (int i = 0; i < MOE_MAX_PEERS; ++i) p.y_peers[i] = i < a->n_y_peers ? a->y_peers[i] : nullptr;
  if (a->n_y_peers > 0) {
    MOE_CHECK_ARG(a->y_rows_per_peer > 0, "moe_grouped_gemm: y_rows_per_peer must be positive with y_peers");
    for (int i = 0; i < a->n_y_peers; ++i)
      MOE_CHECK_ARG(a->y_peers[i] != nullptr && (uintptr_t)a->y_peers[i] % 16 == 0,
                    "moe_grouped_gemm: y_peers[%d] is NULL or not 16-byte aligned", i);
    p.y = a->y_peers[0];
  }

  const char* why = "";
  const bool mx_asked = a->kernel == MOE_GEMM_MX || a->kernel == MOE_GEMM_MX_F8 || a->kernel == MOE_GEMM_MX_F4;
  if (a->w_kind == MOE_W_MX4_B200MX || mx_asked) {
    // weights laid out for the block-scaled MMA: that kernel or nothing
    if (!moe_gemm_mx_supported(*a, &why) || (a->kernel != MOE_GEMM_AUTO && !mx_asked)) {
      moe_set_error("moe_grouped_gemm: block-scaled kernel not applicable: %s", *why ? why : "another kernel was requested");
      return MOE_ERR_UNSUPPORTED;
    }
    return moe_gemm_mx_launch(p, *a, st);
  }
  bool tc = moe_gemm_tc_supported(*a, &why);
  if ((a->kernel == MOE_GEMM_TCGEN05 || a->kernel == MOE_GEMM_TCGEN05_PAIR || a->kernel == MOE_GEMM_STREAM) && !tc) {
    moe_set_error("moe_grouped_gemm: tcgen05 kernel not applicable: %s", why);
    return MOE_ERR_UNSUPPORTED;
  }
  if (a->kernel == MOE_GEMM_SIMT) tc = false;
  if (tc) {
    // A few rows per expert (decode): the weight-streaming kernel, bound by HBM rather than by pipeline hand-offs.
    bool streaming = moe_gemm_stream_supported(*a, &why);
    if (a->kernel == MOE_GEMM_STREAM && !streaming) {
      moe_set_error("moe_grouped_gemm: streaming kernel not applicable: %s", why);
      return MOE_ERR_UNSUPPORTED;
    }
    if (a->kernel == MOE_GEMM_AUTO)
      streaming = streaming && a->tile_m == 0 && a->tile_n == 0 && a->M <= 10 * (int64_t)(a->E > 0 ? a->E : 1);
    else if (a->kernel != MOE_GEMM_STREAM)
      streaming = false;
    if (streaming) return moe_gemm_stream_launch(p, *a, st);
    // Large problems run on pairs of SMs (256 x 256 tiles, cta_group::2); small ones and explicit tile requests on
    // the single-SM kernel.
    bool pair = moe_gemm_tc_pair_supported(*a, &why);
    if (a->kernel == MOE_GEMM_TCGEN05_PAIR && !pair) {
      moe_set_error("moe_grouped_gemm: SM-pair tcgen05 kernel not applicable: %s", why);
      return MOE_ERR_UNSUPPORTED;
    }
    if (a->kernel != MOE_GEMM_TCGEN05_PAIR) pair = false;
    // Large gathered problems: copy the gathered rows once into the caller's scratch, then stream them by TMA.
    const bool big = (a->tile_m == 0 || a->tile_m == 256) && (a->tile_m == 256 || a->M / (a->E > 0 ? a->E : 1) >= 12);
    if (a->gather_indx && a->gather_scratch && big && a->gather_scratch_bytes >= (int64_t)a->M * a->K * 2) {
      const int rc = moe_gather_rows(a->x, a->ld_x * 2, a->gather_indx, a->M, (int64_t)a->K * 2, a->gather_scratch,
                                     (int64_t)a->K * 2, stream);
      if (rc != MOE_OK) return rc;
      p.x = a->gather_scratch; p.ld_x = a->K; p.rows_x = a->M; p.gather_indx = nullptr;
    }
    if (pair) return moe_gemm_tc_pair_launch(p, *a, st);
    return moe_gemm_tc_launch(p, *a, st);
  }

  MOE_CHECK_ARG(a->w_kind == MOE_W_DENSE || a->w_kind == MOE_W_MX4_CANONICAL,
                "moe_grouped_gemm: the SIMT kernel takes dense or canonical MXFP4 weights (%s)", why);
  int64_t grid_m;
  if (a->slice_sizes) {
    p.block_offs = a->block_offs_16 + 2 * a->ld_block_offs;     // block size 64
    p.block_sched = a->block_sched_16 + 2 * a->ld_block_sched;
    grid_m = n_blocks_bound(a->E, a->M, 64);
  } else {
    grid_m = cdiv64(a->M, 64);
  }
  if (grid_m == 0) return MOE_OK;
  return moe_gemm_simt_launch(p, a->x_dtype, a->y_dtype, a->w_kind, grid_m, st);
}
