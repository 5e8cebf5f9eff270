// hb_gemm_epilogue / hb_rms_rowstat: validation, TMA descriptors and launch.
#include "gemm_sm100.cuh"
#include "host_common.h"

#include <algorithm>
#include <cstdlib>

namespace hb {

template <typename T, int EPI>
static int launch_gemm(const GemmParams& p, int grid, const DeviceState* st, cudaStream_t stream) {
  if ((int)sizeof(GemmSmem) > st->smem_optin)
    return set_error(HB_ERR_UNSUPPORTED, "hb_gemm_epilogue: kernel needs %d bytes of shared memory, device offers %d",
                     (int)sizeof(GemmSmem), st->smem_optin);
  auto kernel = gemm_kernel<T, EPI>;
  static bool configured[64] = {};
  if (!configured[st->device & 63]) {
    HB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(GemmSmem)));
    configured[st->device & 63] = true;
  }
  kernel<<<grid, kGemmThreads, sizeof(GemmSmem), stream>>>(p);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

template <typename T, int EPI>
static int launch_gemm_pair(const GemmParams& p, int grid, const DeviceState* st, cudaStream_t stream) {
  if (kPairSmemBytes > st->smem_optin)
    return set_error(HB_ERR_UNSUPPORTED, "hb_gemm_epilogue: kernel needs %d bytes of shared memory, device offers %d",
                     kPairSmemBytes, st->smem_optin);
  auto kernel = gemm_pair_kernel<T, EPI>;
  static bool configured[64] = {};
  if (!configured[st->device & 63]) {
    HB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes));
    configured[st->device & 63] = true;
  }
  kernel<<<grid, kGemmThreads, kPairSmemBytes, stream>>>(p);  // clusters of two CTAs (compile-time attribute)
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

template <typename T>
static int dispatch_gemm(int epi_class, const GemmParams& p, int grid, bool pair, const DeviceState* st, cudaStream_t stream) {
  if (pair) {
    switch (epi_class) {
      case kEpiPlain:
        return launch_gemm_pair<T, kEpiPlain>(p, grid, st, stream);
      case kEpiSwiglu:
        return launch_gemm_pair<T, kEpiSwiglu>(p, grid, st, stream);
      default:
        return launch_gemm_pair<T, kEpiRope>(p, grid, st, stream);
    }
  }
  switch (epi_class) {
    case kEpiPlain:
      return launch_gemm<T, kEpiPlain>(p, grid, st, stream);
    case kEpiSwiglu:
      return launch_gemm<T, kEpiSwiglu>(p, grid, st, stream);
    default:
      return launch_gemm<T, kEpiRope>(p, grid, st, stream);
  }
}

static bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

static int gemm_impl(const hb_gemm_args* a) {
  if (a == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: args is NULL");
  if (a->M < 0 || a->N <= 0 || a->K <= 0)
    return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: bad extents M=%d N=%d K=%d", a->M, a->N, a->K);
  if (a->dtype != HB_BF16 && a->dtype != HB_FP16)
    return set_error(HB_ERR_UNSUPPORTED, "hb_gemm_epilogue: dtype %d not supported (bf16, fp16)", a->dtype);
  if (a->epilogue < HB_EPI_NONE || a->epilogue > HB_EPI_ROPE)
    return set_error(HB_ERR_UNSUPPORTED, "hb_gemm_epilogue: unknown epilogue %d", a->epilogue);
  int n_out = a->N;
  int epi_class = kEpiPlain;
  if (a->epilogue == HB_EPI_SWIGLU) {
    if (a->N % 2 != 0) return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: SWIGLU needs an even N (stacked [Wg; Wu])");
    n_out = a->N / 2;
    epi_class = kEpiSwiglu;
  } else if (a->epilogue == HB_EPI_ROPE) {
    epi_class = kEpiRope;
    if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256)
      return set_error(HB_ERR_UNSUPPORTED, "hb_gemm_epilogue: ROPE head_dim %d not supported (64, 128, 256)", a->head_dim);
    if (a->N % a->head_dim != 0 || a->rope_cols % a->head_dim != 0 || a->rope_cols < 0 || a->rope_cols > a->N)
      return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: ROPE needs head_dim | N and head_dim | rope_cols <= N");
    if (a->rope_cos == nullptr || a->rope_sin == nullptr || a->rope_seq <= 0)
      return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: ROPE needs cos/sin tables and rope_seq > 0");
    if ((reinterpret_cast<uintptr_t>(a->rope_cos) & 15) != 0 || (reinterpret_cast<uintptr_t>(a->rope_sin) & 15) != 0)
      return set_error(HB_ERR_ALIGN, "hb_gemm_epilogue: ROPE tables need 16-byte alignment");
  }
  if (a->schedule < HB_GEMM_AUTO || a->schedule > HB_GEMM_PAIR)
    return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: unknown schedule %d", a->schedule);
  const int batch = a->batch > 0 ? a->batch : 1;
  const bool w_kn = a->w_layout == HB_W_KN;
  if (a->w_layout != HB_W_NK && a->w_layout != HB_W_KN)
    return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: unknown w_layout %d", a->w_layout);
  if (w_kn && epi_class != kEpiPlain)
    return set_error(HB_ERR_UNSUPPORTED, "hb_gemm_epilogue: SWIGLU / ROPE need the weight in [N, K] layout");
  if (batch > 1 && epi_class == kEpiRope)
    return set_error(HB_ERR_UNSUPPORTED, "hb_gemm_epilogue: ROPE is not defined for batched products");
  if (a->M == 0) return HB_OK;
  if (a->a == nullptr || a->w == nullptr || a->out == nullptr)
    return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: a, w and out must be non-NULL");
  if ((a->K % 8) || (n_out % 8) || (a->lda % 8) || (a->ldw % 8) || (a->ldo % 8) ||
      (a->residual != nullptr && (a->ldr % 8)))
    return set_error(HB_ERR_ALIGN, "hb_gemm_epilogue: K, N_out and the leading dimensions must be multiples of 8");
  if (a->lda < a->K || a->ldw < (w_kn ? a->N : a->K) || a->ldo < n_out || (a->residual != nullptr && a->ldr < n_out))
    return set_error(HB_ERR_BAD_ARG, "hb_gemm_epilogue: a leading dimension is smaller than its row");
  const long long w_rows = w_kn ? a->K : a->N;
  // batch strides (elements); 0 selects densely packed batches
  const long long a_bs = a->a_batch_stride ? a->a_batch_stride : (long long)a->M * a->lda;
  const long long w_bs = a->w_batch_stride ? a->w_batch_stride : w_rows * a->ldw;
  const long long o_bs = a->o_batch_stride ? a->o_batch_stride : (long long)a->M * a->ldo;
  const long long r_bs = a->r_batch_stride ? a->r_batch_stride : (long long)a->M * a->ldr;
  if (batch > 1 && ((a_bs % 8) || (w_bs % 8) || (o_bs % 8) || (a->residual != nullptr && (r_bs % 8))))
    return set_error(HB_ERR_ALIGN, "hb_gemm_epilogue: batch strides must be multiples of 8 elements");
  if (!aligned16(a->a) || !aligned16(a->w) || !aligned16(a->out) || !aligned16(a->residual) || !aligned16(a->bias))
    return set_error(HB_ERR_ALIGN, "hb_gemm_epilogue: pointers must be 16-byte aligned");

  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != HB_OK) return rc;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  const CUtensorMapDataType dt = a->dtype == HB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  {
    const uint32_t box[3] = {(uint32_t)kGemmBK, 128, 1};
    const uint64_t dims[3] = {(uint64_t)a->K, (uint64_t)a->M, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)a->lda * 2, (uint64_t)a_bs * 2};
    rc = encode_tensor_map(&p.tm_a, dt, 3, a->a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
  }
  if (w_kn) {
    const uint32_t box[3] = {64, (uint32_t)kGemmBK, 1};  // 64 columns (128 bytes) x 64 k-rows
    const uint64_t dims[3] = {(uint64_t)a->N, (uint64_t)a->K, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)a->ldw * 2, (uint64_t)w_bs * 2};
    rc = encode_tensor_map(&p.tm_w, dt, 3, a->w, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
  } else {
    const uint32_t box[3] = {(uint32_t)kGemmBK, 128, 1};
    const uint64_t dims[3] = {(uint64_t)a->K, (uint64_t)a->N, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)a->ldw * 2, (uint64_t)w_bs * 2};
    rc = encode_tensor_map(&p.tm_w, dt, 3, a->w, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
  }
  if (epi_class == kEpiPlain) {
    const uint32_t box[3] = {64, (uint32_t)kGemmBM, 1};
    const uint64_t dims[3] = {(uint64_t)n_out, (uint64_t)a->M, (uint64_t)batch};
    const uint64_t str[2] = {(uint64_t)a->ldo * 2, (uint64_t)o_bs * 2};
    rc = encode_tensor_map(&p.tm_out, dt, 3, a->out, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
    p.tma_store = 1;
  }
  p.out = a->out;
  p.row_scale = a->row_scale;
  p.residual = a->residual;
  p.bias = a->bias;
  p.rope_cos = a->rope_cos;
  p.rope_sin = a->rope_sin;
  p.status = st->status_word;
  p.ldo = a->ldo;
  p.ldr = a->ldr;
  p.M = a->M;
  p.N_out = n_out;
  p.K = a->K;
  p.tile_cols = epi_class == kEpiSwiglu ? 128 : kGemmBN;
  // CTA pairs (256-row tiles) whenever a problem has more than one 128-row tile of rows
  const bool pair = a->schedule == HB_GEMM_PAIR || (a->schedule == HB_GEMM_AUTO && a->M > kGemmBM && st->sm_count >= 2);
  const int tile_rows = pair ? kPairBM : kGemmBM;
  p.tiles_m = (a->M + tile_rows - 1) / tile_rows;
  p.tiles_n = (n_out + p.tile_cols - 1) / p.tile_cols;
  p.tiles_per_batch = p.tiles_m * p.tiles_n;
  const long long tiles = (long long)p.tiles_m * p.tiles_n * batch;
  if (tiles > 0x7fffffffLL || (long long)batch * a->M > 0x7fffffffLL)
    return set_error(HB_ERR_UNSUPPORTED, "hb_gemm_epilogue: too many tiles");
  p.num_tiles = (int)tiles;
  p.batch = batch;
  p.w_kn = w_kn ? 1 : 0;
  p.o_batch_stride = o_bs;
  p.r_batch_stride = r_bs;
  p.k_steps = (a->K + kGemmBK - 1) / kGemmBK;
  p.act = (a->epilogue >= HB_EPI_SILU && a->epilogue <= HB_EPI_TANH) ? a->epilogue : kActNone;
  p.rope_seq = a->rope_seq;
  p.head_dim = a->head_dim;
  p.rope_cols = a->rope_cols;
  p.w_row2_offset = n_out;
  // shared-memory split of the pair kernel: a long K loop gets the deepest ring; a short one, whose time is
  // the epilogue's, gives one stage to a second staging slab per warpgroup so that a tile's two slabs leave
  // back to back (measured: 1, 2 and 4 slabs are within 2 % of each other, 4 costs the K = 512 case 10 %)
  p.out_slabs = p.k_steps >= 8 ? 1 : 2;
  p.pair_stages = kPairSlots - p.out_slabs;

  const int grid = pair ? 2 * (int)std::min<long long>(tiles, st->sm_count / 2) : (int)std::min<long long>(tiles, st->sm_count);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  return a->dtype == HB_BF16 ? dispatch_gemm<__nv_bfloat16>(epi_class, p, grid, pair, st, stream)
                             : dispatch_gemm<__half>(epi_class, p, grid, pair, st, stream);
}

static int rowstat_impl(const void* x, const void* residual, void* y_out, float* rstd, int M, int N, long long ldx,
                        float eps, int dtype, void* stream) {
  if (M < 0 || N <= 0) return set_error(HB_ERR_BAD_ARG, "hb_rms_rowstat: bad extents M=%d N=%d", M, N);
  if (dtype != HB_BF16 && dtype != HB_FP16) return set_error(HB_ERR_UNSUPPORTED, "hb_rms_rowstat: dtype %d", dtype);
  if (M == 0) return HB_OK;
  if (x == nullptr || rstd == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_rms_rowstat: x and rstd must be non-NULL");
  if ((N % 8) || (ldx % 8) || ldx < N || !aligned16(x) || !aligned16(residual) || !aligned16(y_out))
    return set_error(HB_ERR_ALIGN, "hb_rms_rowstat: N and ldx must be multiples of 8, pointers 16-byte aligned");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  const int grid = (M + 7) / 8;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == HB_BF16) {
    rms_rowstat_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
        static_cast<__nv_bfloat16*>(y_out), rstd, M, N, ldx, eps);
  } else {
    rms_rowstat_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(x), static_cast<const __half*>(residual),
                                                    static_cast<__half*>(y_out), rstd, M, N, ldx, eps);
  }
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

int gemm_smem_bytes() { return (int)sizeof(GemmSmem); }

}  // namespace hb

extern "C" {

int hb_gemm_epilogue(const hb_gemm_args* args) {
  hb::clear_error();
  return hb::gemm_impl(args);
}

int hb_rms_rowstat(const void* x, const void* residual, void* y_out, float* rstd, int32_t M, int32_t N, int64_t ldx,
                   float eps, int32_t dtype, void* stream) {
  hb::clear_error();
  return hb::rowstat_impl(x, residual, y_out, rstd, M, N, ldx, eps, dtype, stream);
}

}  // extern "C"

extern "C" int hb_prepare_weight(const hb_prepare_args* a) {
  using namespace hb;
  if (a == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_prepare_weight: args is NULL");
  if (a->n_src < 1 || a->n_src > 4) return set_error(HB_ERR_BAD_ARG, "hb_prepare_weight: n_src must be 1..4");
  if (a->dtype != HB_BF16 && a->dtype != HB_FP16)
    return set_error(HB_ERR_UNSUPPORTED, "hb_prepare_weight: dtype %d not supported (bf16, fp16)", a->dtype);
  if (a->K <= 0 || a->K % 8 != 0) return set_error(HB_ERR_ALIGN, "hb_prepare_weight: K must be a positive multiple of 8");
  if (a->out == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_prepare_weight: out is NULL");
  if (a->ld_out < a->K || a->ld_out % 8 != 0 || (reinterpret_cast<uintptr_t>(a->out) & 15) != 0)
    return set_error(HB_ERR_ALIGN, "hb_prepare_weight: out needs 16-byte alignment and a row stride that is a multiple of 8");
  if (a->gamma != nullptr && (reinterpret_cast<uintptr_t>(a->gamma) & 15) != 0)
    return set_error(HB_ERR_ALIGN, "hb_prepare_weight: gamma needs 16-byte alignment");
  PrepareParams p;
  memset(&p, 0, sizeof(p));
  long long rows = 0;
  for (int i = 0; i < a->n_src; ++i) {
    if (a->src[i] == nullptr || a->rows[i] <= 0) return set_error(HB_ERR_BAD_ARG, "hb_prepare_weight: source %d is empty", i);
    if (a->ld_src[i] < a->K || a->ld_src[i] % 8 != 0 || (reinterpret_cast<uintptr_t>(a->src[i]) & 15) != 0)
      return set_error(HB_ERR_ALIGN, "hb_prepare_weight: source %d needs 16-byte alignment and a row stride that is a multiple of 8", i);
    rows += a->rows[i];
    if (rows > 0x7fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_prepare_weight: too many rows");
    p.src[i] = a->src[i];
    p.ld_src[i] = a->ld_src[i];
    p.row_end[i] = static_cast<int>(rows);
  }
  for (int i = a->n_src; i < 4; ++i) p.row_end[i] = static_cast<int>(rows);
  p.n_src = a->n_src;
  p.K = a->K;
  p.gamma = a->gamma;
  p.out = a->out;
  p.ld_out = a->ld_out;
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  const long long total = rows * (a->K / 8);
  const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 16ll * st->sm_count));
  if (a->dtype == HB_BF16) {
    prepare_weight_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  } else {
    prepare_weight_kernel<__half><<<grid, 256, 0, stream>>>(p);
  }
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}
