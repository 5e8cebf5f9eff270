// hb_fa_fwd: argument validation, TMA descriptors and launch of the sm_100a
// FlashAttention-forward kernel; plus hb_debug_umma, a one-tile tcgen05 probe that
// goes through the same descriptor helpers.
#include "fa_fwd_sm100.cuh"

#include <cstdlib>
#include "host_common.h"

#include <algorithm>
#include <cmath>
#include <mutex>

namespace hb {

// K/V ring depth: as many 128-key tiles as fit next to the two Q tiles in 227 KB.
template <typename T, int D>
struct FaConfig {
  static constexpr int kStages = (D == 128 && FaTraits<T>::kElemBytes == 2) ? 5 : 8;
};

static std::mutex g_fa_mutex;  // guards the per-device set-up tables below

template <typename T, int D>
static int launch_fa(const FaParams& p, int grid, int smem_optin, cudaStream_t stream) {
  constexpr int NS = FaConfig<T, D>::kStages;
  using Smem = FaSmem<T, D, NS>;
  if ((int)sizeof(Smem) > smem_optin)
    return set_error(HB_ERR_UNSUPPORTED, "hb_fa_fwd: kernel needs %d bytes of shared memory, device offers %d",
                     (int)sizeof(Smem), smem_optin);
  auto kernel = fa_fwd_kernel<T, D, NS>;
  static bool configured[64] = {};
  int dev = 0;
  HB_CUDA_CHECK(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(g_fa_mutex);
    if (!configured[dev & 63]) {
      HB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
      configured[dev & 63] = true;
    }
  }
  kernel<<<grid, kFaThreads, sizeof(Smem), stream>>>(p);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

template <typename T, int D, int NS>
static int launch_fa_stages(const FaParams& p, int grid, int smem_optin, cudaStream_t stream) {
  using Smem = FaSmem<T, D, NS>;
  if ((int)sizeof(Smem) > smem_optin) return set_error(HB_ERR_UNSUPPORTED, "hb_debug_fa_fwd_stages: not enough shared memory");
  auto kernel = fa_fwd_kernel<T, D, NS>;
  // set on every call: this is a diagnostic path, not worth a per-device table
  HB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
  kernel<<<grid, kFaThreads, sizeof(Smem), stream>>>(p);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

static int dispatch_fa(const hb_fa_args* a, const FaParams& p, int grid, int smem_optin) {
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (a->dtype == HB_FP8_E4M3) return launch_fa<__nv_fp8_e4m3, 128>(p, grid, smem_optin, stream);
  if (a->dtype == HB_BF16) {
    return a->D == 128 ? launch_fa<__nv_bfloat16, 128>(p, grid, smem_optin, stream)
                       : launch_fa<__nv_bfloat16, 64>(p, grid, smem_optin, stream);
  }
  return a->D == 128 ? launch_fa<__half, 128>(p, grid, smem_optin, stream)
                     : launch_fa<__half, 64>(p, grid, smem_optin, stream);
}

#ifdef HB_FA_TRACE
static unsigned long long* g_trace_ptr = nullptr;
#endif

// Argument checks shared by hb_fa_fwd and hb_fa_fwd_noalloc (`who` names the entry point in
// messages).  *empty is set when there is nothing to compute.
static int fa_validate(const hb_fa_args* a, const char* who, bool allow_fp8, bool* empty) {
  *empty = false;
  if (a == nullptr) return set_error(HB_ERR_BAD_ARG, "%s: args is NULL", who);
  if (a->B < 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Sq < 0 || a->Skv < 0 || a->D <= 0)
    return set_error(HB_ERR_BAD_ARG, "%s: negative or zero extent (B=%d Hq=%d Hkv=%d Sq=%d Skv=%d D=%d)", who, a->B,
                     a->Hq, a->Hkv, a->Sq, a->Skv, a->D);
  if (a->Hq % a->Hkv != 0)
    return set_error(HB_ERR_BAD_ARG, "%s: Hq=%d is not a multiple of Hkv=%d", who, a->Hq, a->Hkv);
  if (a->dtype != HB_BF16 && a->dtype != HB_FP16 && a->dtype != HB_FP8_E4M3)
    return set_error(HB_ERR_UNSUPPORTED, "%s: unknown dtype %d", who, a->dtype);
  if (a->dtype == HB_FP8_E4M3 && !allow_fp8)
    return set_error(HB_ERR_UNSUPPORTED, "%s: dtype %d not supported (bf16, fp16)", who, a->dtype);
  if (a->D != 64 && a->D != 128)
    return set_error(HB_ERR_UNSUPPORTED, "%s: head_dim %d not supported (64 or 128)", who, a->D);
  if (a->dtype == HB_FP8_E4M3 && a->D != 128)
    return set_error(HB_ERR_UNSUPPORTED, "%s: FP8 needs head_dim 128 (got %d)", who, a->D);
  if (a->B == 0 || a->Sq == 0) {
    *empty = true;
    return HB_OK;
  }
  if (a->Skv == 0) return set_error(HB_ERR_BAD_ARG, "%s: Skv is 0 (softmax over an empty set)", who);
  if (a->causal && a->Skv < a->Sq)
    return set_error(HB_ERR_UNSUPPORTED, "%s: causal attention needs Skv >= Sq (the reference asserts past_len >= 0)",
                     who);
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->o == nullptr)
    return set_error(HB_ERR_BAD_ARG, "%s: q, k, v and o must be non-NULL", who);
  const size_t eso = 2;  // O is 16-bit for every input dtype
  if ((reinterpret_cast<uintptr_t>(a->o) & 15u) != 0 || ((a->o_stride_s * eso) & 15u) != 0 ||
      ((a->o_stride_h * eso) & 15u) != 0 || ((a->o_stride_b * eso) & 15u) != 0)
    return set_error(HB_ERR_ALIGN, "%s: o and its strides must be 16-byte aligned", who);
  if (a->lse != nullptr && (reinterpret_cast<uintptr_t>(a->lse) & 3u) != 0)
    return set_error(HB_ERR_ALIGN, "%s: lse must be 4-byte aligned", who);
  // The work list is indexed with 32-bit integers; this is the largest problem one launch takes.
  const int nqb = (a->Sq + 2 * kTileM - 1) / (2 * kTileM);
  const long long total = (long long)a->B * a->Hq * ((nqb + 1) / 2);
  if (total > 0x7fffffffLL)
    return set_error(HB_ERR_UNSUPPORTED, "%s: problem too large (%lld query blocks, limit %d)", who, total, 0x7fffffff);
  return HB_OK;
}

// Kernel parameters of a validated call: tensor maps over the caller's q, k, v (by strides, so
// BHSD, BSHD and packed views need no copy), the work-list geometry and the scales.  The tensor-map
// encoder must be initialised (get_device_state / get_device_info_noalloc do that).
static int fa_fill_params(const hb_fa_args* a, const char* who, uint32_t* status, FaParams* out) {
  FaParams& p = *out;
  memset(&p, 0, sizeof(p));
  const size_t es = dtype_size(a->dtype);
  const CUtensorMapDataType dt = a->dtype == HB_BF16   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : a->dtype == HB_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const uint32_t box[4] = {(uint32_t)(128 / es), (uint32_t)kTileM, 1, 1};  // 128 bytes of head_dim x 128 rows
  int rc;
  {
    const uint64_t dims[4] = {(uint64_t)a->D, (uint64_t)a->Sq, (uint64_t)a->Hq, (uint64_t)a->B};
    const uint64_t str[3] = {(uint64_t)a->q_stride_s * es, (uint64_t)a->q_stride_h * es, (uint64_t)a->q_stride_b * es};
    rc = encode_tensor_map(&p.tm_q, dt, 4, a->q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
  }
  {
    const uint64_t dims[4] = {(uint64_t)a->D, (uint64_t)a->Skv, (uint64_t)a->Hkv, (uint64_t)a->B};
    const uint64_t str[3] = {(uint64_t)a->k_stride_s * es, (uint64_t)a->k_stride_h * es, (uint64_t)a->k_stride_b * es};
    rc = encode_tensor_map(&p.tm_k, dt, 4, a->k, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
  }
  {
    const uint64_t dims[4] = {(uint64_t)a->D, (uint64_t)a->Skv, (uint64_t)a->Hkv, (uint64_t)a->B};
    const uint64_t str[3] = {(uint64_t)a->v_stride_s * es, (uint64_t)a->v_stride_h * es, (uint64_t)a->v_stride_b * es};
    rc = encode_tensor_map(&p.tm_v, dt, 4, a->v, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
  }
  p.o = a->o;
  p.lse = a->lse;
  p.status = status;
#ifdef HB_FA_TRACE
  p.trace = g_trace_ptr;
#endif
  p.o_sb = a->o_stride_b;
  p.o_sh = a->o_stride_h;
  p.o_ss = a->o_stride_s;
  p.B = a->B;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.Sq = a->Sq;
  p.Skv = a->Skv;
  p.group = a->Hq / a->Hkv;
  p.causal = a->causal ? 1 : 0;
  p.nqb = (a->Sq + 2 * kTileM - 1) / (2 * kTileM);
  p.npairs = (p.nqb + 1) / 2;
  p.total_pairs = (int)((long long)a->B * a->Hq * p.npairs);
  p.nkv = (a->Skv + kTileN - 1) / kTileN;
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / sqrtf((float)a->D);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out_scale = 1.0f;
  if (a->dtype == HB_FP8_E4M3) {
    // scores of the quantised operands are q_scale * k_scale too small; P carries the kernel's
    // fixed requantisation factor, V its dequantisation scale
    const float qs = a->q_scale > 0.f ? a->q_scale : 1.0f, ks = a->k_scale > 0.f ? a->k_scale : 1.0f;
    const float vs = a->v_scale > 0.f ? a->v_scale : 1.0f, os = a->o_scale > 0.f ? a->o_scale : 1.0f;
    if (a->p_scale > 0.f && a->p_scale != 1.0f / FaTraits<__nv_fp8_e4m3>::kPScale)
      return set_error(HB_ERR_UNSUPPORTED, "%s: p_scale is fixed at 1/%d in this build (pass 0)", who,
                       (int)FaTraits<__nv_fp8_e4m3>::kPScale);
    p.scale_log2 *= qs * ks;
    p.out_scale = vs / (FaTraits<__nv_fp8_e4m3>::kPScale * os);
  }
  return HB_OK;
}

static int fa_fwd_impl(const hb_fa_args* a) {
  bool empty = false;
  int rc = fa_validate(a, "hb_fa_fwd", /*allow_fp8=*/true, &empty);
  if (rc != HB_OK || empty) return rc;
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  FaParams p;
  rc = fa_fill_params(a, "hb_fa_fwd", st->status_word, &p);
  if (rc != HB_OK) return rc;
  int grid = std::min(p.total_pairs, st->sm_count);
#ifdef HB_DEBUG_GRID_ENV  // measurement builds only: fewer CTAs than SMs, to see how the per-SM rate depends on the load on L2
  if (const char* e = getenv("HB_GRID")) grid = std::max(1, std::min(grid, atoi(e)));
#endif
  return dispatch_fa(a, p, grid, st->smem_optin);
}

// The same kernel built with a different depth of the K/V ring (bf16, head_dim 128 only).  The
// pipeline depth changes when tiles are loaded, never what is computed, so the results must be
// bit-identical to hb_fa_fwd's: the test-suite uses this as its race check for the mbarrier protocol.
static int fa_fwd_stages_impl(const hb_fa_args* a, int stages) {
  bool empty = false;
  int rc = fa_validate(a, "hb_debug_fa_fwd_stages", /*allow_fp8=*/false, &empty);
  if (rc != HB_OK || empty) return rc;
  if (a->dtype != HB_BF16 || a->D != 128)
    return set_error(HB_ERR_UNSUPPORTED, "hb_debug_fa_fwd_stages: bf16 with head_dim 128 only");
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  FaParams p;
  rc = fa_fill_params(a, "hb_debug_fa_fwd_stages", st->status_word, &p);
  if (rc != HB_OK) return rc;
  const int grid = std::min(p.total_pairs, st->sm_count);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  switch (stages) {
    case 2:
      return launch_fa_stages<__nv_bfloat16, 128, 2>(p, grid, st->smem_optin, stream);
    case 3:
      return launch_fa_stages<__nv_bfloat16, 128, 3>(p, grid, st->smem_optin, stream);
    case 5:
      return launch_fa_stages<__nv_bfloat16, 128, 5>(p, grid, st->smem_optin, stream);
    default:
      return set_error(HB_ERR_UNSUPPORTED, "hb_debug_fa_fwd_stages: stages must be 2, 3 or 5 (got %d)", stages);
  }
}

// ------------------------------------------------------------------------------------
// hb_fa_fwd_noalloc: the same kernel for callers that must not allocate device memory
// ------------------------------------------------------------------------------------
// hb_fa_fwd keeps its device-side status word (the scratch the kernel's bounded waits
// report into) in memory it obtains with cudaMalloc on the first call per device.  A
// host that runs under a fixed memory budget, forbids allocation after start-up, or is
// in the middle of a stream capture cannot make that call.  This variant keeps the
// scratch in the array below instead: it is part of the library image, so every GPU
// that loads the library holds kFaNoallocScratchBytes of it until the process exits.
constexpr size_t kFaNoallocScratchBytes = 256;
static __device__ __align__(256) unsigned char g_fa_noalloc_scratch[kFaNoallocScratchBytes];

// What one launch needs from the scratch: the status word.
constexpr size_t kFaScratchNeeded = sizeof(uint32_t);

// Device address of the scratch array per device.  In host code the array's name is only
// a stand-in for the symbol, never a device pointer; the address the kernel must be given
// comes from cudaGetSymbolAddress, asked once per device with that device current.
static void* g_fa_noalloc_ptr[64] = {};

// Resolves (once per device, under the mutex) and returns the scratch array's device address
// for the current device.  Allocates nothing.
static int fa_noalloc_scratch(const char* who, int device, uint32_t** out) {
  if (device < 0 || device >= 64) return set_error(HB_ERR_UNSUPPORTED, "%s: device index %d out of range", who, device);
  std::lock_guard<std::mutex> lock(g_fa_mutex);
  if (g_fa_noalloc_ptr[device] == nullptr) {
    void* ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&ptr, g_fa_noalloc_scratch);
    if (err != cudaSuccess || ptr == nullptr)
      return set_error(HB_ERR_CUDA, "%s: cudaGetSymbolAddress failed: %s", who, cudaGetErrorString(err));
    g_fa_noalloc_ptr[device] = ptr;
  }
  *out = static_cast<uint32_t*>(g_fa_noalloc_ptr[device]);
  return HB_OK;
}

static int fa_fwd_noalloc_impl(const hb_fa_args* a) {
  bool empty = false;
  int rc = fa_validate(a, "hb_fa_fwd_noalloc", /*allow_fp8=*/false, &empty);
  if (rc != HB_OK || empty) return rc;
  if (kFaScratchNeeded > kFaNoallocScratchBytes)
    return set_error(HB_ERR_UNSUPPORTED, "hb_fa_fwd_noalloc: the kernel needs %zu bytes of scratch, the static array holds %zu",
                     kFaScratchNeeded, kFaNoallocScratchBytes);
  DeviceInfo info;
  rc = get_device_info_noalloc(&info);
  if (rc != HB_OK) return rc;
  uint32_t* status = nullptr;
  rc = fa_noalloc_scratch("hb_fa_fwd_noalloc", info.device, &status);
  if (rc != HB_OK) return rc;
  // The status word is not cleared per call: the array starts out zero when the library is
  // loaded, a kernel only ever moves the word from 0 to a code (first failure wins), and
  // hb_status_word_noalloc hands it to the host and clears it.  A time-out therefore stays
  // visible across later calls until it has been read.
  FaParams p;
  rc = fa_fill_params(a, "hb_fa_fwd_noalloc", status, &p);
  if (rc != HB_OK) return rc;
  return dispatch_fa(a, p, std::min(p.total_pairs, info.sm_count), info.smem_optin);
}

// Reads (and then clears) the status word of the static scratch array on `stream`; waits for
// that stream only.  No allocation: a 4-byte copy from the resolved symbol address.
static int status_word_noalloc_impl(uint32_t* out, void* stream_v) {
  if (out == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_status_word_noalloc: out is NULL");
  DeviceInfo info;
  int rc = get_device_info_noalloc(&info);
  if (rc != HB_OK) return rc;
  uint32_t* status = nullptr;
  rc = fa_noalloc_scratch("hb_status_word_noalloc", info.device, &status);
  if (rc != HB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  HB_CUDA_CHECK(cudaMemcpyAsync(out, status, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
  HB_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (*out != 0) {
    HB_CUDA_CHECK(cudaMemsetAsync(status, 0, sizeof(uint32_t), stream));
    return set_error(HB_ERR_TIMEOUT, "hb_status_word_noalloc: %s", describe_status(*out));
  }
  return HB_OK;
}

// ------------------------------------------------------------------------------------
// one-tile tcgen05 probe
// ------------------------------------------------------------------------------------
struct alignas(64) UmmaProbeParams {
  CUtensorMap tm_a;  // mode 0: A [128, K];  mode 1: unused
  CUtensorMap tm_b;  // mode 0: B [128, K];  mode 1: V [128, N]
  const uint32_t* p_packed;  // mode 1: P [128,128] 16-bit, row-major (64 words per row)
  float* out;
  uint32_t* status;
  int mode, kn, fmt;
};

struct UmmaProbeSmem {
  alignas(1024) uint8_t a[32768];
  alignas(1024) uint8_t b[32768];
  uint64_t full, done;
  uint32_t tmem_base, abort_flag;
};

__global__ void __launch_bounds__(128, 1) umma_probe_kernel(const __grid_constant__ UmmaProbeParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  UmmaProbeSmem& s = *reinterpret_cast<UmmaProbeSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5;
  AbortCtx ctx{&s.abort_flag, p.status};
  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    mbar_init(&s.full, 1);
    mbar_init(&s.done, 1);
    fence_mbar_init();
    if ((smem_u32(smem_raw) & 1023u) != 0u) raise_abort(ctx, kStatusSmemMisaligned);
  }
  if (warp == 0) {
    tmem_alloc(&s.tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  const int halves = p.kn / 64;
  bool ok = (s.abort_flag == 0);

  if (ok && p.mode == 1) {
    // P row of this thread -> TMEM columns [0, 64)
    uint32_t r[64];
#pragma unroll
    for (int c = 0; c < 64; ++c) r[c] = p.p_packed[threadIdx.x * 64 + c];
    tmem_st32(tmem + lane_off, &r[0]);
    tmem_st32(tmem + lane_off + 32, &r[32]);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();

  if (ok && threadIdx.x == 0) {
    tc_fence_after();
    const uint32_t bytes_b = 128u * (uint32_t)p.kn * 2u;
    if (p.mode == 0) {
      mbar_arrive_expect_tx(&s.full, 2 * bytes_b);
      for (int h = 0; h < halves; ++h) {
        tma_load_2d(s.a + h * 16384, &p.tm_a, &s.full, h * 64, 0);
        tma_load_2d(s.b + h * 16384, &p.tm_b, &s.full, h * 64, 0);
      }
    } else {
      mbar_arrive_expect_tx(&s.full, bytes_b);
      for (int h = 0; h < halves; ++h) tma_load_2d(s.b + h * 16384, &p.tm_b, &s.full, h * 64, 0);
    }
    if (mbar_wait(&s.full, 0, ctx, 10)) {
      tc_fence_after();
      if (p.mode == 0) {
        const uint32_t idesc = make_idesc((uint32_t)p.fmt, 128, 128, 0, 0);
        for (int kk = 0; kk < p.kn / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk / 4) * 16384u + (uint32_t)(kk % 4) * 32u;
          umma_ss_f16(tmem + 128, make_smem_desc_sw128(smem_u32(s.a) + off, 16, 1024),
                      make_smem_desc_sw128(smem_u32(s.b) + off, 16, 1024), idesc, kk > 0 ? 1u : 0u);
        }
      } else {
        const uint32_t idesc = make_idesc((uint32_t)p.fmt, 128, (uint32_t)p.kn, 0, 1);
        for (int kk = 0; kk < 8; ++kk) {
          umma_ts_f16(tmem + 128, tmem + (uint32_t)(kk * 8),
                      make_smem_desc_sw128(smem_u32(s.b) + (uint32_t)kk * 2048u, 16384, 1024), idesc,
                      kk > 0 ? 1u : 0u);
        }
      }
      umma_commit(&s.done);
    }
  }
  __syncwarp();
  const int ncols = p.mode == 0 ? 128 : p.kn;
  if (ok && mbar_wait(&s.done, 0, ctx, 11)) {
    tc_fence_after();
    for (int c = 0; c < ncols / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem + lane_off + 128u + (uint32_t)(c * 32), r);
      tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 32; ++e) p.out[threadIdx.x * ncols + c * 32 + e] = __uint_as_float(r[e]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

static int debug_umma_impl(int mode, const void* a, const void* b, float* out, int kn, int dtype, void* stream) {
  if (a == nullptr || b == nullptr || out == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_debug_umma: NULL pointer");
  if (mode != 0 && mode != 1) return set_error(HB_ERR_BAD_ARG, "hb_debug_umma: mode must be 0 or 1");
  if (kn != 64 && kn != 128) return set_error(HB_ERR_BAD_ARG, "hb_debug_umma: kn must be 64 or 128");
  if (dtype != HB_BF16 && dtype != HB_FP16) return set_error(HB_ERR_UNSUPPORTED, "hb_debug_umma: 16-bit dtypes only");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  UmmaProbeParams p;
  memset(&p, 0, sizeof(p));
  const CUtensorMapDataType dt = dtype == HB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const uint64_t dims[2] = {(uint64_t)kn, 128};
  const uint64_t str[1] = {(uint64_t)kn * 2};
  const uint32_t box[2] = {64, 128};
  if (mode == 0) {
    rc = encode_tensor_map(&p.tm_a, dt, 2, a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
  } else {
    p.p_packed = static_cast<const uint32_t*>(a);
  }
  rc = encode_tensor_map(&p.tm_b, dt, 2, b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != HB_OK) return rc;
  p.out = out;
  p.status = st->status_word;
  p.mode = mode;
  p.kn = kn;
  p.fmt = dtype == HB_BF16 ? 1 : 0;
  static bool configured[64] = {};
  if (!configured[st->device & 63]) {
    HB_CUDA_CHECK(cudaFuncSetAttribute(umma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)sizeof(UmmaProbeSmem)));
    configured[st->device & 63] = true;
  }
  umma_probe_kernel<<<1, 128, sizeof(UmmaProbeSmem), static_cast<cudaStream_t>(stream)>>>(p);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

int fa_smem_bytes() { return (int)sizeof(FaSmem<__nv_bfloat16, 128, FaConfig<__nv_bfloat16, 128>::kStages>); }

}  // namespace hb

extern "C" {

int hb_fa_fwd(const hb_fa_args* args) {
  hb::clear_error();
  return hb::fa_fwd_impl(args);
}

#ifdef HB_FA_TRACE
// tracing builds only: device buffer of 16 regions x 4096 x 8 bytes, zeroed by the caller
int hb_debug_set_trace(void* ptr) {
  hb::g_trace_ptr = static_cast<unsigned long long*>(ptr);
  return 0;
}
#endif

int hb_fa_fwd_noalloc(const hb_fa_args* args) {
  hb::clear_error();
  return hb::fa_fwd_noalloc_impl(args);
}

int hb_debug_fa_fwd_stages(const hb_fa_args* args, int32_t stages) {
  hb::clear_error();
  return hb::fa_fwd_stages_impl(args, stages);
}

int hb_status_word_noalloc(uint32_t* out, void* stream) {
  hb::clear_error();
  return hb::status_word_noalloc_impl(out, stream);
}

int hb_debug_umma(int mode, const void* a, const void* b, float* out, int32_t kn, int32_t dtype, void* stream) {
  hb::clear_error();
  return hb::debug_umma_impl(mode, a, b, out, kn, dtype, stream);
}

}  // extern "C"
