// hb_h2o_score:  score[b,h,k] = sum_q exp(scale * q.k + mask - LSE[q])
//
// Restates Heddle/heddle/tileop/h2o_attention.py:27-136: a second pass over Q K^T that
// turns scores into probabilities with the row-wise LSE of the attention kernel and sums
// them over the query axis.  The reference computes S = Q K^T with queries on the rows
// and reduces over rows (T.reduce_sum(dim=0), :122); here the product is issued
// transposed, S^T = K Q^T, so that a key is a TMEM lane: each thread owns one key, the sum
// over queries is a plain per-thread accumulation and needs no cross-thread reduction.
//
// CTA (384 threads), one 128-key tile of one (batch, head) at a time:
//   warp 0      TMA: the K tile (A operand) once per work item, a ring of Q tiles (B operand)
//   warp 1      MMA: tcgen05.mma M=128 (keys) N=128 (queries), two TMEM accumulator buffers
//   warps 4-7   consumer group 0: even query tiles      exp2(s*scale*log2e - LSE*log2e), masks,
//   warps 8-11  consumer group 1: odd query tiles       per-key running sum
#include "host_common.h"
#include "ptx_sm100.cuh"

#include <algorithm>
#include <cmath>

namespace hb {

constexpr int kH2oThreads = 384;
constexpr int kH2oStages = 4;
enum H2oRole : uint32_t { kH2oTma = 0x31, kH2oMma = 0x32, kH2oCons = 0x33, kH2oDrain = 0x34 };

struct alignas(64) H2oParams {
  CUtensorMap tm_q;
  CUtensorMap tm_k;
  const float* lse;
  float* score;
  uint32_t* status;
  int B, Hq, Hkv, Sq, Skv;
  int group, causal;
  int nkb;         // 128-key tiles per head
  int nqb;         // 128-query tiles
  int total_items; // B * Hq * nkb
  float scale_log2;
};

template <int D>
struct H2oSmem {
  static constexpr int kTileBytes = 128 * D * 2;
  alignas(1024) uint8_t k[kTileBytes];
  alignas(1024) uint8_t q[kH2oStages][kTileBytes];
  uint64_t k_full, k_empty;
  uint64_t q_full[kH2oStages], q_empty[kH2oStages];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t drain;
  uint32_t tmem_base, abort_flag;
};

struct H2oItem {
  int b, hq, hkv, k0, qt0;  // first key, first query tile that can see this key tile
};

__device__ __forceinline__ void h2o_get_item(const H2oParams& p, int g, H2oItem& it) {
  // heaviest key tiles first within a head (causal: low key index = most queries)
  const int kb = g % p.nkb;
  const int bh = g / p.nkb;
  it.b = bh / p.Hq;
  it.hq = bh - it.b * p.Hq;
  it.hkv = it.hq / p.group;
  it.k0 = kb * 128;
  // h2o_attention.py:99-101: q_start = max(0, (k0 - past_len) / block_M)
  it.qt0 = p.causal ? max(0, (it.k0 - (p.Skv - p.Sq)) / 128) : 0;
}

template <typename T, int D>
__global__ void __launch_bounds__(kH2oThreads, 1) h2o_score_kernel(const __grid_constant__ H2oParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using Smem = H2oSmem<D>;
  Smem& s = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{&s.abort_flag, p.status};

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    mbar_init(&s.k_full, 1);
    mbar_init(&s.k_empty, 1);
    for (int i = 0; i < kH2oStages; ++i) {
      mbar_init(&s.q_full[i], 1);
      mbar_init(&s.q_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 4);
    }
    mbar_init(&s.drain, 1);
    fence_mbar_init();
    if ((smem_u32(smem_raw) & 1023u) != 0u) raise_abort(ctx, kStatusSmemMisaligned);
    prefetch_tensormap(&p.tm_q);
    prefetch_tensormap(&p.tm_k);
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const bool run = (s.abort_flag == 0);
  constexpr uint32_t kTileBytes = Smem::kTileBytes;
  constexpr uint32_t kHalfBytes = 128 * 128;

  if (warp == 0) {
    if (run && lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t st = 0, phase = 1, k_phase = 1;
      bool ok = true;
      for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x) {
        H2oItem it;
        h2o_get_item(p, g, it);
        if (!mbar_wait(&s.k_empty, k_phase, ctx, kH2oTma)) break;
        k_phase ^= 1;
        mbar_arrive_expect_tx(&s.k_full, kTileBytes);
        for (int h = 0; h < D / 64; ++h) tma_load_4d(s.k + h * kHalfBytes, &p.tm_k, &s.k_full, h * 64, it.k0, it.hkv, it.b);
        for (int qt = it.qt0; qt < p.nqb; ++qt) {
          if (!mbar_wait(&s.q_empty[st], phase, ctx, kH2oTma)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&s.q_full[st], kTileBytes);
          for (int h = 0; h < D / 64; ++h)
            tma_load_4d(s.q[st] + h * kHalfBytes, &p.tm_q, &s.q_full[st], h * 64, qt * 128, it.hq, it.b);
          if (++st == kH2oStages) {
            st = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (run) {
      // ---------------- MMA issuer (warp-uniform, elected lane issues) ----------------
      constexpr uint32_t idesc = make_idesc(Pack2<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kLbo = (16u >> 4) << 16;
      const bool leader = elect_one();
      uint32_t st = 0, phase = 0, k_phase = 0, tile_i = 0;
      bool ok = true;
      const uint32_t k_lo = (smem_u32(s.k) >> 4) | kLbo;
      for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x) {
        H2oItem it;
        h2o_get_item(p, g, it);
        if (!mbar_wait_warp(&s.k_full, k_phase, ctx, kH2oMma)) break;
        k_phase ^= 1;
        for (int qt = it.qt0; qt < p.nqb; ++qt, ++tile_i) {
          const uint32_t acc = tile_i & 1;
          if (!mbar_wait_warp(&s.q_full[st], phase, ctx, kH2oMma) ||
              !mbar_wait_warp(&s.acc_empty[acc], ((tile_i >> 1) & 1) ^ 1, ctx, kH2oMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t q_lo = (smem_u32(s.q[st]) >> 4) | kLbo;
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t off = static_cast<uint32_t>(kk >> 2) * (kHalfBytes >> 4) + static_cast<uint32_t>(kk & 3) * 2u;
              umma_ss_f16(tmem + acc * 128, (static_cast<uint64_t>(kDescHi) << 32) | (k_lo + off),
                          (static_cast<uint64_t>(kDescHi) << 32) | (q_lo + off), idesc, kk > 0 ? 1u : 0u);
            }
            umma_commit(&s.q_empty[st]);
            umma_commit(&s.acc_full[acc]);
          }
          if (++st == kH2oStages) {
            st = 0;
            phase ^= 1;
          }
        }
        if (ok && leader) umma_commit(&s.k_empty);
      }
      __syncwarp();
      if (s.abort_flag && lane == 0) {
        umma_commit(&s.drain);
        mbar_wait(&s.drain, 0, ctx, kH2oDrain);
      }
    }
    __syncwarp();
  } else if (warp >= 4 && run) {
    // ---------------- consumers ----------------
    const int grp = (warp - 4) >> 2;              // 0 or 1
    const int key_in_tile = (warp & 3) * 32 + lane;
    const uint32_t tacc = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(grp * 128);
    const int past = p.Skv - p.Sq;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t tile_base = 0;  // global tile counter at the start of the item (same sequence as the MMA warp)
    for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x) {
      H2oItem it;
      h2o_get_item(p, g, it);
      const int key = it.k0 + key_in_tile;
      const int ntiles = p.nqb - it.qt0;
      float sum = 0.f;
      const float* lse_row = p.lse + (static_cast<long long>(it.b) * p.Hq + it.hq) * p.Sq;
      for (int t = 0; t < ntiles; ++t) {
        if (((tile_base + t) & 1u) != static_cast<uint32_t>(grp)) continue;
        const int q0 = (it.qt0 + t) * 128;
        if (!mbar_wait_warp(&s.acc_full[grp], acc_phase, ctx, kH2oCons)) {
          ok = false;
          break;
        }
        acc_phase ^= 1;
        tc_fence_after();
        // causal: key visible to query q iff key <= q + past  <=>  q >= key - past
        const int q_min = p.causal ? (key - past) : 0;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tacc + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            // the LSE address is the same for every lane: one broadcast load per query
            const int q = q0 + c * 32 + e;
            const float lse2 = (q < p.Sq) ? __ldg(lse_row + q) * 1.4426950408889634f : INFINITY;
            const float pr = fast_exp2(fmaf(__uint_as_float(r[e]), p.scale_log2, -lse2));
            sum += (q >= q_min) ? pr : 0.f;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.acc_empty[grp]);
      }
      tile_base += static_cast<uint32_t>(ntiles);
      // the two groups add their halves into the zero-initialised output (two commutative adds)
      if (key < p.Skv) atomicAdd(p.score + (static_cast<long long>(it.b) * p.Hq + it.hq) * p.Skv + key, sum);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

template <typename T, int D>
static int launch_h2o(const H2oParams& p, int grid, const DeviceState* st, cudaStream_t stream) {
  using Smem = H2oSmem<D>;
  auto kernel = h2o_score_kernel<T, D>;
  static bool configured[64] = {};
  if (!configured[st->device & 63]) {
    HB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
    configured[st->device & 63] = true;
  }
  kernel<<<grid, kH2oThreads, sizeof(Smem), stream>>>(p);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

static int h2o_impl(const hb_h2o_args* a) {
  if (a == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_h2o_score: args is NULL");
  if (a->B < 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Sq < 0 || a->Skv < 0 || a->D <= 0)
    return set_error(HB_ERR_BAD_ARG, "hb_h2o_score: negative or zero extent");
  if (a->Hq % a->Hkv != 0) return set_error(HB_ERR_BAD_ARG, "hb_h2o_score: Hq is not a multiple of Hkv");
  if (a->dtype != HB_BF16 && a->dtype != HB_FP16)
    return set_error(HB_ERR_UNSUPPORTED, "hb_h2o_score: dtype %d not supported (bf16, fp16)", a->dtype);
  if (a->D != 64 && a->D != 128) return set_error(HB_ERR_UNSUPPORTED, "hb_h2o_score: head_dim %d not supported", a->D);
  if (a->B == 0 || a->Skv == 0) return HB_OK;
  if (a->causal && a->Skv < a->Sq) return set_error(HB_ERR_UNSUPPORTED, "hb_h2o_score: causal needs Skv >= Sq");
  if (a->q == nullptr || a->k == nullptr || a->lse == nullptr || a->score == nullptr)
    return set_error(HB_ERR_BAD_ARG, "hb_h2o_score: q, k, lse and score must be non-NULL");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  HB_CUDA_CHECK(cudaMemsetAsync(a->score, 0, sizeof(float) * (size_t)a->B * a->Hq * a->Skv, stream));
  if (a->Sq == 0) return HB_OK;
  H2oParams p;
  memset(&p, 0, sizeof(p));
  const size_t es = 2;
  const CUtensorMapDataType dt = a->dtype == HB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const uint32_t box[4] = {64, 128, 1, 1};
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
  p.lse = a->lse;
  p.score = a->score;
  p.status = st->status_word;
  p.B = a->B;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.Sq = a->Sq;
  p.Skv = a->Skv;
  p.group = a->Hq / a->Hkv;
  p.causal = a->causal ? 1 : 0;
  p.nkb = (a->Skv + 127) / 128;
  p.nqb = (a->Sq + 127) / 128;
  const long long total = (long long)a->B * a->Hq * p.nkb;
  if (total > 0x7fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_h2o_score: problem too large");
  p.total_items = (int)total;
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / sqrtf((float)a->D);
  p.scale_log2 = scale * 1.4426950408889634f;
  const int grid = (int)std::min<long long>(total, st->sm_count);
  if (a->dtype == HB_BF16)
    return a->D == 128 ? launch_h2o<__nv_bfloat16, 128>(p, grid, st, stream) : launch_h2o<__nv_bfloat16, 64>(p, grid, st, stream);
  return a->D == 128 ? launch_h2o<__half, 128>(p, grid, st, stream) : launch_h2o<__half, 64>(p, grid, st, stream);
}

}  // namespace hb

extern "C" int hb_h2o_score(const hb_h2o_args* args) {
  hb::clear_error();
  return hb::h2o_impl(args);
}
