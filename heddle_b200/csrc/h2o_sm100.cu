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
//   warps 0-3   consumer group 0: even query tiles      exp2(s*scale*log2e - LSE*log2e), masks,
//   warps 4-7   consumer group 1: odd query tiles       per-key running sum
//   warp 8      TMA: the K tile (A operand) once per work item, a ring of Q tiles (B operand)
//   warp 9      MMA: tcgen05.mma M=128 (keys) N=128 (queries), two TMEM accumulator buffers
// Each consumer warp stages the 128 LSE values of its query tile in shared memory (prefetched one
// tile ahead) and reads them back as broadcast 16-byte loads.
#include "host_common.h"
#include "ptx_sm100.cuh"

#include <algorithm>
#include <cmath>

namespace hb {

constexpr int kH2oThreads = 384;  // warps 10, 11 only complete the third warpgroup for setmaxnreg
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
  int npairs;      // ceil(nkb / 2)
  int nqb;         // 128-query tiles
  int total_items; // B * Hq * npairs
  float scale_log2;
};

template <int D>
struct H2oSmem {
  static constexpr int kTileBytes = 128 * D * 2;
  alignas(1024) uint8_t k[kTileBytes];
  alignas(1024) uint8_t q[kH2oStages][kTileBytes];
  uint64_t k_full, k_empty;
  uint64_t q_full[kH2oStages], q_empty[kH2oStages];
  uint64_t acc_full[4], acc_empty[4];  // [consumer group * 2 + buffer]
  uint64_t drain;
  uint32_t tmem_base, abort_flag;
  alignas(16) float nlse[8][2][128];  // per consumer warp, double-buffered: -LSE * log2(e) of a query tile
};

struct H2oItem {
  int b, hq, hkv, k0, qt0;  // first key, first query tile that can see this key tile
};

// Entry `g` of the static work list, first (half = 0) or second key tile of the pair.  Under a
// causal mask key tile kb is seen by nqb - qt0(kb) query tiles, so tile `pair` (many queries) and
// tile nkb-1-pair (few) together cost the same for every pair: the persistent CTAs stay balanced.
__device__ __forceinline__ bool h2o_get_item(const H2oParams& p, int g, int half, H2oItem& it) {
  const int pair = g % p.npairs;
  const int bh = g / p.npairs;
  const int kb_hi = p.nkb - 1 - pair;
  const int kb = half == 0 ? pair : kb_hi;
  if (half == 1 && kb_hi == pair) return false;
  it.b = bh / p.Hq;
  it.hq = bh - it.b * p.Hq;
  it.hkv = it.hq / p.group;
  it.k0 = kb * 128;
  // h2o_attention.py:99-101: q_start = max(0, (k0 - past_len) / block_M)
  it.qt0 = p.causal ? max(0, (it.k0 - (p.Skv - p.Sq)) / 128) : 0;
  return true;
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
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 4);
    }
    mbar_init(&s.drain, 1);
    fence_mbar_init();
    if ((smem_u32(smem_raw) & 1023u) != 0u) raise_abort(ctx, kStatusSmemMisaligned);
    prefetch_tensormap(&p.tm_q);
    prefetch_tensormap(&p.tm_k);
  }
  if (warp == 9) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const bool run = (s.abort_flag == 0);
  constexpr uint32_t kTileBytes = Smem::kTileBytes;
  constexpr uint32_t kHalfBytes = 128 * 128;

  // the consumers hold a 128-column tile in registers: they take the registers warps 8-11 do not need
  if (warp >= 8) reg_dec<72>();
  if (warp == 8) {
    if (run && lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t st = 0, phase = 1, k_phase = 1;
      bool ok = true;
      for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1)) {
        H2oItem it;
        if (!h2o_get_item(p, u >> 1, u & 1, it)) continue;
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
  } else if (warp == 9) {
    if (run) {
      // ---------------- MMA issuer (warp-uniform, elected lane issues) ----------------
      constexpr uint32_t idesc = make_idesc(Pack2<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kLbo = (16u >> 4) << 16;
      const bool leader = elect_one();
      uint32_t st = 0, phase = 0, k_phase = 0, tile_i = 0;
      bool ok = true;
      const uint32_t k_lo = (smem_u32(s.k) >> 4) | kLbo;
      for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1)) {
        H2oItem it;
        if (!h2o_get_item(p, u >> 1, u & 1, it)) continue;
        if (!mbar_wait_warp(&s.k_full, k_phase, ctx, kH2oMma)) break;
        k_phase ^= 1;
        for (int qt = it.qt0; qt < p.nqb; ++qt, ++tile_i) {
          // tile i goes to consumer group i & 1, into that group's buffer (i >> 1) & 1
          const uint32_t acc = ((tile_i & 1u) << 1) | ((tile_i >> 1) & 1u);
          if (!mbar_wait_warp(&s.q_full[st], phase, ctx, kH2oMma) ||
              !mbar_wait_warp(&s.acc_empty[acc], ((tile_i >> 2) & 1) ^ 1, ctx, kH2oMma)) {
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
  } else if (warp < 8) {
   reg_inc<208>();
   if (run) {
    // ---------------- consumers ----------------
    const int grp = warp >> 2;                    // 0 or 1
    const int key_in_tile = (warp & 3) * 32 + lane;
    const uint32_t tacc = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(grp * 256);
    const int past = p.Skv - p.Sq;
    uint32_t cg = 0, buf = 0;  // cg: tiles this group has consumed (selects buffer and parity)
    bool ok = true;
    uint32_t tile_base = 0;  // global tile counter at the start of the item (same sequence as the MMA warp)
    const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2);
    for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1)) {
      H2oItem it;
      if (!h2o_get_item(p, u >> 1, u & 1, it)) continue;
      const int key = it.k0 + key_in_tile;
      const int ntiles = p.nqb - it.qt0;
      const float* lse_row = p.lse + (static_cast<long long>(it.b) * p.Hq + it.hq) * p.Sq;
      // -LSE in the exp2 domain of one query of a tile (the thread's own slot of the staging
      // buffer); queries past Sq get -inf, so their probability is exactly 0
      auto load_nlse = [&](int t, float (&v)[4]) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int q = (it.qt0 + t) * 128 + lane * 4 + u;
          v[u] = (q < p.Sq) ? -__ldg(lse_row + q) * 1.4426950408889634f : -INFINITY;
        }
      };
      // this group's tiles of the item: t = t_first, t_first + 2, ...
      const int t_first = static_cast<int>((tile_base ^ static_cast<uint32_t>(grp)) & 1u);
      uint64_t sa = pack_f32x2(0.f, 0.f), sb = pack_f32x2(0.f, 0.f);
      float nl[4] = {0.f, 0.f, 0.f, 0.f};
      if (t_first < ntiles) load_nlse(t_first, nl);
      for (int t = t_first; t < ntiles; t += 2) {
        // every warp stages its own copy of the tile's 128 LSE values (no cross-warp barrier);
        // the next tile's values are fetched behind this tile's math
        float4* stage = reinterpret_cast<float4*>(s.nlse[warp][buf]);
        stage[lane] = make_float4(nl[0], nl[1], nl[2], nl[3]);
        __syncwarp();
        if (t + 2 < ntiles) load_nlse(t + 2, nl);
        const float4* nl4 = stage;
        buf ^= 1;
        const int q0 = (it.qt0 + t) * 128;
        const uint32_t ab = cg & 1u;
        if (!mbar_wait_warp(&s.acc_full[grp * 2 + ab], (cg >> 1) & 1u, ctx, kH2oCons)) {
          ok = false;
          break;
        }
        ++cg;
        tc_fence_after();
        uint32_t r[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tacc + ab * 128 + c * 32, &r[c * 32]);
        tmem_wait_ld();
        // causal: key visible to query q iff key <= q + past  <=>  q >= key - past; only the
        // tile(s) on the diagonal need the test
        const bool need_mask = p.causal && (q0 < it.k0 + 127 - past);
        if (need_mask) {
          const int q_min = key - past - q0;  // first visible query of this key, tile-relative
#pragma unroll
          for (int e = 0; e < 128; ++e) r[e] = (e >= q_min) ? r[e] : 0xff800000u;  // -inf -> p = 0
        }
#pragma unroll
        for (int e = 0; e < 128; e += 4) {
          const float4 l4 = nl4[e >> 2];
          const uint64_t x0 = fma_f32x2(pack_f32x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), sc2, pack_f32x2(l4.x, l4.y));
          const uint64_t x1 = fma_f32x2(pack_f32x2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3])), sc2, pack_f32x2(l4.z, l4.w));
          float a0, a1, b0, b1;
          unpack_f32x2(x0, a0, a1);
          unpack_f32x2(x1, b0, b1);
          sa = add_f32x2(sa, pack_f32x2(fast_exp2(a0), fast_exp2(a1)));
          if ((e & 4) != 0) {
            // every fourth pair on the FMA pipe: two consumer warps share each MUFU, which is the
            // busiest unit of this kernel (relative error 7.5e-5)
            exp2_poly_f32x2(x1, b0, b1);
            sb = add_f32x2(sb, pack_f32x2(b0, b1));
          } else {
            sb = add_f32x2(sb, pack_f32x2(fast_exp2(b0), fast_exp2(b1)));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.acc_empty[grp * 2 + ab]);
      }
      tile_base += static_cast<uint32_t>(ntiles);
      float s0, s1, s2, s3;
      unpack_f32x2(sa, s0, s1);
      unpack_f32x2(sb, s2, s3);
      const float sum = (s0 + s1) + (s2 + s3);
      // the two groups add their halves into the zero-initialised output (two commutative adds)
      if (key < p.Skv) atomicAdd(p.score + (static_cast<long long>(it.b) * p.Hq + it.hq) * p.Skv + key, sum);
    }
   }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
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
  p.npairs = (p.nkb + 1) / 2;
  const long long total = (long long)a->B * a->Hq * p.npairs;
  if (total > 0x3fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_h2o_score: problem too large");
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
