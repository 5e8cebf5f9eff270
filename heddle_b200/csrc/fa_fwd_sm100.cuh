// FlashAttention forward for sm_100a (B200): a fixed warp-specialised schedule.
//
// Arithmetic follows the reference template Heddle/heddle/tileop/flash_attention.py:20-143
// (scores scaled by softmax_scale*log2(e), online row max / row sum with exp2, P
// rounded to the input dtype before the PV product, O divided by the row sum at the
// end) and its LSE twin (:158-300).  The Hopper pipeline the reference derives with
// CP-SAT / TileLang passes is replaced by this schedule, per CTA (512 threads):
//
//   warps 0-3   softmax warpgroup for query tile 0 (128 rows, one row per thread)
//   warps 4-7   softmax warpgroup for query tile 1
//   warps 8-11  correction warpgroup: rescales O in TMEM when a row max moved,
//               final O / l, LSE, conversion and the global store
//   warp  12    MMA issuer (warp-uniform loop, one elected lane issues): S = Q K^T (operands in
//               shared memory) and O += P V (P read from TMEM, V MN-major in shared
//               memory); accumulators live in TMEM
//   warp  13    TMA producer: Q tiles and a ring of K/V tiles behind mbarriers
//
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_i is
// written over the first 64 (16-bit) columns of S_i once the row is in registers.
//
// Work: a CTA handles 256 query rows of one (batch, head) at a time and walks a
// static list of such blocks.  For causal attention block q and block (last-q) are
// paired so that every list entry costs the same; the list is head-major so the
// CTAs running at one time share K/V in L2.
#pragma once

#include "ptx_sm100.cuh"

namespace hb {

constexpr int kFaThreads = 512;
constexpr int kTileM = 128;  // query rows per softmax warpgroup
constexpr int kTileN = 128;  // keys per step

// Per-dtype constants.  16-bit inputs: P is written in the input dtype; a running max that
// grew by less than 2^8 is not adopted.  FP8 e4m3 inputs: P is requantised to e4m3 as
// p * 32 (the factor is divided out in the epilogue) and the adoption threshold is 2^3, so
// that the largest P value, 8 * 32 = 256, stays below the e4m3 maximum of 448; O is bf16.
template <typename T>
struct FaTraits {
  using Out = T;
  static constexpr int kElemBytes = 2;
  static constexpr bool kFp8 = false;
  static constexpr uint32_t kFormat = Pack2<T>::kFormat;
  static constexpr float kRescaleThreshold = 8.0f;  // log2 units
  static constexpr float kPScale = 1.0f;
};
template <>
struct FaTraits<__nv_fp8_e4m3> {
  using Out = __nv_bfloat16;
  static constexpr int kElemBytes = 1;
  static constexpr bool kFp8 = true;
  static constexpr uint32_t kFormat = 0;  // e4m3 in kind::f8f6f4
  static constexpr float kRescaleThreshold = 3.0f;
  static constexpr float kPScale = 32.0f;
};

// Optional phase tracing (compiled in with -DHB_FA_TRACE only): lane 0 of selected warps of
// CTA 0 appends (clock64 << 8 | code) records to a caller-provided, zero-filled buffer, 4096 slots
// per region (slot 0 unused); region 15 holds the CTA's start and end clocks.  A record costs
// roughly 100-150 cycles, so compare traces only with traces of the same mask.
#ifdef HB_FA_TRACE
#ifndef HB_TRACE_MASK
#define HB_TRACE_MASK 0xffffffffu  // bit c set: records with code c are kept
#endif
#define HB_TRACE_DECL(p, region)                                                                          \
  unsigned long long* hb_tr =                                                                             \
      ((p).trace != nullptr && blockIdx.x == 0 && (threadIdx.x & 31) == 0) ? (p).trace + (region) * 4096 + 1 : nullptr; \
  unsigned long long* const hb_tr_end = hb_tr + 4090;
#define HB_TRACE(p, region, code)                                                           \
  do {                                                                                      \
    if (((HB_TRACE_MASK >> (code)) & 1u) && hb_tr != nullptr && hb_tr < hb_tr_end) {        \
      *hb_tr++ = (static_cast<unsigned long long>(clock64()) << 8) | (code);                \
    }                                                                                       \
  } while (0)
#else
#define HB_TRACE_DECL(p, region)
#define HB_TRACE(p, region, code) \
  do {                            \
  } while (0)
#endif

enum FaRole : uint32_t { kRoleSoftmax = 1, kRoleCorrection = 2, kRoleMma = 3, kRoleTma = 4, kRoleDrain = 5 };

struct alignas(64) FaParams {
  CUtensorMap tm_q;
  CUtensorMap tm_k;
  CUtensorMap tm_v;
  void* o;
  float* lse;
  uint32_t* status;
  unsigned long long* trace;  // phase trace buffer (tracing builds only), else NULL
  long long o_sb, o_sh, o_ss;  // elements
  int B, Hq, Hkv, Sq, Skv;
  int group;        // Hq / Hkv
  int causal;
  int nqb;          // 256-row query blocks per head
  int npairs;       // ceil(nqb / 2)
  int total_pairs;  // B * Hq * npairs
  int nkv;          // 128-key tiles
  float scale_log2; // softmax_scale * log2(e) (times q_scale * k_scale for FP8)
  float out_scale;  // multiplies O / l in the epilogue (v_scale / P scale for FP8, else 1)
};

template <typename T, int D, int NS>
struct FaSmem {
  static constexpr int kTileBytes = kTileM * D * FaTraits<T>::kElemBytes;
  alignas(1024) uint8_t q[2][kTileBytes];
  alignas(1024) uint8_t kv[NS][kTileBytes];
  float alpha[2][kTileM];   // per-step rescale factor; carries the final row sum at the end of a block
  float stat_m[2][kTileM];  // final row max
  uint64_t q_full[2], q_empty[2];
  uint64_t kv_full[NS], kv_empty[NS];
  uint64_t s_full[2];     // MMA -> softmax: S_i holds the scores of the next step
  uint64_t p_full[2];     // softmax + correction -> MMA: P_i written and O_i rescaled
  uint64_t corr_full[2];  // softmax -> correction: alpha (or final l, m) published
  uint64_t o_full[2];     // MMA -> correction: O_i complete
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct FaItem {
  int b, hq, hkv, q0;
  int n[2];  // key tiles each query tile visits (0 = tile entirely past Sq)
};

// Entry `g` of the static work list, first (half = 0) or second block of the pair.
__device__ __forceinline__ bool fa_get_item(const FaParams& p, int g, int half, FaItem& it) {
  const int pair = g % p.npairs;
  const int bh = g / p.npairs;
  const int qb_hi = p.nqb - 1 - pair;
  const int qb = half == 0 ? qb_hi : pair;
  if (half == 1 && pair == qb_hi) return false;
  it.b = bh / p.Hq;
  it.hq = bh - it.b * p.Hq;
  it.hkv = it.hq / p.group;
  it.q0 = qb * (2 * kTileM);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r0 = it.q0 + kTileM * i;
    if (r0 >= p.Sq) {
      it.n[i] = 0;
    } else if (p.causal) {
      const int last = min(r0 + kTileM - 1, p.Sq - 1) + (p.Skv - p.Sq);
      it.n[i] = min(p.nkv, last / kTileN + 1);
    } else {
      it.n[i] = p.nkv;
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------
// softmax warpgroup (tile i): one query row per thread
// ------------------------------------------------------------------------------------
template <typename T, int D, int NS>
__device__ __forceinline__ void fa_softmax_role(const FaParams& p, FaSmem<T, D, NS>& s, const AbortCtx& ctx,
                                                uint32_t tmem, int i) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = threadIdx.x & (kTileM - 1);
  const uint32_t tS = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(i * kTileN);
  const float scale_log2 = p.scale_log2;
  uint32_t s_cnt = 0, p_cnt = 0;  // completed s_full waits / own p_full arrivals
  HB_TRACE_DECL(p, warp)

  for (int g = blockIdx.x; g < p.total_pairs; g += gridDim.x) {
    for (int half = 0; half < 2; ++half) {
      FaItem it;
      if (!fa_get_item(p, g, half, it)) continue;
      const int n = it.n[i];
      if (n == 0) continue;
      const int tile_pos0 = it.q0 + kTileM * i + (p.Skv - p.Sq);  // key position the first row may see up to
      const int row_pos = tile_pos0 + row;
      float m = -INFINITY, l = 0.f;

      for (int j = 0; j < n; ++j) {
        HB_TRACE(p, warp, 0);
        if (!mbar_wait_warp(&s.s_full[i], s_cnt & 1, ctx, kRoleSoftmax)) return;
        ++s_cnt;
        tc_fence_after();
        HB_TRACE(p, warp, 1);

        uint32_t v[kTileN];  // fp32 scores of this row, as raw bits
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, &v[c * 32]);
        tmem_wait_ld();
        HB_TRACE(p, warp, 2);

        const int col0 = j * kTileN;
        const bool need_mask = (col0 + kTileN > p.Skv) || (p.causal && (col0 + kTileN - 1 > tile_pos0));
        if (need_mask) {
          int lim = p.Skv - 1 - col0;
          if (p.causal) lim = min(lim, row_pos - col0);
#pragma unroll
          for (int c = 0; c < kTileN; ++c) v[c] = (c <= lim) ? v[c] : 0xff800000u;  // -inf
        }

        float mx0 = __uint_as_float(v[0]), mx1 = __uint_as_float(v[1]);
        float mx2 = __uint_as_float(v[2]), mx3 = __uint_as_float(v[3]);
#pragma unroll
        for (int c = 4; c < kTileN - 4; c += 8) {
          mx0 = max3(mx0, __uint_as_float(v[c]), __uint_as_float(v[c + 1]));
          mx1 = max3(mx1, __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
          mx2 = max3(mx2, __uint_as_float(v[c + 4]), __uint_as_float(v[c + 5]));
          mx3 = max3(mx3, __uint_as_float(v[c + 6]), __uint_as_float(v[c + 7]));
        }
        mx0 = max3(mx0, __uint_as_float(v[kTileN - 4]), __uint_as_float(v[kTileN - 3]));
        mx1 = max3(mx1, __uint_as_float(v[kTileN - 2]), __uint_as_float(v[kTileN - 1]));
        const float row_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));

        // New running max; a max that moved by less than the threshold is not adopted,
        // so O needs no rescale for it (l and O stay relative to the same stale max).
        // Branch-free: m = -inf (first step) gives diff = -inf -> adopt, alpha = 0;
        // m_cand = -inf (nothing visible yet) gives NaN comparisons -> keep, alpha = 1.
        const float m_cand = fmaxf(m, row_max);
        const float diff = (m - m_cand) * scale_log2;
        const bool adopt = diff < -FaTraits<T>::kRescaleThreshold;
        const float alpha = adopt ? fast_exp2(diff) : 1.f;
        m = adopt ? m_cand : m;
        const float m_scaled = (m == -INFINITY) ? 0.f : m * scale_log2;

        // Publish alpha for the correction warpgroup as early as possible.  The slot is free by
        // construction: S(j) only exists because PV(j-1) was issued, which needed the correction
        // warpgroup's arrival for step j-1, which it makes after reading alpha(j-1).  Step 0 has
        // no O to rescale: nothing is written or signalled (the slot may still hold the previous
        // block's row sum, which the correction warpgroup reads in its epilogue).
        if (j > 0) {
          s.alpha[i][row] = alpha;
          __syncwarp();
          if (lane == 0) mbar_arrive(&s.corr_full[i]);
        }
        HB_TRACE(p, warp, 3);

        // p = exp2(s * scale - m): scale-and-subtract and the row sum run on packed fp32 pairs
        // (half the FMA-pipe instructions), the exponentials on the MUFU, one per score.
        float sum0, sum1, sum2, sum3;
        {
          // FP8: P is stored as p * kPScale; the power of two is added to the exponent instead of
          // multiplying each value, so the sums below are kPScale times the row sum (divided out
          // once, when the block's row sum is published)
          constexpr float kPShift = FaTraits<T>::kFp8 ? 5.0f : 0.0f;
          static_assert(!FaTraits<T>::kFp8 || FaTraits<T>::kPScale == 32.0f, "kPShift is log2(kPScale)");
          const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nm2 = pack_f32x2(kPShift - m_scaled, kPShift - m_scaled);
          uint64_t sa = pack_f32x2(0.f, 0.f), sb = pack_f32x2(0.f, 0.f);
          constexpr int kChunk = FaTraits<T>::kFp8 ? 64 : 32;  // scores per 16 packed TMEM columns
#pragma unroll
          for (int q = 0; q < kTileN / kChunk; ++q) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < kChunk; e += 4) {
              const int c = q * kChunk + e;
              const uint64_t x0 = fma_f32x2(pack_f32x2(__uint_as_float(v[c]), __uint_as_float(v[c + 1])), sc2, nm2);
              const uint64_t x1 = fma_f32x2(pack_f32x2(__uint_as_float(v[c + 2]), __uint_as_float(v[c + 3])), sc2, nm2);
              float a0, a1, b0, b1;
              unpack_f32x2(x0, a0, a1);
              unpack_f32x2(x1, b0, b1);
              a0 = fast_exp2(a0);
              a1 = fast_exp2(a1);
              if (FaTraits<T>::kFp8 && (e & 4) != 0) {
                // FP8: the MMAs are half as long, the softmax is what bounds the step; a quarter of
                // the exponentials go to the FMA pipe (+2.6 % measured; no gain for 16-bit types)
                exp2_poly_f32x2(x1, b0, b1);
              } else {
                b0 = fast_exp2(b0);
                b1 = fast_exp2(b1);
              }
              sa = add_f32x2(sa, pack_f32x2(a0, a1));
              sb = add_f32x2(sb, pack_f32x2(b0, b1));
              if constexpr (FaTraits<T>::kFp8) {
                // e4m3 P: four values per TMEM column (already scaled by kPScale)
                pk[e / 4] = pack4_e4m3(a0, a1, b0, b1);
              } else {
                pk[e / 2] = Pack2<T>::pack(a0, a1);
                pk[e / 2 + 1] = Pack2<T>::pack(b0, b1);
              }
            }
            tmem_st16(tS + q * 16, pk);
          }
          unpack_f32x2(sa, sum0, sum1);
          unpack_f32x2(sb, sum2, sum3);
        }
        l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));
        HB_TRACE(p, warp, 4);

        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.p_full[i]);
        ++p_cnt;
        HB_TRACE(p, warp, 5);
      }

      // Final row statistics for the epilogue, in the alpha slot.  The last alpha must have been
      // consumed first: the correction warpgroup arrives on p_full after reading it (and, for a
      // one-step block, after the previous block's epilogue read this slot).
      if (!mbar_wait_warp(&s.p_full[i], (p_cnt & 1) ^ 1, ctx, kRoleSoftmax)) return;
      s.alpha[i][row] = l * (1.0f / FaTraits<T>::kPScale);
      s.stat_m[i][row] = m;
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.corr_full[i]);
    }
  }
}

// ------------------------------------------------------------------------------------
// correction warpgroup
// ------------------------------------------------------------------------------------
template <typename T, int D, int NS>
__device__ __forceinline__ void fa_correction_role(const FaParams& p, FaSmem<T, D, NS>& s, const AbortCtx& ctx,
                                                   uint32_t tmem) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = threadIdx.x & (kTileM - 1);
  const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
  uint32_t c_cnt[2] = {0, 0}, o_cnt[2] = {0, 0};
  HB_TRACE_DECL(p, warp)

  for (int g = blockIdx.x; g < p.total_pairs; g += gridDim.x) {
    for (int half = 0; half < 2; ++half) {
      FaItem it;
      if (!fa_get_item(p, g, half, it)) continue;
      const int nmax = max(it.n[0], it.n[1]);

      for (int j = 0; j < nmax; ++j) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (j >= it.n[i]) continue;
          float a = 1.f;
          if (j > 0) {
            if (!mbar_wait_warp(&s.corr_full[i], c_cnt[i] & 1, ctx, kRoleCorrection)) return;
            ++c_cnt[i];
            a = s.alpha[i][row];
          }
          HB_TRACE(p, warp, 20 + i);
          if (j > 0 && __any_sync(0xffffffffu, a != 1.f)) {
            tc_fence_after();
            const uint32_t tO = tmem + lane_off + 256u + static_cast<uint32_t>(i * 128);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t r[32];
              tmem_ld32(tO + c * 32, r);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * a);
              tmem_st32(tO + c * 32, r);
            }
            tmem_wait_st();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s.p_full[i]);
          HB_TRACE(p, warp, 22 + i);
        }
      }

      // epilogue: O_i / l, LSE, convert, store
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (it.n[i] == 0) continue;
        if (!mbar_wait_warp(&s.corr_full[i], c_cnt[i] & 1, ctx, kRoleCorrection)) return;
        ++c_cnt[i];
        const float l = s.alpha[i][row];
        const float m = s.stat_m[i][row];
        if (!mbar_wait_warp(&s.o_full[i], o_cnt[i] & 1, ctx, kRoleCorrection)) return;
        ++o_cnt[i];
        tc_fence_after();

        const int qrow = it.q0 + kTileM * i + row;
        const bool live = qrow < p.Sq;
        using Out = typename FaTraits<T>::Out;
        const float inv_l = (l > 0.f) ? (p.out_scale / l) : 0.f;
        Out* orow = static_cast<Out*>(p.o) + it.b * p.o_sb + it.hq * p.o_sh + static_cast<long long>(qrow) * p.o_ss;
        const uint32_t tO = tmem + lane_off + 256u + static_cast<uint32_t>(i * 128);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          __syncwarp();  // reconverge after the predicated stores of the previous chunk
          tmem_ld32(tO + c * 32, r);
          tmem_wait_ld();
          if (live) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 w;
              w.x = Pack2<Out>::pack(__uint_as_float(r[e]) * inv_l, __uint_as_float(r[e + 1]) * inv_l);
              w.y = Pack2<Out>::pack(__uint_as_float(r[e + 2]) * inv_l, __uint_as_float(r[e + 3]) * inv_l);
              w.z = Pack2<Out>::pack(__uint_as_float(r[e + 4]) * inv_l, __uint_as_float(r[e + 5]) * inv_l);
              w.w = Pack2<Out>::pack(__uint_as_float(r[e + 6]) * inv_l, __uint_as_float(r[e + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + c * 32 + e) = w;
            }
          }
        }
        if (live && p.lse != nullptr) {
          // natural-log LSE of the scaled, masked scores
          const float lse2 = (l > 0.f) ? (m * p.scale_log2 + fast_log2(l)) : -INFINITY;
          p.lse[(static_cast<long long>(it.b) * p.Hq + it.hq) * p.Sq + qrow] = lse2 * 0.6931471805599453f;
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// MMA issuer (one warp; an elected lane issues)
// ------------------------------------------------------------------------------------
template <typename T, int D, int NS>
__device__ __forceinline__ void fa_mma_role(const FaParams& p, FaSmem<T, D, NS>& s, const AbortCtx& ctx,
                                            uint32_t tmem) {
  using Tr = FaTraits<T>;
  constexpr uint32_t kFmt = Tr::kFormat;
  constexpr uint32_t idesc_qk = make_idesc(kFmt, kTileM, kTileN, 0, 0);
  constexpr uint32_t idesc_pv = make_idesc(kFmt, kTileM, D, 0, 1);
  constexpr uint32_t kSubBytes = kTileM * 128;            // one 128-byte-wide, 128-row sub-tile
  constexpr int kQkSteps = D * Tr::kElemBytes / 32;       // each MMA consumes 32 bytes of head_dim
  constexpr int kPvSteps = kTileN * Tr::kElemBytes / 32;  // ... and 32 bytes' worth of keys of P
  constexpr uint32_t kVStep16 = (32u / Tr::kElemBytes) * 128u >> 4;  // V rows per MMA x 128 B, in 16-byte units
  // Shared-memory descriptors: the high word (SBO = 1024 B, version 1, SWIZZLE_128B) is constant;
  // the low word is (address >> 4) | (LBO >> 4) << 16 and only its address field moves per MMA.
  constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
  constexpr uint32_t kLboK = (16u >> 4) << 16;
  constexpr uint32_t kLboV = (kSubBytes >> 4) << 16;  // next 128-byte group of head_dim
  constexpr uint32_t kTile16 = FaSmem<T, D, NS>::kTileBytes >> 4;
  const uint32_t q_lo = (smem_u32(s.q[0]) >> 4) | kLboK;
  const uint32_t kv_lo = smem_u32(s.kv[0]) >> 4;
  auto desc = [](uint32_t lo) -> uint64_t { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };

  // The whole warp runs this role so that addresses and descriptors stay warp-uniform (they
  // then live in uniform registers, which is what tcgen05.mma takes); one elected lane issues.
  const bool leader = elect_one();
  auto commit = [&](uint64_t* bar) {
    if (leader) umma_commit(bar);
  };

  auto issue_qk = [&](int i, uint32_t slot) {
    const uint32_t qa = q_lo + static_cast<uint32_t>(i) * kTile16;
    const uint32_t ka = (kv_lo + slot * kTile16) | kLboK;
    const uint32_t d_tmem = tmem + static_cast<uint32_t>(i * kTileN);
    if (leader) {
#pragma unroll
      for (int kk = 0; kk < kQkSteps; ++kk) {
        // 32 bytes per step inside a 128-byte-wide sub-tile, then the next sub-tile
        constexpr uint32_t kSub = kSubBytes >> 4;
        const uint32_t off = static_cast<uint32_t>(kk >> 2) * kSub + static_cast<uint32_t>(kk & 3) * 2u;
        if constexpr (Tr::kFp8) {
          umma_ss_f8(d_tmem, desc(qa + off), desc(ka + off), idesc_qk, kk > 0 ? 1u : 0u);
        } else {
          umma_ss_f16(d_tmem, desc(qa + off), desc(ka + off), idesc_qk, kk > 0 ? 1u : 0u);
        }
      }
    }
  };
  auto issue_pv = [&](int i, uint32_t slot, uint32_t accumulate) {
    const uint32_t va = (kv_lo + slot * kTile16) | kLboV;
    const uint32_t d_tmem = tmem + 256u + static_cast<uint32_t>(i * 128);
    const uint32_t a_tmem = tmem + static_cast<uint32_t>(i * kTileN);
    if (leader) {
#pragma unroll
      for (int kk = 0; kk < kPvSteps; ++kk) {
        // per step: 8 TMEM columns of packed P, and the matching key rows of V
        if constexpr (Tr::kFp8) {
          umma_ts_f8(d_tmem, a_tmem + static_cast<uint32_t>(kk * 8), desc(va + static_cast<uint32_t>(kk) * kVStep16),
                     idesc_pv, kk > 0 ? 1u : accumulate);
        } else {
          umma_ts_f16(d_tmem, a_tmem + static_cast<uint32_t>(kk * 8), desc(va + static_cast<uint32_t>(kk) * kVStep16),
                      idesc_pv, kk > 0 ? 1u : accumulate);
        }
      }
    }
  };

  // consumer side of the K/V ring
  uint32_t slot = 0, phase = 0;
  auto advance = [&]() {
    if (++slot == NS) {
      slot = 0;
      phase ^= 1;
    }
  };
  uint32_t q_phase = 0, p_phase = 0;  // bit i = parity of tile i's barrier
  HB_TRACE_DECL(p, 12)

  for (int g = blockIdx.x; g < p.total_pairs; g += gridDim.x) {
    for (int half = 0; half < 2; ++half) {
      FaItem it;
      if (!fa_get_item(p, g, half, it)) continue;
      const int n0 = it.n[0], n1 = it.n[1];
      const int nmax = max(n0, n1);

      // step 0 scores
      uint32_t slot_k = slot;
      if (!mbar_wait_warp(&s.kv_full[slot], phase, ctx, kRoleMma)) return;
      advance();
#pragma unroll 1
      for (int i = 0; i < 2; ++i) {
        const int ni = i == 0 ? n0 : n1;
        if (ni == 0) continue;
        if (!mbar_wait_warp(&s.q_full[i], (q_phase >> i) & 1u, ctx, kRoleMma)) return;
        q_phase ^= 1u << i;
        tc_fence_after();
        issue_qk(i, slot_k);
        commit(&s.s_full[i]);
        if (ni == 1) commit(&s.q_empty[i]);
      }
      commit(&s.kv_empty[slot_k]);

      for (int j = 0; j < nmax; ++j) {
        const uint32_t slot_v = slot;
        if (!mbar_wait_warp(&s.kv_full[slot], phase, ctx, kRoleMma)) return;
        advance();
        const bool has_next = (j + 1 < nmax);
        bool k_ready = false;
        slot_k = slot;
#pragma unroll 1
        for (int i = 0; i < 2; ++i) {
          const int ni = i == 0 ? n0 : n1;
          if (j < ni) {
            HB_TRACE(p, 12, 10 + i);
            if (!mbar_wait_warp(&s.p_full[i], (p_phase >> i) & 1u, ctx, kRoleMma)) return;
            p_phase ^= 1u << i;
            tc_fence_after();
            HB_TRACE(p, 12, 12 + i);
            issue_pv(i, slot_v, j > 0 ? 1u : 0u);
            if (j == ni - 1) commit(&s.o_full[i]);
          }
          if (j + 1 < ni) {
            if (!k_ready) {
              if (!mbar_wait_warp(&s.kv_full[slot], phase, ctx, kRoleMma)) return;
              tc_fence_after();
              k_ready = true;
            }
            issue_qk(i, slot_k);
            commit(&s.s_full[i]);
            HB_TRACE(p, 12, 14 + i);
            if (j + 2 == ni) commit(&s.q_empty[i]);
          }
        }
        commit(&s.kv_empty[slot_v]);
        if (has_next) {
          commit(&s.kv_empty[slot_k]);
          advance();
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// TMA producer (one thread)
// ------------------------------------------------------------------------------------
template <typename T, int D, int NS>
__device__ __forceinline__ void fa_tma_role(const FaParams& p, FaSmem<T, D, NS>& s, const AbortCtx& ctx) {
  constexpr uint32_t kTileBytes = FaSmem<T, D, NS>::kTileBytes;
  constexpr uint32_t kSubBytes = kTileM * 128;                       // 128-byte-wide, 128-row sub-tile
  constexpr int kSubTiles = D * FaTraits<T>::kElemBytes / 128;      // sub-tiles per tile
  constexpr int kSubElems = 128 / FaTraits<T>::kElemBytes;          // head_dim elements per sub-tile
  uint32_t slot = 0, phase = 1, q_phase[2] = {1, 1};  // "empty" barriers start out free

  for (int g = blockIdx.x; g < p.total_pairs; g += gridDim.x) {
    for (int half = 0; half < 2; ++half) {
      FaItem it;
      if (!fa_get_item(p, g, half, it)) continue;
      const int nmax = max(it.n[0], it.n[1]);

      auto load_q = [&](int i) -> bool {
        if (!mbar_wait(&s.q_empty[i], q_phase[i], ctx, kRoleTma)) return false;
        q_phase[i] ^= 1;
        mbar_arrive_expect_tx(&s.q_full[i], kTileBytes);
#pragma unroll
        for (int h = 0; h < kSubTiles; ++h) {
          tma_load_4d(s.q[i] + h * kSubBytes, &p.tm_q, &s.q_full[i], h * kSubElems, it.q0 + kTileM * i, it.hq, it.b);
        }
        return true;
      };
      auto load_kv = [&](const CUtensorMap* tm, int j) -> bool {
        if (!mbar_wait(&s.kv_empty[slot], phase, ctx, kRoleTma)) return false;
        mbar_arrive_expect_tx(&s.kv_full[slot], kTileBytes);
#pragma unroll
        for (int h = 0; h < kSubTiles; ++h) {
          tma_load_4d(s.kv[slot] + h * kSubBytes, tm, &s.kv_full[slot], h * kSubElems, j * kTileN, it.hkv, it.b);
        }
        if (++slot == NS) {
          slot = 0;
          phase ^= 1;
        }
        return true;
      };

      if (it.n[0] > 0 && !load_q(0)) return;
      if (!load_kv(&p.tm_k, 0)) return;
      if (it.n[1] > 0 && !load_q(1)) return;
      for (int j = 0; j < nmax; ++j) {
        if (!load_kv(&p.tm_v, j)) return;
        if (j + 1 < nmax && !load_kv(&p.tm_k, j + 1)) return;
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------
template <typename T, int D, int NS>
__global__ void __launch_bounds__(kFaThreads, 1) fa_fwd_kernel(const __grid_constant__ FaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using Smem = FaSmem<T, D, NS>;
  Smem& s = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{&s.abort_flag, p.status};

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.q_full[i], 1);
      mbar_init(&s.q_empty[i], 1);
      mbar_init(&s.s_full[i], 1);
      mbar_init(&s.p_full[i], 8);
      mbar_init(&s.corr_full[i], 4);
      mbar_init(&s.o_full[i], 1);
    }
    for (int i = 0; i < NS; ++i) {
      mbar_init(&s.kv_full[i], 1);
      mbar_init(&s.kv_empty[i], 1);
    }
    mbar_init(&s.drain, 1);
    fence_mbar_init();
    if ((smem_u32(smem_raw) & 1023u) != 0u) raise_abort(ctx, kStatusSmemMisaligned);
  }
  if (warp == 13 && lane == 0) {
    prefetch_tensormap(&p.tm_q);
    prefetch_tensormap(&p.tm_k);
    prefetch_tensormap(&p.tm_v);
  }
  if (warp == 12) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const bool run = (s.abort_flag == 0);
#ifdef HB_FA_TRACE
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[15 * 4096 + 1] = clock64();
#endif

  // setmaxnreg.inc only hands out registers that other warpgroups of this CTA have returned with
  // setmaxnreg.dec, so the budget has to balance or the increase waits for ever: 512 threads start with 128
  // registers each; eight softmax warps grow by 56, four correction warps return 48 and the last four 64
  static_assert(8 * 32 * (184 - 128) <= 4 * 32 * (128 - 80) + 4 * 32 * (128 - 64), "setmaxnreg budget does not balance");
  if (warp < 8) {
    reg_inc<184>();
    if (run) fa_softmax_role<T, D, NS>(p, s, ctx, tmem, warp >> 2);
  } else if (warp < 12) {
    reg_dec<80>();
    if (run) fa_correction_role<T, D, NS>(p, s, ctx, tmem);
  } else {
    reg_dec<64>();
    if (run && warp == 12) {
      fa_mma_role<T, D, NS>(p, s, ctx, tmem);
      __syncwarp();
      if (s.abort_flag && lane == 0) {
        // aborting: let the tensor pipe drain before TMEM is released
        umma_commit(&s.drain);
        mbar_wait(&s.drain, 0, ctx, kRoleDrain);
      }
    } else if (run && warp == 13 && lane == 0) {
      fa_tma_role<T, D, NS>(p, s, ctx);
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
#ifdef HB_FA_TRACE
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[15 * 4096 + 2] = clock64();
#endif
  if (warp == 12) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace hb
