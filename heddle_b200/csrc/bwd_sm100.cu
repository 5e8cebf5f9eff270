// FlashAttention backward for sm_100a, split into the three kernels whose interface the reference
// sketches in Heddle/heddle/frontend/bwd_separator.py:366-455 (preprocess -> dK,dV -> dQ; every
// output is written by exactly one CTA, no atomic adds):
//
//   delta[b,h,q] = sum_d O * dO                                        (hb_fa_bwd_preprocess)
//   P = exp(scale * Q K^T + mask - LSE);  dP = dO V^T;  dS = P o (dP - delta)
//   dV = P^T dO;  dK = scale * dS^T Q                                   (hb_fa_bwd_dkdv)
//   dQ = scale * dS K                                                   (hb_fa_bwd_dq)
//
// Both main kernels recompute S and dP with tcgen05.mma into TMEM and keep their accumulators
// there.  The dK/dV kernel issues the products transposed (S^T = K Q^T, dP^T = V dO^T), so that a
// key is a TMEM lane: P^T and dS^T are then exactly the A operands (from TMEM) of dV += P^T dO
// and dK += dS^T Q, and each thread owns one key row.  The dQ kernel keeps queries on the lanes.
// One CTA (192 threads): warps 0-3 turn scores into P / dS (one row per thread), warp 4 is the TMA
// producer, warp 5 issues the MMAs.  The schedule is a plain one (S and dP single-buffered): this is
// a first, correct version of a "next" row, not a tuned one.  head_dim 128, bf16 / fp16.
#include "host_common.h"
#include "ptx_sm100.cuh"

#include <algorithm>
#include <cmath>

namespace hb {

constexpr int kBwdThreads = 192;
constexpr int kBwdStages = 2;
constexpr int kBwdD = 128;
constexpr uint32_t kBwdTileBytes = 128 * kBwdD * 2;  // one 128-row tile of a 16-bit tensor
enum BwdRole : uint32_t { kBwdTma = 0x41, kBwdMma = 0x42, kBwdCons = 0x43, kBwdDrain = 0x44 };

struct alignas(64) BwdParams {
  CUtensorMap tm_q, tm_k, tm_v, tm_do;
  const float* lse;    // [B, Hq, Sq], natural log
  const float* delta;  // [B, Hq, Sq]
  void* dq;            // [B, Hq, Sq, D] contiguous
  void* dk;            // [B, Hkv, Skv, D] contiguous
  void* dv;
  uint32_t* status;
  int B, Hq, Hkv, Sq, Skv;
  int group, causal;
  int nkb, nqb;     // 128-row key / query tiles
  int total_items;  // dkdv: B * Hkv * nkb;  dq: B * Hq * nqb
  float scale_log2, scale;
};

struct BwdSmem {
  alignas(1024) uint8_t fixed[2][kBwdTileBytes];              // dkdv: K, V of the item;  dq: Q, dO of the item
  alignas(1024) uint8_t ring[kBwdStages][2][kBwdTileBytes];   // dkdv: {Q, dO} per step;  dq: {K, V} per step
  uint64_t fixed_full, fixed_empty;
  uint64_t ring_full[kBwdStages], ring_empty[kBwdStages];
  uint64_t s_full;     // MMA -> consumers: scores and dP of the step are in TMEM
  uint64_t p_ready;    // consumers -> MMA: P / dS written back to TMEM
  uint64_t acc_full;   // MMA -> consumers: the item's accumulators are complete
  uint64_t acc_empty;  // consumers -> MMA: accumulators read out
  uint64_t drain;
  uint32_t tmem_base, abort_flag;
  alignas(16) float stage[4][2][2][128];  // dkdv: per consumer warp, double-buffered {-LSE*log2e, delta} of a query tile
};

// Shared-memory descriptor pieces (same conventions as the forward kernel)
constexpr uint32_t kBwdDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t kBwdLboK = (16u >> 4) << 16;                // K-major operand
constexpr uint32_t kBwdSub16 = (128u * 128u) >> 4;             // one 128-byte-wide, 128-row sub-tile in 16-byte units
constexpr uint32_t kBwdLboMn = kBwdSub16 << 16;                // MN-major operand: next 64 head_dim columns
__device__ __forceinline__ uint64_t bwd_desc(uint32_t lo) { return (static_cast<uint64_t>(kBwdDescHi) << 32) | lo; }

// D[128 x 128] (+)= A[128 x 128(K = head_dim)] . B[128 x 128(K = head_dim)]^T, both operands K-major tiles in smem
template <typename T>
__device__ __forceinline__ void bwd_mma_kk(uint32_t d_tmem, const void* a_tile, const void* b_tile) {
  constexpr uint32_t idesc = make_idesc(Pack2<T>::kFormat, 128, 128, 0, 0);
  const uint32_t a_lo = (smem_u32(a_tile) >> 4) | kBwdLboK, b_lo = (smem_u32(b_tile) >> 4) | kBwdLboK;
#pragma unroll
  for (int kk = 0; kk < kBwdD / 16; ++kk) {
    const uint32_t off = static_cast<uint32_t>(kk >> 2) * kBwdSub16 + static_cast<uint32_t>(kk & 3) * 2u;
    umma_ss_f16(d_tmem, bwd_desc(a_lo + off), bwd_desc(b_lo + off), idesc, kk > 0 ? 1u : 0u);
  }
}
// D[128 x head_dim] (+)= A[128 x 128] (packed 16-bit, in TMEM) . B[128(K) x head_dim] (a row tile in smem, MN-major)
template <typename T>
__device__ __forceinline__ void bwd_mma_ts(uint32_t d_tmem, uint32_t a_tmem, const void* b_tile, uint32_t accumulate) {
  constexpr uint32_t idesc = make_idesc(Pack2<T>::kFormat, 128, kBwdD, 0, 1);
  const uint32_t b_lo = (smem_u32(b_tile) >> 4) | kBwdLboMn;
#pragma unroll
  for (int kk = 0; kk < 128 / 16; ++kk) {
    umma_ts_f16(d_tmem, a_tmem + static_cast<uint32_t>(kk * 8), bwd_desc(b_lo + static_cast<uint32_t>(kk) * 128u), idesc,
                kk > 0 ? 1u : accumulate);
  }
}

__device__ __forceinline__ void bwd_load_tile(void* dst, const CUtensorMap* tm, uint64_t* bar, int row0, int h, int b) {
#pragma unroll
  for (int hh = 0; hh < kBwdD / 64; ++hh)
    tma_load_4d(static_cast<uint8_t*>(dst) + hh * (128 * 128), tm, bar, hh * 64, row0, h, b);
}

template <typename T>
__device__ __forceinline__ void bwd_store_row(T* dst, const uint32_t (&r)[32], float mul) {
#pragma unroll
  for (int e = 0; e < 32; e += 8) {
    uint4 w;
    w.x = Pack2<T>::pack(__uint_as_float(r[e]) * mul, __uint_as_float(r[e + 1]) * mul);
    w.y = Pack2<T>::pack(__uint_as_float(r[e + 2]) * mul, __uint_as_float(r[e + 3]) * mul);
    w.z = Pack2<T>::pack(__uint_as_float(r[e + 4]) * mul, __uint_as_float(r[e + 5]) * mul);
    w.w = Pack2<T>::pack(__uint_as_float(r[e + 6]) * mul, __uint_as_float(r[e + 7]) * mul);
    *reinterpret_cast<uint4*>(dst + e) = w;
  }
}

__device__ __forceinline__ void bwd_init(BwdSmem& s, const AbortCtx& ctx, const void* smem_raw) {
  s.abort_flag = 0;
  mbar_init(&s.fixed_full, 1);
  mbar_init(&s.fixed_empty, 1);
  for (int i = 0; i < kBwdStages; ++i) {
    mbar_init(&s.ring_full[i], 1);
    mbar_init(&s.ring_empty[i], 1);
  }
  mbar_init(&s.s_full, 1);
  mbar_init(&s.p_ready, 4);
  mbar_init(&s.acc_full, 1);
  mbar_init(&s.acc_empty, 4);
  mbar_init(&s.drain, 1);
  fence_mbar_init();
  if ((smem_u32(smem_raw) & 1023u) != 0u) raise_abort(ctx, kStatusSmemMisaligned);
}

// ------------------------------------------------------------------------------------------
// dK, dV: one CTA per (batch, kv head, 128-key tile); loops over the group's query heads and the
// query tiles that can see the key tile.  TMEM: S^T [0,128) dP^T [128,256) dV [256,384) dK [384,512).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBwdThreads, 1) fa_bwd_dkdv_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  BwdSmem& s = *reinterpret_cast<BwdSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{&s.abort_flag, p.status};
  if (threadIdx.x == 0) {
    bwd_init(s, ctx, smem_raw);
    prefetch_tensormap(&p.tm_q);
    prefetch_tensormap(&p.tm_k);
    prefetch_tensormap(&p.tm_v);
    prefetch_tensormap(&p.tm_do);
  }
  if (warp == 5) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const bool run = (s.abort_flag == 0);
  const int past = p.Skv - p.Sq;

  auto item_of = [&](int g, int& b, int& hkv, int& k0, int& qt0) {
    // heaviest key tiles (lowest index under a causal mask) first
    const int kb = g % p.nkb;
    const int bh = g / p.nkb;
    b = bh / p.Hkv;
    hkv = bh - b * p.Hkv;
    k0 = kb * 128;
    qt0 = p.causal ? max(0, (k0 - past) / 128) : 0;
  };

  if (warp == 4) {
    if (run && lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t st = 0, phase = 1, f_phase = 1;
      bool ok = true;
      for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x) {
        int b, hkv, k0, qt0;
        item_of(g, b, hkv, k0, qt0);
        if (!mbar_wait(&s.fixed_empty, f_phase, ctx, kBwdTma)) break;
        f_phase ^= 1;
        mbar_arrive_expect_tx(&s.fixed_full, 2 * kBwdTileBytes);
        bwd_load_tile(s.fixed[0], &p.tm_k, &s.fixed_full, k0, hkv, b);
        bwd_load_tile(s.fixed[1], &p.tm_v, &s.fixed_full, k0, hkv, b);
        for (int hg = 0; ok && hg < p.group; ++hg) {
          const int hq = hkv * p.group + hg;
          for (int qt = qt0; qt < p.nqb; ++qt) {
            if (!mbar_wait(&s.ring_empty[st], phase, ctx, kBwdTma)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&s.ring_full[st], 2 * kBwdTileBytes);
            bwd_load_tile(s.ring[st][0], &p.tm_q, &s.ring_full[st], qt * 128, hq, b);
            bwd_load_tile(s.ring[st][1], &p.tm_do, &s.ring_full[st], qt * 128, hq, b);
            if (++st == kBwdStages) {
              st = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (run) {
      // ---------------- MMA issuer (warp-uniform, elected lane issues) ----------------
      const bool leader = elect_one();
      uint32_t st = 0, phase = 0, f_phase = 0, s_cnt = 0, items = 0;
      bool ok = true;
      for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x, ++items) {
        int b, hkv, k0, qt0;
        item_of(g, b, hkv, k0, qt0);
        if (!mbar_wait_warp(&s.fixed_full, f_phase, ctx, kBwdMma)) break;
        f_phase ^= 1;
        bool first = true;
        for (int hg = 0; ok && hg < p.group; ++hg) {
          for (int qt = qt0; qt < p.nqb; ++qt) {
            if (!mbar_wait_warp(&s.ring_full[st], phase, ctx, kBwdMma)) {
              ok = false;
              break;
            }
            tc_fence_after();
            if (leader) {
              bwd_mma_kk<T>(tmem + 0, s.fixed[0], s.ring[st][0]);    // S^T  = K Q^T
              bwd_mma_kk<T>(tmem + 128, s.fixed[1], s.ring[st][1]);  // dP^T = V dO^T
              umma_commit(&s.s_full);
            }
            __syncwarp();
            if (!mbar_wait_warp(&s.p_ready, s_cnt & 1, ctx, kBwdMma)) {
              ok = false;
              break;
            }
            ++s_cnt;
            if (first) {
              // the first accumulation of the item overwrites dV, dK: the previous item's read-out must be over
              if (!mbar_wait_warp(&s.acc_empty, (items & 1) ^ 1, ctx, kBwdMma)) {
                ok = false;
                break;
              }
            }
            tc_fence_after();
            if (leader) {
              bwd_mma_ts<T>(tmem + 256, tmem + 0, s.ring[st][1], first ? 0u : 1u);    // dV += P^T dO
              bwd_mma_ts<T>(tmem + 384, tmem + 128, s.ring[st][0], first ? 0u : 1u);  // dK += dS^T Q
              umma_commit(&s.ring_empty[st]);
            }
            __syncwarp();
            first = false;
            if (++st == kBwdStages) {
              st = 0;
              phase ^= 1;
            }
          }
        }
        if (ok && leader) {
          umma_commit(&s.acc_full);
          umma_commit(&s.fixed_empty);
        }
        __syncwarp();
      }
      __syncwarp();
      if (s.abort_flag && lane == 0) {
        umma_commit(&s.drain);
        mbar_wait(&s.drain, 0, ctx, kBwdDrain);
      }
    }
    __syncwarp();
  } else if (run) {
    // ---------------- consumers: one key per thread ----------------
    const int key_in_tile = warp * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    uint32_t s_cnt = 0, items = 0, buf = 0;
    bool ok = true;
    for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x, ++items) {
      int b, hkv, k0, qt0;
      item_of(g, b, hkv, k0, qt0);
      const int key = k0 + key_in_tile;
      for (int hg = 0; ok && hg < p.group; ++hg) {
        const int hq = hkv * p.group + hg;
        const float* lse_row = p.lse + (static_cast<long long>(b) * p.Hq + hq) * p.Sq;
        const float* dl_row = p.delta + (static_cast<long long>(b) * p.Hq + hq) * p.Sq;
        for (int qt = qt0; qt < p.nqb; ++qt) {
          // this warp's copy of the tile's per-query terms; queries past Sq get -inf, so P is exactly 0
          float* nl = s.stage[warp][buf][0];
          float* dl = s.stage[warp][buf][1];
          buf ^= 1;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int q = qt * 128 + lane * 4 + u;
            nl[lane * 4 + u] = (q < p.Sq) ? -__ldg(lse_row + q) * 1.4426950408889634f : -INFINITY;
            dl[lane * 4 + u] = (q < p.Sq) ? __ldg(dl_row + q) : 0.f;
          }
          __syncwarp();
          if (!mbar_wait_warp(&s.s_full, s_cnt & 1, ctx, kBwdCons)) {
            ok = false;
            break;
          }
          ++s_cnt;
          tc_fence_after();
          // causal: key visible to query q iff key <= q + past
          const int q_min = p.causal ? (key - past - qt * 128) : -1;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t sv[32], dv[32], pk[16], dk[16];
            tmem_ld32(tmem + lane_off + c * 32, sv);
            tmem_ld32(tmem + lane_off + 128 + c * 32, dv);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              float pe[2], de[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int qi = c * 32 + e + u;
                float pr = fast_exp2(fmaf(__uint_as_float(sv[e + u]), p.scale_log2, nl[qi]));
                pr = (qi >= q_min) ? pr : 0.f;
                pe[u] = pr;
                de[u] = pr * (__uint_as_float(dv[e + u]) - dl[qi]);
              }
              pk[e / 2] = Pack2<T>::pack(pe[0], pe[1]);
              dk[e / 2] = Pack2<T>::pack(de[0], de[1]);
            }
            // P^T chunk c lands on columns of S^T chunks <= c, which are already in registers
            tmem_st16(tmem + lane_off + c * 16, pk);
            tmem_st16(tmem + lane_off + 128 + c * 16, dk);
          }
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s.p_ready);
        }
      }
      if (!ok) break;
      // read-out: dV as is, dK times the softmax scale
      if (!mbar_wait_warp(&s.acc_full, items & 1, ctx, kBwdCons)) break;
      tc_fence_after();
      const bool live = key < p.Skv;
      T* dv_row = static_cast<T*>(p.dv) + ((static_cast<long long>(b) * p.Hkv + hkv) * p.Skv + key) * kBwdD;
      T* dk_row = static_cast<T*>(p.dk) + ((static_cast<long long>(b) * p.Hkv + hkv) * p.Skv + key) * kBwdD;
#pragma unroll 1
      for (int c = 0; c < kBwdD / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem + lane_off + 256 + c * 32, r);
        tmem_wait_ld();
        if (live) bwd_store_row<T>(dv_row + c * 32, r, 1.0f);
        __syncwarp();
        tmem_ld32(tmem + lane_off + 384 + c * 32, r);
        tmem_wait_ld();
        if (live) bwd_store_row<T>(dk_row + c * 32, r, p.scale);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// dQ: one CTA per (batch, query head, 128-query tile); loops over the key tiles the queries see.
// TMEM: S [0,128) dP [128,256) dQ [256,384).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBwdThreads, 1) fa_bwd_dq_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  BwdSmem& s = *reinterpret_cast<BwdSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{&s.abort_flag, p.status};
  if (threadIdx.x == 0) {
    bwd_init(s, ctx, smem_raw);
    prefetch_tensormap(&p.tm_q);
    prefetch_tensormap(&p.tm_k);
    prefetch_tensormap(&p.tm_v);
    prefetch_tensormap(&p.tm_do);
  }
  if (warp == 5) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const bool run = (s.abort_flag == 0);
  const int past = p.Skv - p.Sq;

  auto item_of = [&](int g, int& b, int& hq, int& q0, int& nk) {
    // heaviest query tiles (highest index under a causal mask) first
    const int qb = p.nqb - 1 - (g % p.nqb);
    const int bh = g / p.nqb;
    b = bh / p.Hq;
    hq = bh - b * p.Hq;
    q0 = qb * 128;
    nk = p.causal ? min(p.nkb, (min(q0 + 127, p.Sq - 1) + past) / 128 + 1) : p.nkb;
  };

  if (warp == 4) {
    if (run && lane == 0) {
      uint32_t st = 0, phase = 1, f_phase = 1;
      bool ok = true;
      for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x) {
        int b, hq, q0, nk;
        item_of(g, b, hq, q0, nk);
        const int hkv = hq / p.group;
        if (!mbar_wait(&s.fixed_empty, f_phase, ctx, kBwdTma)) break;
        f_phase ^= 1;
        mbar_arrive_expect_tx(&s.fixed_full, 2 * kBwdTileBytes);
        bwd_load_tile(s.fixed[0], &p.tm_q, &s.fixed_full, q0, hq, b);
        bwd_load_tile(s.fixed[1], &p.tm_do, &s.fixed_full, q0, hq, b);
        for (int kt = 0; kt < nk; ++kt) {
          if (!mbar_wait(&s.ring_empty[st], phase, ctx, kBwdTma)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&s.ring_full[st], 2 * kBwdTileBytes);
          bwd_load_tile(s.ring[st][0], &p.tm_k, &s.ring_full[st], kt * 128, hkv, b);
          bwd_load_tile(s.ring[st][1], &p.tm_v, &s.ring_full[st], kt * 128, hkv, b);
          if (++st == kBwdStages) {
            st = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (run) {
      const bool leader = elect_one();
      uint32_t st = 0, phase = 0, f_phase = 0, s_cnt = 0, items = 0;
      bool ok = true;
      for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x, ++items) {
        int b, hq, q0, nk;
        item_of(g, b, hq, q0, nk);
        if (!mbar_wait_warp(&s.fixed_full, f_phase, ctx, kBwdMma)) break;
        f_phase ^= 1;
        for (int kt = 0; kt < nk; ++kt) {
          if (!mbar_wait_warp(&s.ring_full[st], phase, ctx, kBwdMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (leader) {
            bwd_mma_kk<T>(tmem + 0, s.fixed[0], s.ring[st][0]);    // S  = Q K^T
            bwd_mma_kk<T>(tmem + 128, s.fixed[1], s.ring[st][1]);  // dP = dO V^T
            umma_commit(&s.s_full);
          }
          __syncwarp();
          if (!mbar_wait_warp(&s.p_ready, s_cnt & 1, ctx, kBwdMma)) {
            ok = false;
            break;
          }
          ++s_cnt;
          if (kt == 0) {
            if (!mbar_wait_warp(&s.acc_empty, (items & 1) ^ 1, ctx, kBwdMma)) {
              ok = false;
              break;
            }
          }
          tc_fence_after();
          if (leader) {
            bwd_mma_ts<T>(tmem + 256, tmem + 128, s.ring[st][0], kt > 0 ? 1u : 0u);  // dQ += dS K
            umma_commit(&s.ring_empty[st]);
          }
          __syncwarp();
          if (++st == kBwdStages) {
            st = 0;
            phase ^= 1;
          }
        }
        if (ok && leader) {
          umma_commit(&s.acc_full);
          umma_commit(&s.fixed_empty);
        }
        __syncwarp();
      }
      __syncwarp();
      if (s.abort_flag && lane == 0) {
        umma_commit(&s.drain);
        mbar_wait(&s.drain, 0, ctx, kBwdDrain);
      }
    }
    __syncwarp();
  } else if (run) {
    // ---------------- consumers: one query per thread ----------------
    const int row_in_tile = warp * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    uint32_t s_cnt = 0, items = 0;
    bool ok = true;
    for (int g = blockIdx.x; ok && g < p.total_items; g += gridDim.x, ++items) {
      int b, hq, q0, nk;
      item_of(g, b, hq, q0, nk);
      const int q = q0 + row_in_tile;
      const bool live = q < p.Sq;
      const long long stat = (static_cast<long long>(b) * p.Hq + hq) * p.Sq + q;
      const float nlse2 = live ? -__ldg(p.lse + stat) * 1.4426950408889634f : -INFINITY;
      const float dlt = live ? __ldg(p.delta + stat) : 0.f;
      for (int kt = 0; kt < nk; ++kt) {
        if (!mbar_wait_warp(&s.s_full, s_cnt & 1, ctx, kBwdCons)) {
          ok = false;
          break;
        }
        ++s_cnt;
        tc_fence_after();
        // keys this query sees in the tile: key <= q + past (causal) and key < Skv
        int lim = p.Skv - 1 - kt * 128;
        if (p.causal) lim = min(lim, q + past - kt * 128);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t sv[32], dv[32], dk[16];
          tmem_ld32(tmem + lane_off + c * 32, sv);
          tmem_ld32(tmem + lane_off + 128 + c * 32, dv);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float de[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              float pr = fast_exp2(fmaf(__uint_as_float(sv[e + u]), p.scale_log2, nlse2));
              pr = (c * 32 + e + u <= lim) ? pr : 0.f;
              de[u] = pr * (__uint_as_float(dv[e + u]) - dlt);
            }
            dk[e / 2] = Pack2<T>::pack(de[0], de[1]);
          }
          tmem_st16(tmem + lane_off + 128 + c * 16, dk);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.p_ready);
      }
      if (!ok) break;
      if (!mbar_wait_warp(&s.acc_full, items & 1, ctx, kBwdCons)) break;
      tc_fence_after();
      T* dq_row = static_cast<T*>(p.dq) + stat * kBwdD;
#pragma unroll 1
      for (int c = 0; c < kBwdD / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem + lane_off + 256 + c * 32, r);
        tmem_wait_ld();
        if (live) bwd_store_row<T>(dq_row + c * 32, r, p.scale);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// delta = rowsum(O o dO): one warp per row, 8 bytes per lane (head_dim 128)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) fa_bwd_preprocess_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                                 float* __restrict__ delta, int B, int H, int S,
                                                                 long long o_sb, long long o_sh, long long o_ss,
                                                                 long long g_sb, long long g_sh, long long g_ss) {
  const long long row = blockIdx.x * 8ll + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<long long>(B) * H * S) return;
  const int sq = static_cast<int>(row % S);
  const long long bh = row / S;
  const int h = static_cast<int>(bh % H), b = static_cast<int>(bh / H);
  const uint2 a = *reinterpret_cast<const uint2*>(o + b * o_sb + h * o_sh + sq * o_ss + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(d_o + b * g_sb + h * g_sh + sq * g_ss + lane * 4);
  const T* ap = reinterpret_cast<const T*>(&a);
  const T* gp = reinterpret_cast<const T*>(&g);
  float acc = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) acc += static_cast<float>(ap[e]) * static_cast<float>(gp[e]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[row] = acc;
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static int bwd_check(const hb_fa_bwd_args* a, const char* who) {
  if (a == nullptr) return set_error(HB_ERR_BAD_ARG, "%s: args is NULL", who);
  if (a->B < 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Sq < 0 || a->Skv < 0)
    return set_error(HB_ERR_BAD_ARG, "%s: negative or zero extent", who);
  if (a->Hq % a->Hkv != 0) return set_error(HB_ERR_BAD_ARG, "%s: Hq is not a multiple of Hkv", who);
  if (a->dtype != HB_BF16 && a->dtype != HB_FP16) return set_error(HB_ERR_UNSUPPORTED, "%s: dtype %d not supported (bf16, fp16)", who, a->dtype);
  if (a->D != kBwdD) return set_error(HB_ERR_UNSUPPORTED, "%s: head_dim %d not supported (128)", who, a->D);
  if (a->causal && a->Skv < a->Sq) return set_error(HB_ERR_UNSUPPORTED, "%s: causal needs Skv >= Sq", who);
  return HB_OK;
}

static int bwd_fill(const hb_fa_bwd_args* a, BwdParams& p, const DeviceState* st) {
  memset(&p, 0, sizeof(p));
  const size_t es = 2;
  const CUtensorMapDataType dt = a->dtype == HB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const uint32_t box[4] = {64, 128, 1, 1};
  struct Desc {
    CUtensorMap* tm;
    const void* ptr;
    int S, H;
    int64_t sb, sh, ss;
  } d[4] = {{&p.tm_q, a->q, a->Sq, a->Hq, a->q_stride_b, a->q_stride_h, a->q_stride_s},
            {&p.tm_k, a->k, a->Skv, a->Hkv, a->k_stride_b, a->k_stride_h, a->k_stride_s},
            {&p.tm_v, a->v, a->Skv, a->Hkv, a->v_stride_b, a->v_stride_h, a->v_stride_s},
            {&p.tm_do, a->d_o, a->Sq, a->Hq, a->do_stride_b, a->do_stride_h, a->do_stride_s}};
  for (auto& t : d) {
    const uint64_t dims[4] = {(uint64_t)a->D, (uint64_t)t.S, (uint64_t)t.H, (uint64_t)a->B};
    const uint64_t str[3] = {(uint64_t)t.ss * es, (uint64_t)t.sh * es, (uint64_t)t.sb * es};
    const int rc = encode_tensor_map(t.tm, dt, 4, t.ptr, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB_OK) return rc;
  }
  p.lse = a->lse;
  p.delta = a->delta;
  p.dq = a->dq;
  p.dk = a->dk;
  p.dv = a->dv;
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
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / sqrtf((float)a->D);
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  return HB_OK;
}

template <typename K>
static int bwd_launch(K kernel, const BwdParams& p, int grid, const DeviceState* st, cudaStream_t stream, bool* configured) {
  if ((int)sizeof(BwdSmem) > st->smem_optin)
    return set_error(HB_ERR_UNSUPPORTED, "attention backward needs %d bytes of shared memory per CTA, the device offers %d",
                     (int)sizeof(BwdSmem), st->smem_optin);
  if (!configured[st->device & 63]) {
    HB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(BwdSmem)));
    configured[st->device & 63] = true;
  }
  kernel<<<grid, kBwdThreads, sizeof(BwdSmem), stream>>>(p);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

}  // namespace hb

extern "C" int hb_fa_bwd_preprocess(const hb_fa_bwd_args* a) {
  using namespace hb;
  clear_error();
  int rc = bwd_check(a, "hb_fa_bwd_preprocess");
  if (rc != HB_OK) return rc;
  if (a->B == 0 || a->Sq == 0) return HB_OK;
  if (a->o == nullptr || a->d_o == nullptr || a->delta == nullptr)
    return set_error(HB_ERR_BAD_ARG, "hb_fa_bwd_preprocess: o, d_o and delta must be non-NULL");
  if ((reinterpret_cast<uintptr_t>(a->o) & 7) || (reinterpret_cast<uintptr_t>(a->d_o) & 7) || (a->o_stride_s & 3) ||
      (a->o_stride_h & 3) || (a->o_stride_b & 3) || (a->do_stride_s & 3) || (a->do_stride_h & 3) || (a->do_stride_b & 3))
    return set_error(HB_ERR_ALIGN, "hb_fa_bwd_preprocess: o and d_o need 8-byte aligned rows");
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  const long long rows = (long long)a->B * a->Hq * a->Sq;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (a->dtype == HB_BF16)
    fa_bwd_preprocess_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(a->o), static_cast<const __nv_bfloat16*>(a->d_o), a->delta, a->B, a->Hq, a->Sq,
        a->o_stride_b, a->o_stride_h, a->o_stride_s, a->do_stride_b, a->do_stride_h, a->do_stride_s);
  else
    fa_bwd_preprocess_kernel<__half><<<grid, 256, 0, stream>>>(
        static_cast<const __half*>(a->o), static_cast<const __half*>(a->d_o), a->delta, a->B, a->Hq, a->Sq, a->o_stride_b,
        a->o_stride_h, a->o_stride_s, a->do_stride_b, a->do_stride_h, a->do_stride_s);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

extern "C" int hb_fa_bwd_dkdv(const hb_fa_bwd_args* a) {
  using namespace hb;
  clear_error();
  int rc = bwd_check(a, "hb_fa_bwd_dkdv");
  if (rc != HB_OK) return rc;
  if (a->B == 0 || a->Skv == 0) return HB_OK;
  if (a->dk == nullptr || a->dv == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_fa_bwd_dkdv: dk and dv must be non-NULL");
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (a->Sq == 0) {
    const size_t bytes = (size_t)a->B * a->Hkv * a->Skv * a->D * 2;
    HB_CUDA_CHECK(cudaMemsetAsync(a->dk, 0, bytes, stream));
    HB_CUDA_CHECK(cudaMemsetAsync(a->dv, 0, bytes, stream));
    return HB_OK;
  }
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->d_o == nullptr || a->lse == nullptr || a->delta == nullptr)
    return set_error(HB_ERR_BAD_ARG, "hb_fa_bwd_dkdv: q, k, v, d_o, lse and delta must be non-NULL");
  if ((reinterpret_cast<uintptr_t>(a->dk) & 15) || (reinterpret_cast<uintptr_t>(a->dv) & 15))
    return set_error(HB_ERR_ALIGN, "hb_fa_bwd_dkdv: dk and dv need 16-byte alignment");
  BwdParams p;
  rc = bwd_fill(a, p, st);
  if (rc != HB_OK) return rc;
  const long long total = (long long)a->B * a->Hkv * p.nkb;
  if (total > 0x7fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_fa_bwd_dkdv: problem too large");
  p.total_items = (int)total;
  const int grid = (int)std::min<long long>(total, st->sm_count);
  static bool cfg_bf16[64] = {}, cfg_f16[64] = {};
  if (a->dtype == HB_BF16) return bwd_launch(fa_bwd_dkdv_kernel<__nv_bfloat16>, p, grid, st, stream, cfg_bf16);
  return bwd_launch(fa_bwd_dkdv_kernel<__half>, p, grid, st, stream, cfg_f16);
}

extern "C" int hb_fa_bwd_dq(const hb_fa_bwd_args* a) {
  using namespace hb;
  clear_error();
  int rc = bwd_check(a, "hb_fa_bwd_dq");
  if (rc != HB_OK) return rc;
  if (a->B == 0 || a->Sq == 0) return HB_OK;
  if (a->dq == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_fa_bwd_dq: dq must be non-NULL");
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (a->Skv == 0) {
    HB_CUDA_CHECK(cudaMemsetAsync(a->dq, 0, (size_t)a->B * a->Hq * a->Sq * a->D * 2, stream));
    return HB_OK;
  }
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->d_o == nullptr || a->lse == nullptr || a->delta == nullptr)
    return set_error(HB_ERR_BAD_ARG, "hb_fa_bwd_dq: q, k, v, d_o, lse and delta must be non-NULL");
  if (reinterpret_cast<uintptr_t>(a->dq) & 15) return set_error(HB_ERR_ALIGN, "hb_fa_bwd_dq: dq needs 16-byte alignment");
  BwdParams p;
  rc = bwd_fill(a, p, st);
  if (rc != HB_OK) return rc;
  const long long total = (long long)a->B * a->Hq * p.nqb;
  if (total > 0x7fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_fa_bwd_dq: problem too large");
  p.total_items = (int)total;
  const int grid = (int)std::min<long long>(total, st->sm_count);
  static bool cfg_bf16[64] = {}, cfg_f16[64] = {};
  if (a->dtype == HB_BF16) return bwd_launch(fa_bwd_dq_kernel<__nv_bfloat16>, p, grid, st, stream, cfg_bf16);
  return bwd_launch(fa_bwd_dq_kernel<__half>, p, grid, st, stream, cfg_f16);
}
