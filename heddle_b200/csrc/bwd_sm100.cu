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
// One CTA (320 threads): warps 0-7 turn scores into P / dS (P stays in fp32 registers between the two
// phases; in the dK/dV kernel a row is shared by two threads, warp w takes columns [0,64) and warp w+4
// columns [64,128) of the same 32 TMEM lanes), warp 8 is the TMA producer, warp 9 issues the MMAs.
//
// Schedules (n = step, one 128 x 128 tile of scores; A = scores -> P, B = dP -> dS):
//   dK/dV  tensor pipe:  S(0) dP(0) | dV(n) S(n+1) | dK(n) dP(n+1) | ...
//          TMEM is full (S^T, dP^T, dV, dK = 512 columns), P^T overwrites S^T and dS^T overwrites
//          dP^T in place, so S(n+1) follows dV(n) and dP(n+1) follows dK(n) on the in-order tensor
//          pipe; phase B(n) and the MMAs dK(n), dP(n+1) hide behind the chain A(n) -> dV(n) -> S(n+1).
//   dQ     tensor pipe:  S(0) dP(0) S(1) | dP(n+1) dQ(n) S(n+2) | ...
//          S is double-buffered (S0, S1, dP, dQ = 512 columns) and dS(n) is written over S(n), so the
//          dP region is free as soon as phase B(n) has read it.  Here a thread owns a whole query row and
//          the two groups of four consumer warps take alternate steps (group g = score buffer g): phase
//          A(n+1) of one group runs beside phase B(n) of the other.
// head_dim 128 or 64, bf16 / fp16.
#include "host_common.h"
#include "ptx_sm100.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>

namespace hb {

constexpr int kBwdThreads = 320;    // dK/dV kernel
constexpr int kBwdDqThreads = 384;  // dQ kernel: a third (partly idle) warpgroup, so that registers can be re-split
__host__ __device__ constexpr uint32_t bwd_tile_bytes(int d) { return 128u * static_cast<uint32_t>(d) * 2u; }  // one 128-row tile of a 16-bit tensor
enum BwdRole : uint32_t { kBwdTma = 0x41, kBwdMma = 0x42, kBwdCons = 0x43, kBwdDrain = 0x44 };
// Share of the exponentials evaluated on the FMA pipe instead of the MUFU: 0 none, 1 a quarter, 2 half.
#ifndef HB_BWD_POLY
#define HB_BWD_POLY 0
#endif

// Measurement builds (-DHB_BWD_PROF): every warp of the dQ kernel sums the cycles it spends in up to
// eight sections of its loop; hb_debug_bwd_prof copies the sums out.
#ifdef HB_BWD_PROF
__device__ unsigned long long g_bwd_prof[148 * 10 * 8];
#define BWD_PROF_DECL                                     \
  unsigned long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; \
  long long prof_t = clock64();
#define BWD_PROF(i)                                              \
  {                                                              \
    const long long t_ = clock64();                              \
    prof_acc[i] += static_cast<unsigned long long>(t_ - prof_t); \
    prof_t = t_;                                                 \
  }
#define BWD_PROF_FLUSH                                                                                    \
  if (lane == 0 && blockIdx.x < 148)                                                                      \
    for (int i_ = 0; i_ < 8; ++i_) g_bwd_prof[(blockIdx.x * 10 + warp) * 8 + i_] = prof_acc[i_];
#else
#define BWD_PROF_DECL
#define BWD_PROF(i)
#define BWD_PROF_FLUSH
#endif

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
  int npairs;       // pairs of tiles per head: dkdv ceil(nkb / 2), dq ceil(nqb / 2)
  int total_items;  // pairs: dkdv B * Hkv * npairs;  dq B * Hq * npairs
  float scale_log2, scale;
};

// rings: A feeds the score product and the last product of the step, B the dP product (and dV)
template <int D, int kStagesA, int kStagesB, bool kStage>
struct BwdSmem {
  static constexpr uint32_t kBwdTileBytes = bwd_tile_bytes(D);
  static constexpr int kSA = kStagesA, kSB = kStagesB;
  alignas(1024) uint8_t fixed[2][kBwdTileBytes];        // dkdv: K, V of the item;  dq: Q, dO of the item
  alignas(1024) uint8_t ring_a[kStagesA][kBwdTileBytes];  // dkdv: Q tiles;  dq: K tiles
  alignas(1024) uint8_t ring_b[kStagesB][kBwdTileBytes];  // dkdv: dO tiles; dq: V tiles
  uint64_t fixed_full, fixed_empty;
  uint64_t a_full[kStagesA], a_empty[kStagesA];
  uint64_t b_full[kStagesB], b_empty[kStagesB];
  uint64_t s_full[2];  // MMA -> consumers: scores are in TMEM (dkdv uses [0] only)
  uint64_t dp_full;    // MMA -> consumers: dP is in TMEM
  uint64_t p_ready[2]; // consumers -> MMA: first / second half of every warp's P columns written (dkdv only)
  uint64_t ds_ready;   // consumers -> MMA: dS written, dP read
  // warps 0-3 -> warps 4-7: columns [32,64) of a tile have been read (the upper warps' 16-bit results
  // land there).  One completion per step and barrier (dkdv: [0] scores, [1] dP; dq: [score buffer]),
  // so the lower warps can never be two phases ahead of a waiting upper warp.
  uint64_t half_read[2];
  uint64_t acc_full;   // MMA -> consumers: the item's accumulators are complete
  uint64_t acc_empty;  // consumers -> MMA: accumulators read out
  uint64_t drain;
  uint32_t tmem_base, abort_flag;
  // dkdv: per consumer warp, double-buffered {-LSE*log2e, delta} of a query tile
  alignas(16) float stage[kStage ? 8 : 1][2][2][kStage ? 64 : 4];
};
template <int D>
using BwdSmemKv = BwdSmem<D, 2, 2, true>;
template <int D>
using BwdSmemQ = BwdSmem<D, 3, 2, false>;

// Shared-memory descriptor pieces (same conventions as the forward kernel)
constexpr uint32_t kBwdDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t kBwdLboK = (16u >> 4) << 16;     // K-major operand
constexpr uint32_t kBwdSub16 = (128u * 128u) >> 4;  // one 128-byte-wide, 128-row sub-tile in 16-byte units
constexpr uint32_t kBwdLboMn = kBwdSub16 << 16;     // MN-major operand: next 64 head_dim columns
__device__ __forceinline__ uint64_t bwd_desc(uint32_t lo) { return (static_cast<uint64_t>(kBwdDescHi) << 32) | lo; }

// D[128 x 128] = A[128 x head_dim] . B[128 x head_dim]^T, both operands K-major tiles in smem
template <typename T, int D>
__device__ __forceinline__ void bwd_mma_kk(uint32_t d_tmem, const void* a_tile, const void* b_tile) {
  constexpr uint32_t idesc = make_idesc(Pack2<T>::kFormat, 128, 128, 0, 0);
  const uint32_t a_lo = (smem_u32(a_tile) >> 4) | kBwdLboK, b_lo = (smem_u32(b_tile) >> 4) | kBwdLboK;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const uint32_t off = static_cast<uint32_t>(kk >> 2) * kBwdSub16 + static_cast<uint32_t>(kk & 3) * 2u;
    umma_ss_f16(d_tmem, bwd_desc(a_lo + off), bwd_desc(b_lo + off), idesc, kk > 0 ? 1u : 0u);
  }
}
// D[128 x head_dim] (+)= A[128 x 128] (packed 16-bit, in TMEM) . B[128(K) x head_dim] (a row tile in smem, MN-major)
template <typename T, int D>
__device__ __forceinline__ void bwd_mma_ts(uint32_t d_tmem, uint32_t a_tmem, const void* b_tile, uint32_t accumulate) {
  constexpr uint32_t idesc = make_idesc(Pack2<T>::kFormat, 128, D, 0, 1);
  const uint32_t b_lo = (smem_u32(b_tile) >> 4) | kBwdLboMn;
#pragma unroll
  for (int kk = 0; kk < 128 / 16; ++kk) {
    umma_ts_f16(d_tmem, a_tmem + static_cast<uint32_t>(kk * 8), bwd_desc(b_lo + static_cast<uint32_t>(kk) * 128u), idesc,
                kk > 0 ? 1u : accumulate);
  }
}

// The same product restricted to the K-steps (16 rows of A's columns / B's rows each) named in kMask
template <typename T, int D, uint32_t kMask>
__device__ __forceinline__ void bwd_mma_ts_part(uint32_t d_tmem, uint32_t a_tmem, const void* b_tile, uint32_t accumulate) {
  constexpr uint32_t idesc = make_idesc(Pack2<T>::kFormat, 128, D, 0, 1);
  const uint32_t b_lo = (smem_u32(b_tile) >> 4) | kBwdLboMn;
  uint32_t acc = accumulate;
#pragma unroll
  for (int kk = 0; kk < 128 / 16; ++kk) {
    if ((kMask >> kk) & 1u) {
      umma_ts_f16(d_tmem, a_tmem + static_cast<uint32_t>(kk * 8), bwd_desc(b_lo + static_cast<uint32_t>(kk) * 128u), idesc, acc);
      acc = 1u;
    }
  }
}

template <int D>
__device__ __forceinline__ void bwd_load_tile(void* dst, const CUtensorMap* tm, uint64_t* bar, int row0, int h, int b) {
  mbar_arrive_expect_tx(bar, bwd_tile_bytes(D));
#pragma unroll
  for (int hh = 0; hh < D / 64; ++hh)
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

// Four probabilities 2^(s * scale_log2 + nl) of one thread's row; with HB_BWD_POLY part of them on the FMA pipe.
__device__ __forceinline__ void bwd_exp4(const uint32_t* sv, int e, uint64_t sc2, float4 l4, float* out) {
#ifdef HB_BWD_KO_EXP  // measurement builds only: no exponentials (wrong results)
  out[0] = __uint_as_float(sv[0]) + l4.x;
  out[1] = __uint_as_float(sv[1]) + l4.y;
  out[2] = __uint_as_float(sv[2]) + l4.z;
  out[3] = __uint_as_float(sv[3]) + l4.w;
  return;
#endif
  const uint64_t x0 = fma_f32x2(pack_f32x2(__uint_as_float(sv[0]), __uint_as_float(sv[1])), sc2, pack_f32x2(l4.x, l4.y));
  const uint64_t x1 = fma_f32x2(pack_f32x2(__uint_as_float(sv[2]), __uint_as_float(sv[3])), sc2, pack_f32x2(l4.z, l4.w));
  float a0, a1, b0, b1;
  unpack_f32x2(x0, a0, a1);
  out[0] = fast_exp2(a0);
  out[1] = fast_exp2(a1);
  const bool poly = (HB_BWD_POLY == 2) || (HB_BWD_POLY == 1 && (e & 4) != 0);
  if (poly) {
    exp2_poly_f32x2(x1, b0, b1);
  } else {
    unpack_f32x2(x1, b0, b1);
    b0 = fast_exp2(b0);
    b1 = fast_exp2(b1);
  }
  out[2] = b0;
  out[3] = b1;
}

template <typename Smem>
__device__ __forceinline__ void bwd_init(Smem& s, const AbortCtx& ctx, const void* smem_raw, uint32_t ds_arrivals) {
  s.abort_flag = 0;
  mbar_init(&s.fixed_full, 1);
  mbar_init(&s.fixed_empty, 1);
  for (int i = 0; i < Smem::kSA; ++i) {
    mbar_init(&s.a_full[i], 1);
    mbar_init(&s.a_empty[i], 1);
  }
  for (int i = 0; i < Smem::kSB; ++i) {
    mbar_init(&s.b_full[i], 1);
    mbar_init(&s.b_empty[i], 1);
  }
  mbar_init(&s.s_full[0], 1);
  mbar_init(&s.s_full[1], 1);
  mbar_init(&s.dp_full, 1);
  mbar_init(&s.p_ready[0], 8);
  mbar_init(&s.p_ready[1], 8);
  mbar_init(&s.ds_ready, ds_arrivals);
  mbar_init(&s.half_read[0], 4);
  mbar_init(&s.half_read[1], 4);
  mbar_init(&s.acc_full, 1);
  mbar_init(&s.acc_empty, 8);
  mbar_init(&s.drain, 1);
  fence_mbar_init();
  if ((smem_u32(smem_raw) & 1023u) != 0u) raise_abort(ctx, kStatusSmemMisaligned);
}

// ------------------------------------------------------------------------------------------
// dK, dV: one CTA per (batch, kv head, 128-key tile); loops over the group's query heads and the
// query tiles that can see the key tile.  TMEM: S^T [0,128) dP^T [128,256) dV [256,384) dK [384,512).
// ------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads, 1) fa_bwd_dkdv_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using Smem = BwdSmemKv<D>;
  constexpr uint32_t kBwdTileBytes = bwd_tile_bytes(D);
  Smem& s = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{&s.abort_flag, p.status};
  if (threadIdx.x == 0) {
    bwd_init(s, ctx, smem_raw, 8);
    prefetch_tensormap(&p.tm_q);
    prefetch_tensormap(&p.tm_k);
    prefetch_tensormap(&p.tm_v);
    prefetch_tensormap(&p.tm_do);
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
  const int past = p.Skv - p.Sq;

  // Work list: entry u >> 1 is a pair of key tiles (pair, nkb-1-pair) of one (batch, kv head), u & 1 selects
  // the tile.  Under a causal mask the two tiles of a pair together see nqb + 1 query tiles whatever the pair, so
  // the static round-robin over pairs keeps the persistent CTAs balanced.
  auto item_of = [&](int u, int& b, int& hkv, int& k0, int& qt0) -> bool {
    const int g = u >> 1;
    const int pair = g % p.npairs;
    const int bh = g / p.npairs;
    const int kb = (u & 1) ? p.nkb - 1 - pair : pair;
    if ((u & 1) && kb == pair) return false;  // middle tile of an odd count
    b = bh / p.Hkv;
    hkv = bh - b * p.Hkv;
    k0 = kb * 128;
    qt0 = p.causal ? max(0, (k0 - past) / 128) : 0;
    return true;
  };

  if (warp == 8) {
    if (run && lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t cnt = 0, f_phase = 1;  // cnt: steps loaded so far (stage = cnt & 1 in both rings)
      bool ok = true;
      for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1)) {
        int b, hkv, k0, qt0;
        if (!item_of(u, b, hkv, k0, qt0)) continue;
        if (!mbar_wait(&s.fixed_empty, f_phase, ctx, kBwdTma)) break;
        f_phase ^= 1;
        mbar_arrive_expect_tx(&s.fixed_full, 2 * kBwdTileBytes);
#pragma unroll
        for (int hh = 0; hh < D / 64; ++hh) {
          tma_load_4d(s.fixed[0] + hh * (128 * 128), &p.tm_k, &s.fixed_full, hh * 64, k0, hkv, b);
          tma_load_4d(s.fixed[1] + hh * (128 * 128), &p.tm_v, &s.fixed_full, hh * 64, k0, hkv, b);
        }
        for (int hg = 0; ok && hg < p.group; ++hg) {
          const int hq = hkv * p.group + hg;
          for (int qt = qt0; qt < p.nqb; ++qt, ++cnt) {
            const uint32_t st = cnt & 1u, ph = ((cnt >> 1) & 1u) ^ 1u;
            if (!mbar_wait(&s.a_empty[st], ph, ctx, kBwdTma)) {
              ok = false;
              break;
            }
            bwd_load_tile<D>(s.ring_a[st], &p.tm_q, &s.a_full[st], qt * 128, hq, b);
            if (!mbar_wait(&s.b_empty[st], ph, ctx, kBwdTma)) {
              ok = false;
              break;
            }
            bwd_load_tile<D>(s.ring_b[st], &p.tm_do, &s.b_full[st], qt * 128, hq, b);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    if (run) {
      // ---------------- MMA issuer (warp-uniform, elected lane issues) ----------------
      const bool leader = elect_one();
      uint32_t cnt = 0, f_phase = 0, items = 0;  // cnt: global step counter
      bool ok = true;
      BWD_PROF_DECL
      auto full_a = [&](uint32_t c) { return mbar_wait_warp(&s.a_full[c & 1u], (c >> 1) & 1u, ctx, kBwdMma); };
      auto full_b = [&](uint32_t c) { return mbar_wait_warp(&s.b_full[c & 1u], (c >> 1) & 1u, ctx, kBwdMma); };
      for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1), ++items) {
        int b, hkv, k0, qt0;
        if (!item_of(u, b, hkv, k0, qt0)) {
          --items;  // not an item: keep the count of real items
          continue;
        }
        const int n_steps = p.group * (p.nqb - qt0);
        if (!mbar_wait_warp(&s.fixed_full, f_phase, ctx, kBwdMma)) break;
        f_phase ^= 1;
        // prologue: S(0), dP(0)
        if (!full_a(cnt)) break;
        tc_fence_after();
        if (leader) {
          bwd_mma_kk<T, D>(tmem + 0, s.fixed[0], s.ring_a[cnt & 1u]);  // S^T = K Q^T
          umma_commit(&s.s_full[0]);
        }
        __syncwarp();
        if (!full_b(cnt)) break;
        tc_fence_after();
        if (leader) {
          bwd_mma_kk<T, D>(tmem + 128, s.fixed[1], s.ring_b[cnt & 1u]);  // dP^T = V dO^T
          umma_commit(&s.dp_full);
          if (n_steps == 1) umma_commit(&s.fixed_empty);  // K and V are not read again
        }
        __syncwarp();
        BWD_PROF(0)
        for (int n = 0; n < n_steps; ++n, ++cnt) {
          const uint32_t st = cnt & 1u, nx = (cnt + 1) & 1u, par = cnt & 1u;
          const bool more = n + 1 < n_steps;
          // the first accumulation of the item overwrites dV, dK: the previous item's read-out must be over
          if (n == 0 && !mbar_wait_warp(&s.acc_empty, (items & 1u) ^ 1u, ctx, kBwdMma)) {
            ok = false;
            break;
          }
          // dV += P^T dO in two parts: queries [0,32) and [64,96) of the tile (the first half of every
          // consumer warp's columns) while the consumers are still working on the other half
          if (!mbar_wait_warp(&s.p_ready[0], par, ctx, kBwdMma)) {
            ok = false;
            break;
          }
          BWD_PROF(1)
          tc_fence_after();
          if (leader) bwd_mma_ts_part<T, D, 0x33u>(tmem + 256, tmem + 0, s.ring_b[st], n > 0 ? 1u : 0u);
          __syncwarp();
          // the Q tile of the next step was requested when dK of the previous step completed
          if (more && !full_a(cnt + 1)) {
            ok = false;
            break;
          }
          BWD_PROF(3)
          if (!mbar_wait_warp(&s.p_ready[1], par, ctx, kBwdMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (leader) {
            bwd_mma_ts_part<T, D, 0xCCu>(tmem + 256, tmem + 0, s.ring_b[st], 1u);
            umma_commit(&s.b_empty[st]);
          }
          __syncwarp();
          BWD_PROF(2)
          if (more) {
            if (leader) {
              bwd_mma_kk<T, D>(tmem + 0, s.fixed[0], s.ring_a[nx]);  // S^T of the next step, over P^T
              umma_commit(&s.s_full[0]);
            }
            __syncwarp();
            BWD_PROF(4)
            if (!full_b(cnt + 1)) {
              ok = false;
              break;
            }
          }
          if (!mbar_wait_warp(&s.ds_ready, par, ctx, kBwdMma)) {
            ok = false;
            break;
          }
          BWD_PROF(5)
          tc_fence_after();
          if (leader) {
            bwd_mma_ts<T, D>(tmem + 384, tmem + 128, s.ring_a[st], n > 0 ? 1u : 0u);  // dK += dS^T Q
            umma_commit(&s.a_empty[st]);
            if (more) {
              bwd_mma_kk<T, D>(tmem + 128, s.fixed[1], s.ring_b[nx]);  // dP^T of the next step, over dS^T
              umma_commit(&s.dp_full);
              // the item's last products with K and V are out: the next item's tiles load behind the last step
              if (n + 2 == n_steps) umma_commit(&s.fixed_empty);
            }
          }
          __syncwarp();
          BWD_PROF(6)
        }
        if (ok && leader) umma_commit(&s.acc_full);
        __syncwarp();
      }
      __syncwarp();
      BWD_PROF_FLUSH
      if (s.abort_flag && lane == 0) {
        umma_commit(&s.drain);
        mbar_wait(&s.drain, 0, ctx, kBwdDrain);
      }
    }
    __syncwarp();
  } else if (run) {
    // ---------------- consumers: one key per pair of threads ----------------
    const int slab = warp & 3, half = warp >> 2;
    const int key_in_tile = slab * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(slab * 32) << 16;
    const uint32_t col_in = static_cast<uint32_t>(half * 64);   // fp32 columns this thread reads
    const uint32_t col_out = static_cast<uint32_t>(half * 32);  // 16-bit columns it writes
    const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), one2 = pack_f32x2(1.0f, 1.0f);
    uint32_t cnt = 0, items = 0;
    bool ok = true;
    for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1), ++items) {
      int b, hkv, k0, qt0;
      if (!item_of(u, b, hkv, k0, qt0)) {
        --items;  // not an item: keep the count of real items
        continue;
      }
      const int key = k0 + key_in_tile;
      for (int hg = 0; ok && hg < p.group; ++hg) {
        const int hq = hkv * p.group + hg;
        const float* lse_row = p.lse + (static_cast<long long>(b) * p.Hq + hq) * p.Sq;
        const float* dl_row = p.delta + (static_cast<long long>(b) * p.Hq + hq) * p.Sq;
        for (int qt = qt0; qt < p.nqb; ++qt, ++cnt) {
          // this warp's copy of the per-query terms of its 64 queries; queries past Sq get -inf (P = 0)
          float2* nl2 = reinterpret_cast<float2*>(s.stage[warp][cnt & 1u][0]);
          float2* dl2 = reinterpret_cast<float2*>(s.stage[warp][cnt & 1u][1]);
          {
            const int q = qt * 128 + half * 64 + lane * 2;
            float2 nv, dv;
            nv.x = (q < p.Sq) ? -__ldg(lse_row + q) * 1.4426950408889634f : -INFINITY;
            nv.y = (q + 1 < p.Sq) ? -__ldg(lse_row + q + 1) * 1.4426950408889634f : -INFINITY;
            dv.x = (q < p.Sq) ? __ldg(dl_row + q) : 0.f;
            dv.y = (q + 1 < p.Sq) ? __ldg(dl_row + q + 1) : 0.f;
            nl2[lane] = nv;
            dl2[lane] = dv;
          }
          __syncwarp();
          const float4* nl4 = reinterpret_cast<const float4*>(nl2);
          const float4* dl4 = reinterpret_cast<const float4*>(dl2);
          // ---- phase A: scores -> P (kept in registers, 16-bit copy over S^T for dV += P^T dO) ----
          if (!mbar_wait_warp(&s.s_full[0], cnt & 1u, ctx, kBwdCons)) {
            ok = false;
            break;
          }
          tc_fence_after();
          float pr[64];
          {
            uint32_t sv[64], pk[32];
            tmem_ld32(tmem + lane_off + col_in, sv);
            tmem_ld32(tmem + lane_off + col_in + 32, sv + 32);
            tmem_wait_ld();
            if (half == 0) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&s.half_read[0]);
            }
            // causal: key visible to query q iff key <= q + past; only tiles on the diagonal need the test
            const bool need_mask = p.causal && (qt * 128 < k0 + 127 - past);
            const int q_min = key - past - qt * 128 - half * 64;  // first visible query, relative to this thread's columns
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
#pragma unroll
              for (int e = h2 * 32; e < h2 * 32 + 32; e += 4) {
                bwd_exp4(&sv[e], e, sc2, nl4[e >> 2], &pr[e]);
                if (need_mask) {
#pragma unroll
                  for (int u = 0; u < 4; ++u) pr[e + u] = (e + u >= q_min) ? pr[e + u] : 0.f;
                }
                pk[e / 2] = Pack2<T>::pack(pr[e], pr[e + 1]);
                pk[e / 2 + 1] = Pack2<T>::pack(pr[e + 2], pr[e + 3]);
              }
              // the lower warps overwrite columns they have read themselves; the upper warps' P^T lands on
              // columns [32,64), which the lower warps have read once half_read completes
              if (half == 1 && h2 == 0) {
                if (!mbar_wait_warp(&s.half_read[0], cnt & 1u, ctx, kBwdCons)) {
                  ok = false;
                  break;
                }
                tc_fence_after();
              }
              // 32 queries at a time, so that the matching part of dV += P^T dO starts behind the other 32
              tmem_st16(tmem + lane_off + col_out + h2 * 16, pk + h2 * 16);
              tmem_wait_st();
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&s.p_ready[h2]);
            }
            if (!ok) break;
          }
          // ---- phase B: dP -> dS = P o (dP - delta), 16-bit over dP^T for dK += dS^T Q ----
          if (!mbar_wait_warp(&s.dp_full, cnt & 1u, ctx, kBwdCons)) {
            ok = false;
            break;
          }
          tc_fence_after();
          {
            uint32_t dv[64], dk[32];
            tmem_ld32(tmem + lane_off + 128 + col_in, dv);
            tmem_ld32(tmem + lane_off + 128 + col_in + 32, dv + 32);
            tmem_wait_ld();
            if (half == 0) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&s.half_read[1]);
            }
#pragma unroll
            for (int e = 0; e < 64; e += 4) {
              const float4 d4 = dl4[e >> 2];
              // two elements per instruction: (dP - delta) as dP * 1 + (-delta), then P * that
              const uint64_t t01 = fma_f32x2(pack_f32x2(__uint_as_float(dv[e]), __uint_as_float(dv[e + 1])), one2, pack_f32x2(-d4.x, -d4.y));
              const uint64_t t23 = fma_f32x2(pack_f32x2(__uint_as_float(dv[e + 2]), __uint_as_float(dv[e + 3])), one2, pack_f32x2(-d4.z, -d4.w));
              float x0, x1, x2, x3;
              unpack_f32x2(mul_f32x2(pack_f32x2(pr[e], pr[e + 1]), t01), x0, x1);
              unpack_f32x2(mul_f32x2(pack_f32x2(pr[e + 2], pr[e + 3]), t23), x2, x3);
              dk[e / 2] = Pack2<T>::pack(x0, x1);
              dk[e / 2 + 1] = Pack2<T>::pack(x2, x3);
            }
            if (half == 1) {
              if (!mbar_wait_warp(&s.half_read[1], cnt & 1u, ctx, kBwdCons)) {
                ok = false;
                break;
              }
              tc_fence_after();
            }
            tmem_st32(tmem + lane_off + 128 + col_out, dk);
          }
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s.ds_ready);
        }
      }
      if (!ok) break;
      // read-out: dV as is, dK times the softmax scale; each thread stores its half of the row's head_dim columns
      if (!mbar_wait_warp(&s.acc_full, items & 1u, ctx, kBwdCons)) break;
      tc_fence_after();
      const bool live = key < p.Skv;
      const uint32_t col_acc = static_cast<uint32_t>(half * (D / 2));
      T* dv_row = static_cast<T*>(p.dv) + ((static_cast<long long>(b) * p.Hkv + hkv) * p.Skv + key) * D + col_acc;
      T* dk_row = static_cast<T*>(p.dk) + ((static_cast<long long>(b) * p.Hkv + hkv) * p.Skv + key) * D + col_acc;
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem + lane_off + 256 + col_acc + c * 32, r);
        tmem_wait_ld();
        if (live) bwd_store_row<T>(dv_row + c * 32, r, 1.0f);
        __syncwarp();
        tmem_ld32(tmem + lane_off + 384 + col_acc + c * 32, r);
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
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// dQ: one CTA per (batch, query head, 128-query tile); loops over the key tiles the queries see.
// TMEM: S buffers [0,128) [128,256), dP [256,384), dQ [384,512).
// ------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kBwdDqThreads, 1) fa_bwd_dq_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using Smem = BwdSmemQ<D>;
  constexpr uint32_t kBwdTileBytes = bwd_tile_bytes(D);
  Smem& s = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{&s.abort_flag, p.status};
  if (threadIdx.x == 0) {
    bwd_init(s, ctx, smem_raw, 4);
    prefetch_tensormap(&p.tm_q);
    prefetch_tensormap(&p.tm_k);
    prefetch_tensormap(&p.tm_v);
    prefetch_tensormap(&p.tm_do);
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
  const int past = p.Skv - p.Sq;

  // Work list: entry u >> 1 is a pair of query tiles (nqb-1-pair, pair) of one (batch, head), u & 1 selects
  // the tile; under a causal mask the two together see about the same number of key tiles for every pair.
  auto item_of = [&](int u, int& b, int& hq, int& q0, int& nk) -> bool {
    const int g = u >> 1;
    const int pair = g % p.npairs;
    const int bh = g / p.npairs;
    const int qb = (u & 1) ? pair : p.nqb - 1 - pair;
    if ((u & 1) && qb == p.nqb - 1 - pair) return false;  // middle tile of an odd count
    b = bh / p.Hq;
    hq = bh - b * p.Hq;
    q0 = qb * 128;
    nk = p.causal ? min(p.nkb, (min(q0 + 127, p.Sq - 1) + past) / 128 + 1) : p.nkb;
    return true;
  };

  // Registers: the consumers keep a whole row of P (128 fp32) between the phases; warps 8-11 give theirs up
  // (setmaxnreg is per warpgroup: warps 10 and 11 exist only for that).  Per scheduler 2 x 216 + 72 <= 512.
  if (warp >= 8) reg_dec<72>();
  if (warp == 8) {
    if (run && lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t cnt = 0, f_phase = 1;
      bool ok = true;
      for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1)) {
        int b, hq, q0, nk;
        if (!item_of(u, b, hq, q0, nk)) continue;
        const int hkv = hq / p.group;
        if (!mbar_wait(&s.fixed_empty, f_phase, ctx, kBwdTma)) break;
        f_phase ^= 1;
        mbar_arrive_expect_tx(&s.fixed_full, 2 * kBwdTileBytes);
#pragma unroll
        for (int hh = 0; hh < D / 64; ++hh) {
          tma_load_4d(s.fixed[0] + hh * (128 * 128), &p.tm_q, &s.fixed_full, hh * 64, q0, hq, b);
          tma_load_4d(s.fixed[1] + hh * (128 * 128), &p.tm_do, &s.fixed_full, hh * 64, q0, hq, b);
        }
        for (int kt = 0; kt < nk; ++kt, ++cnt) {
          const uint32_t sa = cnt % 3u, pa = ((cnt / 3u) & 1u) ^ 1u;
          const uint32_t sb = cnt & 1u, pb = ((cnt >> 1) & 1u) ^ 1u;
          if (!mbar_wait(&s.a_empty[sa], pa, ctx, kBwdTma)) {
            ok = false;
            break;
          }
          bwd_load_tile<D>(s.ring_a[sa], &p.tm_k, &s.a_full[sa], kt * 128, hkv, b);
          if (!mbar_wait(&s.b_empty[sb], pb, ctx, kBwdTma)) {
            ok = false;
            break;
          }
          bwd_load_tile<D>(s.ring_b[sb], &p.tm_v, &s.b_full[sb], kt * 128, hkv, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    if (run) {
      // ---------------- MMA issuer ----------------
      const bool leader = elect_one();
      uint32_t cnt = 0, f_phase = 0, items = 0;  // cnt: global step counter
      bool ok = true;
      BWD_PROF_DECL
      // S(c) = Q K(c)^T into score buffer c & 1
      auto issue_s = [&](uint32_t c) -> bool {
        if (!mbar_wait_warp(&s.a_full[c % 3u], (c / 3u) & 1u, ctx, kBwdMma)) return false;
        tc_fence_after();
        if (leader) {
          bwd_mma_kk<T, D>(tmem + (c & 1u) * 128u, s.fixed[0], s.ring_a[c % 3u]);
          umma_commit(&s.s_full[c & 1u]);
        }
        __syncwarp();
        return true;
      };
      // dP(c) = dO V(c)^T; V(c) is not needed again
      auto issue_dp = [&](uint32_t c) -> bool {
        if (!mbar_wait_warp(&s.b_full[c & 1u], (c >> 1) & 1u, ctx, kBwdMma)) return false;
        tc_fence_after();
        if (leader) {
          bwd_mma_kk<T, D>(tmem + 256, s.fixed[1], s.ring_b[c & 1u]);
          umma_commit(&s.dp_full);
          umma_commit(&s.b_empty[c & 1u]);
        }
        __syncwarp();
        return true;
      };
      for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1), ++items) {
        int b, hq, q0, nk;
        if (!item_of(u, b, hq, q0, nk)) {
          --items;  // not an item: keep the count of real items
          continue;
        }
        if (!mbar_wait_warp(&s.fixed_full, f_phase, ctx, kBwdMma)) break;
        f_phase ^= 1;
        if (!issue_s(cnt) || !issue_dp(cnt)) break;
        if (nk > 1 && !issue_s(cnt + 1)) break;
        if (nk == 1 && leader) umma_commit(&s.fixed_empty);  // Q and dO are not read again
        __syncwarp();
        BWD_PROF(0)
        for (int n = 0; n < nk; ++n, ++cnt) {
          // the V tile of the next dP was requested a step ago: waited for before the consumers' result,
          // so that dP and dQ go out back to back
          if ((n + 1 < nk && !mbar_wait_warp(&s.b_full[(cnt + 1) & 1u], ((cnt + 1) >> 1) & 1u, ctx, kBwdMma)) ||
              (n == 0 && !mbar_wait_warp(&s.acc_empty, (items & 1u) ^ 1u, ctx, kBwdMma))) {
            ok = false;
            break;
          }
          BWD_PROF(1)
          if (!mbar_wait_warp(&s.ds_ready, cnt & 1u, ctx, kBwdMma)) {
            ok = false;
            break;
          }
          BWD_PROF(2)
          tc_fence_after();
          if (leader) {
            // dP of the step has been read and dS written over S: the next dP goes first, phase B of the
            // next step waits for it
            if (n + 1 < nk) {
              bwd_mma_kk<T, D>(tmem + 256, s.fixed[1], s.ring_b[(cnt + 1) & 1u]);
              umma_commit(&s.dp_full);
              umma_commit(&s.b_empty[(cnt + 1) & 1u]);
              // the item's last products with Q and dO are out: the next item's tiles load behind the last step
              if (n + 2 == nk) umma_commit(&s.fixed_empty);
            }
            bwd_mma_ts<T, D>(tmem + 384, tmem + (cnt & 1u) * 128u, s.ring_a[cnt % 3u], n > 0 ? 1u : 0u);  // dQ += dS K
            umma_commit(&s.a_empty[cnt % 3u]);
          }
          __syncwarp();
          BWD_PROF(3)
          // the K tile two steps ahead was requested when dQ of the previous step completed; its scores
          // are not needed before the next step's phase A
          if (n + 2 < nk && !issue_s(cnt + 2)) {
            ok = false;
            break;
          }
          BWD_PROF(4)
        }
        if (ok && leader) umma_commit(&s.acc_full);
        __syncwarp();
      }
      __syncwarp();
      BWD_PROF_FLUSH
      if (s.abort_flag && lane == 0) {
        umma_commit(&s.drain);
        mbar_wait(&s.drain, 0, ctx, kBwdDrain);
      }
    }
    __syncwarp();
  } else if (warp < 8) {
   reg_inc<216>();
   if (run) {
    // ---------------- consumers: one query per thread, the two groups of four warps take alternate steps ----------------
    // Group g owns the steps whose global index is g modulo 2, i.e. score buffer g.  While one group turns dP of
    // step n into dS (the link of the chain dS(n) -> dP(n+1) -> dS(n+1)), the other is already past the
    // exponentials of step n+1 and only waits for its dP.
    const int slab = warp & 3, grp = warp >> 2;
    const int row_in_tile = slab * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(slab * 32) << 16;
    const uint32_t sbuf = tmem + lane_off + static_cast<uint32_t>(grp) * 128u;
    const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2);
    uint32_t cnt = 0, items = 0;
    bool ok = true;
    BWD_PROF_DECL
    for (int u = 2 * blockIdx.x; ok && u < 2 * p.total_items; u += ((u & 1) ? 2 * (int)gridDim.x - 1 : 1), ++items) {
      int b, hq, q0, nk;
      if (!item_of(u, b, hq, q0, nk)) {
        --items;  // not an item: keep the count of real items
        continue;
      }
      const int q = q0 + row_in_tile;
      const bool live = q < p.Sq;
      const long long stat = (static_cast<long long>(b) * p.Hq + hq) * p.Sq + q;
      const float nlse2 = live ? -__ldg(p.lse + stat) * 1.4426950408889634f : -INFINITY;
      const float dlt = live ? __ldg(p.delta + stat) : 0.f;
      const float4 l4 = make_float4(nlse2, nlse2, nlse2, nlse2);
      const uint64_t ndl2 = pack_f32x2(-dlt, -dlt);
      for (int kt = 0; kt < nk; ++kt, ++cnt) {
        if ((cnt & 1u) != static_cast<uint32_t>(grp)) continue;
        // ---- phase A: scores -> P in registers ----
        if (!mbar_wait_warp(&s.s_full[grp], (cnt >> 1) & 1u, ctx, kBwdCons)) {
          ok = false;
          break;
        }
        tc_fence_after();
        BWD_PROF(0)
        // keys this query sees in the tile: key <= q + past (causal) and key < Skv
        int lim = p.Skv - 1 - kt * 128;
        if (p.causal) lim = min(lim, q + past - kt * 128);
        const bool need_mask = (kt * 128 + 127 >= p.Skv) || (p.causal && kt * 128 + 127 > q0 + past);
        float pr[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t sv[32];
          tmem_ld32(sbuf + c * 32, sv);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            bwd_exp4(&sv[e], e, sc2, l4, &pr[c * 32 + e]);
            if (need_mask) {
#pragma unroll
              for (int w = 0; w < 4; ++w) pr[c * 32 + e + w] = (c * 32 + e + w <= lim) ? pr[c * 32 + e + w] : 0.f;
            }
          }
        }
        BWD_PROF(2)
        // ---- phase B: dP -> dS, 16-bit over the score buffer of the step (all of it is in registers by now) ----
        if (!mbar_wait_warp(&s.dp_full, cnt & 1u, ctx, kBwdCons)) {
          ok = false;
          break;
        }
        tc_fence_after();
        BWD_PROF(3)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t dv[32], dk[16];
          tmem_ld32(tmem + lane_off + 256 + c * 32, dv);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            // two elements per instruction: (dP - delta), then P * that
            const uint64_t t2 = add_f32x2(pack_f32x2(__uint_as_float(dv[e]), __uint_as_float(dv[e + 1])), ndl2);
            float x0, x1;
            unpack_f32x2(mul_f32x2(pack_f32x2(pr[c * 32 + e], pr[c * 32 + e + 1]), t2), x0, x1);
            dk[e / 2] = Pack2<T>::pack(x0, x1);
          }
          tmem_st16(sbuf + c * 16, dk);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.ds_ready);
        BWD_PROF(7)
      }
      if (!ok) break;
      if (!mbar_wait_warp(&s.acc_full, items & 1u, ctx, kBwdCons)) break;
      tc_fence_after();
      const uint32_t col_acc = static_cast<uint32_t>(grp * (D / 2));
      T* dq_row = static_cast<T*>(p.dq) + stat * D + col_acc;
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem + lane_off + 384 + col_acc + c * 32, r);
        tmem_wait_ld();
        if (live) bwd_store_row<T>(dq_row + c * 32, r, p.scale);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty);
      BWD_PROF(0)
    }
    BWD_PROF_FLUSH
   }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// delta = rowsum(O o dO): HBM-bound (reads 2 x 2 D bytes per row, writes 4 B).  D / 8 lanes share a row
// (16 bytes each); a warp covers 4 * 256 / D rows with all eight 16-byte loads of a lane in flight at once.
// ------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(256, 4) fa_bwd_preprocess_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                                 float* __restrict__ delta, int B, int H, int S,
                                                                 long long o_sb, long long o_sh, long long o_ss,
                                                                 long long g_sb, long long g_sh, long long g_ss) {
  constexpr int kLanesPerRow = D / 8, kRowsPerLoad = 32 / kLanesPerRow, kRowsPerWarp = 4 * kRowsPerLoad;
  const int lane = threadIdx.x & 31, sub = lane / kLanesPerRow, lr = lane % kLanesPerRow;
  // the host checks that B * H * S fits 31 bits: 32-bit divisions (the 64-bit ones are emulated and were
  // a visible part of this short kernel)
  const uint32_t total = static_cast<uint32_t>(B) * static_cast<uint32_t>(H) * static_cast<uint32_t>(S);
  const uint32_t row0 = (blockIdx.x * 8u + (threadIdx.x >> 5)) * kRowsPerWarp;
  uint4 a[4], g[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t row = row0 + i * kRowsPerLoad + sub;
    a[i] = make_uint4(0u, 0u, 0u, 0u);
    g[i] = a[i];
    if (row < total) {
      const uint32_t bh = row / static_cast<uint32_t>(S), sq = row - bh * static_cast<uint32_t>(S);
      const uint32_t b = bh / static_cast<uint32_t>(H), h = bh - b * static_cast<uint32_t>(H);
      a[i] = *reinterpret_cast<const uint4*>(o + b * o_sb + h * o_sh + sq * o_ss + lr * 8);
      g[i] = *reinterpret_cast<const uint4*>(d_o + b * g_sb + h * g_sh + sq * g_ss + lr * 8);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const T* ap = reinterpret_cast<const T*>(&a[i]);
    const T* gp = reinterpret_cast<const T*>(&g[i]);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc = fmaf(static_cast<float>(ap[e]), static_cast<float>(gp[e]), acc);
#pragma unroll
    for (int off = kLanesPerRow / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    const uint32_t row = row0 + i * kRowsPerLoad + sub;
    if (lr == 0 && row < total) delta[row] = acc;
  }
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
  if (a->D != 128 && a->D != 64) return set_error(HB_ERR_UNSUPPORTED, "%s: head_dim %d not supported (64, 128)", who, a->D);
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

template <typename Smem>
static int bwd_launch(void (*kernel)(const BwdParams), const BwdParams& p, int grid, int threads, const DeviceState* st,
                      cudaStream_t stream, bool* configured) {
  if ((int)sizeof(Smem) > st->smem_optin)
    return set_error(HB_ERR_UNSUPPORTED, "attention backward needs %d bytes of shared memory per CTA, the device offers %d",
                     (int)sizeof(Smem), st->smem_optin);
  if (!configured[st->device & 63]) {
    HB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
    configured[st->device & 63] = true;
  }
  kernel<<<grid, threads, sizeof(Smem), stream>>>(p);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}
template <typename T, int D>
static int launch_dkdv(const BwdParams& p, int grid, const DeviceState* st, cudaStream_t stream) {
  static bool configured[64] = {};
  return bwd_launch<BwdSmemKv<D>>(fa_bwd_dkdv_kernel<T, D>, p, grid, kBwdThreads, st, stream, configured);
}
template <typename T, int D>
static int launch_dq(const BwdParams& p, int grid, const DeviceState* st, cudaStream_t stream) {
  static bool configured[64] = {};
  return bwd_launch<BwdSmemQ<D>>(fa_bwd_dq_kernel<T, D>, p, grid, kBwdDqThreads, st, stream, configured);
}
template <typename T, int D>
static int launch_preprocess(const hb_fa_bwd_args* a, cudaStream_t stream) {
  constexpr int kRowsPerBlock = 8 * 4 * (32 / (D / 8));
  const long long rows = (long long)a->B * a->Hq * a->Sq;
  const unsigned grid = (unsigned)((rows + kRowsPerBlock - 1) / kRowsPerBlock);
  fa_bwd_preprocess_kernel<T, D><<<grid, 256, 0, stream>>>(static_cast<const T*>(a->o), static_cast<const T*>(a->d_o), a->delta,
                                                          a->B, a->Hq, a->Sq, a->o_stride_b, a->o_stride_h, a->o_stride_s,
                                                          a->do_stride_b, a->do_stride_h, a->do_stride_s);
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
  if ((long long)a->B * a->Hq * a->Sq > 0x7fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_fa_bwd_preprocess: problem too large");
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) || (reinterpret_cast<uintptr_t>(a->d_o) & 15) || (a->o_stride_s & 7) ||
      (a->o_stride_h & 7) || (a->o_stride_b & 7) || (a->do_stride_s & 7) || (a->do_stride_h & 7) || (a->do_stride_b & 7))
    return set_error(HB_ERR_ALIGN, "hb_fa_bwd_preprocess: o and d_o need 16-byte aligned rows");
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (a->dtype == HB_BF16)
    return a->D == 128 ? launch_preprocess<__nv_bfloat16, 128>(a, stream) : launch_preprocess<__nv_bfloat16, 64>(a, stream);
  return a->D == 128 ? launch_preprocess<__half, 128>(a, stream) : launch_preprocess<__half, 64>(a, stream);
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
  p.npairs = (p.nkb + 1) / 2;
  const long long total = (long long)a->B * a->Hkv * p.npairs;
  if (total > 0x3fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_fa_bwd_dkdv: problem too large");
  p.total_items = (int)total;
  int grid = (int)std::min<long long>(total, st->sm_count);
#ifdef HB_DEBUG_GRID_ENV  // measurement builds only: fewer CTAs than SMs
  if (const char* e = getenv("HB_GRID")) grid = std::max(1, std::min(grid, atoi(e)));
#endif
  if (a->dtype == HB_BF16)
    return a->D == 128 ? launch_dkdv<__nv_bfloat16, 128>(p, grid, st, stream) : launch_dkdv<__nv_bfloat16, 64>(p, grid, st, stream);
  return a->D == 128 ? launch_dkdv<__half, 128>(p, grid, st, stream) : launch_dkdv<__half, 64>(p, grid, st, stream);
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
  p.npairs = (p.nqb + 1) / 2;
  const long long total = (long long)a->B * a->Hq * p.npairs;
  if (total > 0x3fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_fa_bwd_dq: problem too large");
  p.total_items = (int)total;
  int grid = (int)std::min<long long>(total, st->sm_count);
#ifdef HB_DEBUG_GRID_ENV  // measurement builds only: fewer CTAs than SMs
  if (const char* e = getenv("HB_GRID")) grid = std::max(1, std::min(grid, atoi(e)));
#endif
  if (a->dtype == HB_BF16)
    return a->D == 128 ? launch_dq<__nv_bfloat16, 128>(p, grid, st, stream) : launch_dq<__nv_bfloat16, 64>(p, grid, st, stream);
  return a->D == 128 ? launch_dq<__half, 128>(p, grid, st, stream) : launch_dq<__half, 64>(p, grid, st, stream);
}

#ifdef HB_BWD_PROF
extern "C" int hb_debug_bwd_prof(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, hb::g_bwd_prof, sizeof(hb::g_bwd_prof)) == cudaSuccess ? 0 : 4;
}
#endif
