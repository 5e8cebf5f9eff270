// tcgen05 GEMM with fused epilogues for sm_100a:  out[M, N_out] = epilogue(a[M,K] . w[N,K]^T)
//
// Both operands are K-major (activations row-major, weights in nn.Linear layout), so
// TMA brings 128-byte-swizzled [rows x 64] slabs straight into the layout tcgen05.mma
// consumes and no transposed weight copy exists (the reference makes one,
// Heddle/heddle/frontend/codegen.py:1124-1131).  Epilogue arithmetic restates
// codegen.py:1204-1244 (fp32 on the accumulator, then cast).
//
// Persistent, warp-specialised CTA (320 threads), one 128 x 256 accumulator tile at a time:
//   warp 0     TMA producer: a 4-deep ring of {A 128x64, B 256x64} stages behind mbarriers
//   warp 1     MMA issuer: warp-uniform loop, one elected lane issues tcgen05.mma M=128 N=256 K=16, fp32 accumulators in
//              TMEM, two accumulator buffers (2 x 256 columns) so the epilogue of tile t
//              overlaps the main loop of tile t+1
//   warps 2-9  epilogue, two warpgroups: a thread owns one row and half of the tile's columns;
//              TMEM -> registers -> epilogue math -> 16-byte global stores
//
// Batched products (torch.bmm, the reference's _build_bmm_kernel, Heddle/heddle/frontend/backend.py:491-517)
// put the batch index into the tile list: the tensor maps are 3-D (K, rows, batch), a tile is
// (batch, m, n).  The second operand may also be given as [K, N] row-major (what torch.mm / bmm and
// the reference's _build_gemm_kernel, backend.py:227-252, take): its tiles are then loaded as four
// [64 k-rows x 64 columns] slabs and consumed through an MN-major shared-memory descriptor, so no
// transposed copy is made for that layout either.
//
// Epilogue classes:
//   PLAIN   row_scale, bias, unary activation, residual              (256 output columns / tile)
//   SWIGLU  B tile = 128 rows of Wg and the matching 128 rows of Wu;  out = silu(g) * u
//           (128 output columns / tile; the reference leaves this product to PyTorch,
//           codegen.py:1155-1160)
//   ROPE    rotate-half rotary embedding on head_dim-wide column groups
#pragma once

#include "ptx_sm100.cuh"

namespace hb {

constexpr int kGemmThreads = 320;  // TMA warp, MMA warp, two epilogue warpgroups
constexpr int kGemmBM = 128;
constexpr int kGemmBN = 256;
constexpr int kGemmBK = 64;
constexpr int kGemmStages = 4;
#ifndef HB_GEMM_GROUP_M
#define HB_GEMM_GROUP_M 16
#endif
constexpr int kGemmGroupM = HB_GEMM_GROUP_M;  // M-tiles per rasterisation group (L2 reuse of the weight slabs)

enum GemmEpiClass : int { kEpiPlain = 0, kEpiSwiglu = 1, kEpiRope = 2 };
enum GemmAct : int { kActNone = 0, kActSilu = 1, kActRelu = 2, kActGeluTanh = 3, kActSigmoid = 4, kActTanh = 5 };
enum GemmRole : uint32_t { kGemmRoleTma = 0x21, kGemmRoleMma = 0x22, kGemmRoleEpi = 0x23, kGemmRoleDrain = 0x24 };

struct alignas(64) GemmParams {
  CUtensorMap tm_a;
  CUtensorMap tm_w;
  CUtensorMap tm_out;  // PLAIN epilogue: [N_out, M, batch] tiles of 64 columns x 128 rows, stored by TMA
  void* out;
  const float* row_scale;
  const void* residual;
  const void* bias;
  const float* rope_cos;
  const float* rope_sin;
  uint32_t* status;
  long long ldo, ldr;
  int M, N_out, K;
  int tile_cols;  // output columns per tile (256, or 128 for SWIGLU)
  int tiles_m, tiles_n, num_tiles, k_steps;
  int act;
  int rope_seq, head_dim, rope_cols;
  int w_row2_offset;  // SWIGLU: first row of Wu inside the stacked weight
  int batch;          // number of independent products (>= 1)
  int tiles_per_batch;
  int w_kn;           // 1: the second operand is [K, N] row-major
  long long o_batch_stride, r_batch_stride;  // elements between consecutive batches of out / residual
  int tma_store;      // PLAIN epilogue: results leave through shared memory and a TMA store
  int pair_stages;    // CTA-pair kernel: depth of the operand ring (3..6) ...
  int out_slabs;      // ... and staging slabs per epilogue warpgroup (1, 2 or 4); stages + slabs = 7
};

struct GemmSmem {
  alignas(1024) uint8_t a[kGemmStages][kGemmBM * kGemmBK * 2];
  alignas(1024) uint8_t b[kGemmStages][kGemmBN * kGemmBK * 2];
  // one 128-row x 64-column (128-byte rows, 128B-swizzled) output slab per epilogue warpgroup
  alignas(1024) uint8_t stage_out[2][kGemmBM * 128];
  uint64_t full[kGemmStages], empty[kGemmStages];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

__device__ __forceinline__ void gemm_tile_coords(const GemmParams& p, int t, int& m_t, int& n_t, int& b) {
  b = t / p.tiles_per_batch;
  t -= b * p.tiles_per_batch;
  const int per_group = kGemmGroupM * p.tiles_n;
  const int g = t / per_group;
  const int first_m = g * kGemmGroupM;
  const int gsz = min(p.tiles_m - first_m, kGemmGroupM);
  const int r = t - g * per_group;
  m_t = first_m + r % gsz;
  n_t = r / gsz;
}

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case kActSilu:
      return v * (1.0f / (1.0f + __expf(-v)));
    case kActRelu:
      return fmaxf(v, 0.0f);
    case kActGeluTanh:
      return v * 0.5f * (1.0f + tanhf(0.7978845608f * (v + 0.044715f * v * v * v)));
    case kActSigmoid:
      return 1.0f / (1.0f + __expf(-v));
    case kActTanh:
      return tanhf(v);
    default:
      return v;
  }
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& w, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& w, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 w;
  w.x = Pack2<T>::pack(f[0], f[1]);
  w.y = Pack2<T>::pack(f[2], f[3]);
  w.z = Pack2<T>::pack(f[4], f[5]);
  w.w = Pack2<T>::pack(f[6], f[7]);
  return w;
}

// Stores 8 consecutive output values of one row (16 bytes), adding the residual if any.
template <typename T>
__device__ __forceinline__ void store8(const GemmParams& p, int b, int row, int col, float (&v)[8]) {
  if (p.residual != nullptr) {
    float r[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(p.residual) + b * p.r_batch_stride +
                                               (long long)row * p.ldr + col),
               r);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] += r[i];
  }
  *reinterpret_cast<uint4*>(static_cast<T*>(p.out) + b * p.o_batch_stride + (long long)row * p.ldo + col) = pack8<T>(v);
}

// Adds the residual (if any) to 8 consecutive values of one row.
template <typename T>
__device__ __forceinline__ void add_residual8(const GemmParams& p, int b, int row, int col, float (&v)[8]) {
  if (p.residual != nullptr) {
    float r[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(p.residual) + b * p.r_batch_stride +
                                               (long long)row * p.ldr + col),
               r);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] += r[i];
  }
}

template <typename T>
__device__ __forceinline__ void load_bias8(const GemmParams& p, int col, float (&b)[8]) {
  unpack8<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias) + col), b);
}

// Epilogue of one accumulator tile for the row owned by this thread.  `tacc` carries the
// warp's TMEM lane offset and the accumulator buffer's first column.  Two warpgroups share a
// tile: `part` (0 or 1) selects this thread's half of the output columns.  `release` is the
// shared::cluster address of the barrier that hands the accumulator buffer back to the MMA warp
// (this CTA's own, or the leader's when a CTA pair shares the MMA).
template <typename T, int EPI>
__device__ __forceinline__ void gemm_epilogue_row(const GemmParams& p, uint32_t tacc, int b, int m0, int n0,
                                                  int row_in_tile, int part, uint8_t* stage_base, int n_slabs, uint32_t& slab_cursor,
                                                  uint32_t release) {
  const int row = m0 + row_in_tile;
  const bool row_ok = row < p.M;
  const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[(long long)b * p.M + row] : 1.0f;

  if constexpr (EPI == kEpiPlain) {
    // The thread's half row of the accumulator (128 columns) is read with ONE wait: a TMEM load issued
    // while the tensor pipe is busy queues behind the MMAs in flight (its latency is then well over a
    // thousand cycles), so the loads are issued together and the accumulator buffer is handed back to
    // the MMA warp as soon as they have landed, before any arithmetic or store.
    uint32_t r[4][32];
#pragma unroll
    for (int h = 0; h < 4; ++h) tmem_ld32(tacc + part * (kGemmBN / 2) + h * 32, r[h]);
    tmem_wait_ld();
    tc_fence_before();
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive_cluster(release);
    // Coalesced stores: the warpgroup's 128 rows x 64 columns go to shared memory in the 128-byte
    // swizzled layout (a thread writes its own row: conflict-free), one thread hands the slab to the
    // TMA, which clips rows past M and columns past N_out.  Two slabs per tile and warpgroup.
    // The warpgroup owns a ring of `n_slabs` staging slabs; a slab is rewritten once the TMA store that
    // last used it has read it (`wait_group.read` with n_slabs - 1 younger groups allowed in flight), so
    // with several slabs the stores of consecutive slabs and tiles overlap (products with a short K loop
    // are bound by this path).  Every slab commits a group, stored or not, to keep that count exact.
    const bool issuer = row_in_tile == 0;
    const bool raw = p.row_scale == nullptr && p.bias == nullptr && p.residual == nullptr && p.act == kActNone;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int col0 = n0 + part * (kGemmBN / 2) + cc * 64;
      uint8_t* stage = stage_base + (slab_cursor % static_cast<uint32_t>(n_slabs)) * (kGemmBM * 128);
      ++slab_cursor;
      if (issuer) {
        if (n_slabs == 1) tma_store_wait_read<0>();
        else if (n_slabs == 2) tma_store_wait_read<1>();
        else tma_store_wait_read<3>();
      }
      named_bar_sync(1 + part, 128);
      if (raw) {
        // nothing to apply: round and store (products with a short K loop are bound by this path's
        // instruction count, so it carries no scale, bias, activation or residual tests)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t* x = &r[cc * 2 + h][g * 8];
            uint4 w;
            w.x = Pack2<T>::pack(__uint_as_float(x[0]), __uint_as_float(x[1]));
            w.y = Pack2<T>::pack(__uint_as_float(x[2]), __uint_as_float(x[3]));
            w.z = Pack2<T>::pack(__uint_as_float(x[4]), __uint_as_float(x[5]));
            w.w = Pack2<T>::pack(__uint_as_float(x[6]), __uint_as_float(x[7]));
            const int chunk = (h * 4 + g) ^ (row_in_tile & 7);
            *reinterpret_cast<uint4*>(stage + row_in_tile * 128 + chunk * 16) = w;
          }
        }
      } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int col = col0 + h * 32;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[cc * 2 + h][g * 8 + e]) * rs;
          const bool live = row_ok && col + g * 8 < p.N_out;
          if (p.bias != nullptr && col + g * 8 < p.N_out) {
            float bb[8];
            load_bias8<T>(p, col + g * 8, bb);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] += bb[e];
          }
          if (p.act != kActNone) {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = apply_act(v[e], p.act);
          }
          if (live) add_residual8<T>(p, b, row, col + g * 8, v);
          const int chunk = (h * 4 + g) ^ (row_in_tile & 7);
          *reinterpret_cast<uint4*>(stage + row_in_tile * 128 + chunk * 16) = pack8<T>(v);
        }
      }
      }
      fence_proxy_async();
      named_bar_sync(1 + part, 128);
      if (issuer) {
        if (col0 < p.N_out && m0 < p.M) tma_store_3d(&p.tm_out, stage, col0, m0, b);
        tma_store_commit();
      }
    }
  } else if constexpr (EPI == kEpiSwiglu) {
    // gate and up columns of this thread's half row, read with one wait (see the plain epilogue) and the
    // accumulator released before the arithmetic
    uint32_t rg[2][32], ru[2][32];
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      tmem_ld32(tacc + (part * 2 + cc) * 32, rg[cc]);
      tmem_ld32(tacc + 128 + (part * 2 + cc) * 32, ru[cc]);
    }
    tmem_wait_ld();
    tc_fence_before();
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive_cluster(release);
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int col = n0 + (part * 2 + cc) * 32;
      if (!row_ok || col >= p.N_out) continue;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (col + g * 8 >= p.N_out) break;
        float v[8], u[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          v[e] = __uint_as_float(rg[cc][g * 8 + e]) * rs;
          u[e] = __uint_as_float(ru[cc][g * 8 + e]) * rs;
        }
        if (p.bias != nullptr) {
          float bg[8], bu[8];
          load_bias8<T>(p, col + g * 8, bg);
          load_bias8<T>(p, p.w_row2_offset + col + g * 8, bu);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            v[e] += bg[e];
            u[e] += bu[e];
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = v[e] * (1.0f / (1.0f + __expf(-v[e]))) * u[e];
        store8<T>(p, b, row, col + g * 8, v);
      }
    }
  } else {  // kEpiRope
    const int hd = p.head_dim, half = hd >> 1;
    const int pos = row_ok ? (row % p.rope_seq) : 0;
    const float* cosr = p.rope_cos + (long long)pos * half;
    const float* sinr = p.rope_sin + (long long)pos * half;
    // two or more heads per tile: each warpgroup takes whole heads; one 256-wide head: each takes
    // half of the rotation pairs
    const bool split_heads = hd <= kGemmBN / 2;
    const int h_begin = split_heads ? part * (kGemmBN / 2) : 0, h_end = split_heads ? h_begin + kGemmBN / 2 : kGemmBN;
    const int c_begin = split_heads ? 0 : part * (half / 2), c_end = split_heads ? half : c_begin + half / 2;
    // rotation of 32 column pairs (x1 = columns h0 + c .., x2 = the same columns half a head further)
    auto rotate_store = [&](const uint32_t (&r1)[32], const uint32_t (&r2)[32], int h0, int c) {
      const int col = n0 + h0 + c;
      if (!row_ok || col >= p.N_out) return;
      const bool rotate = col < p.rope_cols;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float x1[8], x2[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          x1[e] = __uint_as_float(r1[g * 8 + e]) * rs;
          x2[e] = __uint_as_float(r2[g * 8 + e]) * rs;
        }
        if (p.bias != nullptr) {
          float b1[8], b2[8];
          load_bias8<T>(p, col + g * 8, b1);
          load_bias8<T>(p, col + half + g * 8, b2);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            x1[e] += b1[e];
            x2[e] += b2[e];
          }
        }
        if (rotate) {
          // eight consecutive angles as two 16-byte loads per table (rows are 16-byte aligned:
          // head_dim / 2 is a multiple of 32)
          const float4 c0 = *reinterpret_cast<const float4*>(cosr + c + g * 8), c1 = *reinterpret_cast<const float4*>(cosr + c + g * 8 + 4);
          const float4 s0 = *reinterpret_cast<const float4*>(sinr + c + g * 8), s1 = *reinterpret_cast<const float4*>(sinr + c + g * 8 + 4);
          const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float xa = x1[e], xb = x2[e];
            x1[e] = xa * cs[e] - xb * sn[e];
            x2[e] = xb * cs[e] + xa * sn[e];
          }
        }
        store8<T>(p, b, row, col + g * 8, x1);
        store8<T>(p, b, row, col + half + g * 8, x2);
      }
    };
    auto release_acc = [&]() {
      tc_fence_before();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive_cluster(release);
    };
    if (split_heads) {
      // head_dim 64 or 128: the warpgroup's 128 columns are read with one wait and the accumulator is
      // released before the arithmetic (see the plain epilogue)
      uint32_t r[4][32];
#pragma unroll
      for (int h = 0; h < 4; ++h) tmem_ld32(tacc + h_begin + h * 32, r[h]);
      tmem_wait_ld();
      release_acc();
      if (hd == 128) {
        rotate_store(r[0], r[2], h_begin, 0);
        rotate_store(r[1], r[3], h_begin, 32);
      } else {
        rotate_store(r[0], r[1], h_begin, 0);
        rotate_store(r[2], r[3], h_begin + 64, 0);
      }
    } else {
#pragma unroll 1
      for (int h0 = h_begin; h0 < h_end; h0 += hd) {
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 32) {
          uint32_t r1[32], r2[32];
          __syncwarp();
          tmem_ld32(tacc + h0 + c, r1);
          tmem_ld32(tacc + h0 + half + c, r2);
          tmem_wait_ld();
          rotate_store(r1, r2, h0, c);
        }
      }
      release_acc();
    }
  }
}

template <typename T, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  GemmSmem& s = *reinterpret_cast<GemmSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{&s.abort_flag, p.status};

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < kGemmStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 8);
    }
    mbar_init(&s.drain, 1);
    fence_mbar_init();
    if ((smem_u32(smem_raw) & 1023u) != 0u) raise_abort(ctx, kStatusSmemMisaligned);
    prefetch_tensormap(&p.tm_a);
    prefetch_tensormap(&p.tm_w);
    if (p.tma_store) prefetch_tensormap(&p.tm_out);
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const bool run = (s.abort_flag == 0);

  if (warp == 0) {
    if (run && lane == 0) {
      // ---------------- TMA producer ----------------
      constexpr uint32_t kStageBytes = (kGemmBM + kGemmBN) * kGemmBK * 2;
      uint32_t st = 0, phase = 1;  // "empty" barriers start out free
      bool ok = true;
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        int m_t, n_t, b;
        gemm_tile_coords(p, t, m_t, n_t, b);
        const int m0 = m_t * kGemmBM;
        const int n0 = n_t * p.tile_cols;
        const int row_b0 = n0;
        const int row_b1 = (EPI == kEpiSwiglu) ? (p.w_row2_offset + n0) : (n0 + 128);
        for (int ks = 0; ks < p.k_steps; ++ks) {
          if (!mbar_wait(&s.empty[st], phase, ctx, kGemmRoleTma)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&s.full[st], kStageBytes);
          tma_load_3d(s.a[st], &p.tm_a, &s.full[st], ks * kGemmBK, m0, b);
          if (p.w_kn) {
            // [K, N] operand: four slabs of 64 k-rows x 64 columns (128 bytes per row)
#pragma unroll
            for (int i = 0; i < kGemmBN / 64; ++i)
              tma_load_3d(s.b[st] + i * (kGemmBK * 128), &p.tm_w, &s.full[st], n0 + i * 64, ks * kGemmBK, b);
          } else {
            tma_load_3d(s.b[st], &p.tm_w, &s.full[st], ks * kGemmBK, row_b0, b);
            tma_load_3d(s.b[st] + 128 * kGemmBK * 2, &p.tm_w, &s.full[st], ks * kGemmBK, row_b1, b);
          }
          if (++st == kGemmStages) {
            st = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (run) {
      // ---------------- MMA issuer: the whole warp runs the loop (operands stay warp-uniform),
      // one elected lane issues ----------------
      constexpr uint32_t idesc_nk = make_idesc(Pack2<T>::kFormat, kGemmBM, kGemmBN, 0, 0);
      constexpr uint32_t idesc_kn = make_idesc(Pack2<T>::kFormat, kGemmBM, kGemmBN, 0, 1);
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kLbo = (16u >> 4) << 16;
      // [K, N] operand (MN-major): the next 64 columns live one slab (64 k-rows x 128 bytes) further,
      // a K = 16 step advances by 16 rows of 128 bytes
      constexpr uint32_t kLboKn = ((kGemmBK * 128u) >> 4) << 16;
      const uint32_t idesc = p.w_kn ? idesc_kn : idesc_nk;
      const uint32_t b_lbo = p.w_kn ? kLboKn : kLbo;
      const uint32_t b_step = p.w_kn ? (16u * 128u >> 4) : 2u;
      const bool leader = elect_one();
      uint32_t stage = 0, phase = 0, tile_i = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x, ++tile_i) {
        const uint32_t acc = tile_i & 1;
        if (!mbar_wait_warp(&s.acc_empty[acc], ((tile_i >> 1) & 1) ^ 1, ctx, kGemmRoleMma)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * kGemmBN;
        for (int ks = 0; ks < p.k_steps; ++ks) {
          if (!mbar_wait_warp(&s.full[stage], phase, ctx, kGemmRoleMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = (smem_u32(s.a[stage]) >> 4) | kLbo, b_lo = (smem_u32(s.b[stage]) >> 4) | b_lbo;
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < kGemmBK / 16; ++kk) {
              umma_ss_f16(d_tmem, (static_cast<uint64_t>(kDescHi) << 32) | (a_lo + kk * 2),
                          (static_cast<uint64_t>(kDescHi) << 32) | (b_lo + kk * b_step), idesc, (ks > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(&s.empty[stage]);
          }
          if (++stage == kGemmStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && leader) umma_commit(&s.acc_full[acc]);
      }
      __syncwarp();
      if (s.abort_flag && lane == 0) {
        umma_commit(&s.drain);
        mbar_wait(&s.drain, 0, ctx, kGemmRoleDrain);
      }
    }
    __syncwarp();
  } else if (run) {
    // ---------------- epilogue warps ----------------
    const int quarter = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t tile_i = 0, slab_cursor = 0;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++tile_i) {
      int m_t, n_t, b;
      gemm_tile_coords(p, t, m_t, n_t, b);
      const uint32_t acc = tile_i & 1;
      if (!mbar_wait_warp(&s.acc_full[acc], (tile_i >> 1) & 1, ctx, kGemmRoleEpi)) break;
      tc_fence_after();
      gemm_epilogue_row<T, EPI>(p, tmem + lane_off + acc * kGemmBN, b, m_t * kGemmBM, n_t * p.tile_cols,
                                quarter * 32 + lane, (warp - 2) >> 2, s.stage_out[(warp - 2) >> 2], 1, slab_cursor,
                                smem_u32(&s.acc_empty[acc]));
      // the epilogue hands the accumulator buffer back itself (acc_empty), as soon as it has read it
    }
    // the slabs handed to the TMA must have been written out before shared memory goes away
    if (p.tma_store && quarter == 0 && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// The same GEMM on CTA pairs: a cluster of two CTAs owns a 256 x 256 accumulator tile and the
// leader's MMA warp issues tcgen05.mma.cta_group::2 (M = 256).  Each CTA loads only its own 128 rows
// of A and its own 128 of the tile's 256 B rows (plain tiled TMA loads, no multicast) and holds its
// 128 x 256 half of the accumulator in its own TMEM, so a CTA moves 32 KB per K step of 64 through
// shared memory instead of 48 KB and the ring is 6 stages deep.  Epilogues are the single-CTA ones.
//
// Barriers: the leader's full[s] counts the bytes of both CTAs' loads; empty[s] and acc_full[a] exist in
// both CTAs and the leader's MMA warp commits to each (two commits, no multicast); the leader's
// acc_empty[a] collects the 8 epilogue warps of both CTAs.  Every wait is on a barrier of the waiting
// CTA and is bounded like the single-CTA kernel's.  Before a CTA leaves, its producer has seen every
// commit aimed at its ring, the leader has seen every release aimed at it, and the pair meets at a
// cluster barrier, so nothing can arrive at shared memory that is gone.
// ------------------------------------------------------------------------------------------
constexpr int kPairBM = 256;  // rows of a pair's tile (128 per CTA)
constexpr int kPairMaxStages = 6;
constexpr int kPairSlots = 7;              // 32 KB slots of shared memory: ring stages + staging slabs per warpgroup
constexpr int kPairStageA = kGemmBM * kGemmBK * 2;        // 16 KB
constexpr int kPairStageB = (kGemmBN / 2) * kGemmBK * 2;  // 16 KB
constexpr int kPairSlab = kGemmBM * 128;                  // 16 KB: 128 rows x 64 columns

// Shared memory of the pair kernel, carved at run time: [A ring][B ring][staging slabs: warpgroup 0, 1][control].
// Long K loops get the deepest ring and one slab per warpgroup; short ones, which are bound by the stores,
// trade ring stages for slabs (GemmParams::pair_stages / out_slabs).
struct GemmPairCtrl {
  uint64_t full[kPairMaxStages], empty[kPairMaxStages];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
};
constexpr int kPairSmemBytes = kPairSlots * 32768 + static_cast<int>(sizeof(GemmPairCtrl));

// bounded wait that also orders against the peer CTA's arrivals
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const AbortCtx& ctx, uint32_t role) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 0xFFu) == 0u) {
      if (*ctx.cta_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > ctx.limit_ns) {
        raise_abort(ctx, kStatusWaitTimeout | role);
        return false;
      }
    }
  }
}

// tile t of the pair grid: tiles_m counts 256-row tiles
__device__ __forceinline__ void gemm_pair_tile_coords(const GemmParams& p, int t, int& m_t, int& n_t, int& b) {
  gemm_tile_coords(p, t, m_t, n_t, b);
}

template <typename T, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1) gemm_pair_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int kStages = p.pair_stages;
  uint8_t* const ring_a = smem_raw;
  uint8_t* const ring_b = ring_a + kStages * kPairStageA;
  uint8_t* const slabs = ring_b + kStages * kPairStageB;
  GemmPairCtrl& s = *reinterpret_cast<GemmPairCtrl*>(smem_raw + kPairSlots * 32768);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  AbortCtx ctx{&s.abort_flag, p.status};

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < kPairMaxStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 16);  // 8 epilogue warps of each CTA (used in the leader only)
    }
    mbar_init(&s.drain, 1);
    fence_mbar_init();
    if ((smem_u32(smem_raw) & 1023u) != 0u) raise_abort(ctx, kStatusSmemMisaligned);
    prefetch_tensormap(&p.tm_a);
    prefetch_tensormap(&p.tm_w);
    if (p.tma_store) prefetch_tensormap(&p.tm_out);
  }
  if (warp == 1) {
    tmem_alloc_pair(&s.tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // both CTAs' barriers are initialised before anything arrives at them
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const bool run = (s.abort_flag == 0);

  if (warp == 0) {
    if (run && lane == 0) {
      // ---------------- TMA producer (both CTAs) ----------------
      constexpr uint32_t kPairStageBytes = 2u * (kGemmBM + kGemmBN / 2) * kGemmBK * 2;  // both CTAs' loads
      uint32_t st = 0, phase = 1;
      bool ok = true;
      for (int t = pair; ok && t < p.num_tiles; t += n_pairs) {
        int m_t, n_t, b;
        gemm_pair_tile_coords(p, t, m_t, n_t, b);
        const int m0 = m_t * kPairBM + static_cast<int>(rank) * kGemmBM;
        const int n0 = n_t * p.tile_cols;
        // this CTA's 128 B rows: the first or the second half of a plain tile; the gate (leader) or the up
        // (peer) rows of a SwiGLU tile
        const int row_b = (EPI == kEpiSwiglu) ? (rank == 0 ? n0 : p.w_row2_offset + n0) : n0 + static_cast<int>(rank) * 128;
        for (int ks = 0; ks < p.k_steps; ++ks) {
          if (!mbar_wait(&s.empty[st], phase, ctx, kGemmRoleTma)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = mapa_u32(smem_u32(&s.full[st]), 0);
          if (rank == 0) mbar_arrive_expect_tx(&s.full[st], kPairStageBytes);
          tma_load_3d_pair(ring_a + st * kPairStageA, &p.tm_a, full_leader, ks * kGemmBK, m0, b);
          if (p.w_kn) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
              tma_load_3d_pair(ring_b + st * kPairStageB + i * (kGemmBK * 128), &p.tm_w, full_leader, row_b + i * 64, ks * kGemmBK, b);
          } else {
            tma_load_3d_pair(ring_b + st * kPairStageB, &p.tm_w, full_leader, ks * kGemmBK, row_b, b);
          }
          if (++st == static_cast<uint32_t>(kStages)) {
            st = 0;
            phase ^= 1;
          }
        }
      }
      // tail: every commit aimed at this CTA's ring has arrived before the CTA may leave (a slot that
      // was never filled passes at once)
      for (int i = 0; ok && i < kStages; ++i) {
        if (!mbar_wait(&s.empty[st], phase, ctx, kGemmRoleTma)) break;
        if (++st == static_cast<uint32_t>(kStages)) {
          st = 0;
          phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (run && rank == 0) {
      // ---------------- MMA issuer (leader CTA only) ----------------
      constexpr uint32_t idesc_nk = make_idesc(Pack2<T>::kFormat, kPairBM, kGemmBN, 0, 0);
      constexpr uint32_t idesc_kn = make_idesc(Pack2<T>::kFormat, kPairBM, kGemmBN, 0, 1);
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kLbo = (16u >> 4) << 16;
      constexpr uint32_t kLboKn = ((kGemmBK * 128u) >> 4) << 16;
      const uint32_t idesc = p.w_kn ? idesc_kn : idesc_nk;
      const uint32_t b_lbo = p.w_kn ? kLboKn : kLbo;
      const uint32_t b_step = p.w_kn ? (16u * 128u >> 4) : 2u;
      const bool leader = elect_one();
      uint32_t stage = 0, phase = 0, tile_i = 0;
      bool ok = true;
      for (int t = pair; ok && t < p.num_tiles; t += n_pairs, ++tile_i) {
        const uint32_t acc = tile_i & 1;
        bool got = mbar_wait_cluster(&s.acc_empty[acc], ((tile_i >> 1) & 1) ^ 1, ctx, kGemmRoleMma);
        got = __all_sync(0xffffffffu, got);
        if (!got) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * kGemmBN;
        for (int ks = 0; ks < p.k_steps; ++ks) {
          if (!mbar_wait_warp(&s.full[stage], phase, ctx, kGemmRoleMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = (smem_u32(ring_a + stage * kPairStageA) >> 4) | kLbo;
          const uint32_t b_lo = (smem_u32(ring_b + stage * kPairStageB) >> 4) | b_lbo;
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < kGemmBK / 16; ++kk) {
              umma_ss_f16_pair(d_tmem, (static_cast<uint64_t>(kDescHi) << 32) | (a_lo + kk * 2),
                               (static_cast<uint64_t>(kDescHi) << 32) | (b_lo + kk * b_step), idesc, (ks > 0 || kk > 0) ? 1u : 0u);
            }
            const uint32_t e = smem_u32(&s.empty[stage]);
            umma_commit_pair(mapa_u32(e, 0));
            umma_commit_pair(mapa_u32(e, 1));
          }
          if (++stage == static_cast<uint32_t>(kStages)) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && leader) {
          const uint32_t f = smem_u32(&s.acc_full[acc]);
          umma_commit_pair(mapa_u32(f, 0));
          umma_commit_pair(mapa_u32(f, 1));
        }
      }
      // tail: the peer's last releases have arrived here before the leader may leave
      for (uint32_t a = 0; ok && a < 2 && a < tile_i; ++a) {
        const uint32_t uses = (tile_i + 1 - a) >> 1;  // tiles that used buffer a
        bool got = mbar_wait_cluster(&s.acc_empty[a], (uses - 1) & 1, ctx, kGemmRoleMma);
        got = __all_sync(0xffffffffu, got);
        if (!got) break;
      }
      __syncwarp();
      if (s.abort_flag && lane == 0) {
        umma_commit_pair(mapa_u32(smem_u32(&s.drain), 0));
        mbar_wait(&s.drain, 0, ctx, kGemmRoleDrain);
      }
    }
    __syncwarp();
  } else if (run) {
    // ---------------- epilogue warps (both CTAs, each on its own 128 rows) ----------------
    const int quarter = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t tile_i = 0, slab_cursor = 0;
    uint8_t* const my_slabs = slabs + ((warp - 2) >> 2) * p.out_slabs * kPairSlab;
    for (int t = pair; t < p.num_tiles; t += n_pairs, ++tile_i) {
      int m_t, n_t, b;
      gemm_pair_tile_coords(p, t, m_t, n_t, b);
      const uint32_t acc = tile_i & 1;
      if (!mbar_wait_warp(&s.acc_full[acc], (tile_i >> 1) & 1, ctx, kGemmRoleEpi)) break;
      tc_fence_after();
      gemm_epilogue_row<T, EPI>(p, tmem + lane_off + acc * kGemmBN, b, m_t * kPairBM + static_cast<int>(rank) * kGemmBM,
                                n_t * p.tile_cols, quarter * 32 + lane, (warp - 2) >> 2, my_slabs, p.out_slabs, slab_cursor,
                                mapa_u32(smem_u32(&s.acc_empty[acc]), 0));
    }
    if (p.tma_store && quarter == 0 && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  cluster_sync_all();  // the leader's MMAs read the peer's shared memory: nobody leaves before all are done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// RMSNorm row statistic fused with the residual add (HBM-bound): one warp per row.
//   y = x (+ residual), rounded to T;  rstd[m] = rsqrt(mean(y^2) + eps)
// ------------------------------------------------------------------------------------------
// 16-byte read-once load that does not displace L1 lines
template <typename T>
__device__ __forceinline__ uint4 ld_stream(const T* ptr) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256) rms_rowstat_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                                                          T* __restrict__ y_out, float* __restrict__ rstd, int M,
                                                          int N, long long ldx, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= M) return;
  const T* xr = x + (long long)row * ldx;
  const T* rr = residual != nullptr ? residual + (long long)row * ldx : nullptr;
  T* yr = y_out != nullptr ? y_out + (long long)row * ldx : nullptr;
  float acc = 0.f;
  auto consume = [&](const uint4& xv, const uint4& rv, int c) {
    float v[8];
    unpack8<T>(xv, v);
    if (rr != nullptr) {
      float r[8];
      unpack8<T>(rv, r);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += r[e];
    }
    const uint4 packed = pack8<T>(v);
    if (yr != nullptr) *reinterpret_cast<uint4*>(yr + c) = packed;
    float w[8];
    unpack8<T>(packed, w);  // statistics of the rounded values, as a consumer of y sees them
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += w[e] * w[e];
  };
  // four 16-byte loads per operand in flight per lane (1 KB per warp and operand) before any use
  constexpr int kStride = 32 * 8, kBatch = 4;
  int c = lane * 8;
  for (; c + (kBatch - 1) * kStride < N; c += kBatch * kStride) {
    uint4 xv[kBatch], rv[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) xv[u] = ld_stream(xr + c + u * kStride);
    if (rr != nullptr) {
#pragma unroll
      for (int u = 0; u < kBatch; ++u) rv[u] = ld_stream(rr + c + u * kStride);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) consume(xv[u], rv[u], c + u * kStride);
  }
  for (; c < N; c += kStride) {
    const uint4 xv = ld_stream(xr + c);
    uint4 rv = xv;
    if (rr != nullptr) rv = ld_stream(rr + c);
    consume(xv, rv, c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) rstd[row] = rsqrtf(acc / (float)N + eps);
}

// ------------------------------------------------------------------------------------------
// weight preparation: row-stack up to four [rows_i, K] matrices, optional column scale
// ------------------------------------------------------------------------------------------
struct PrepareParams {
  const void* src[4];
  long long ld_src[4];
  int row_end[4];  // exclusive prefix sums of the row counts
  int n_src, K;
  const void* gamma;
  void* out;
  long long ld_out;
};

template <typename T>
__global__ void __launch_bounds__(256) prepare_weight_kernel(const PrepareParams p) {
  const int chunks = p.K / 8;  // 16-byte chunks per row
  const long long total = static_cast<long long>(p.row_end[p.n_src - 1]) * chunks;
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total; idx += 256ll * gridDim.x) {
    const int row = static_cast<int>(idx / chunks), c = static_cast<int>(idx - static_cast<long long>(row) * chunks) * 8;
    int which = 0, base = 0;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      if (i + 1 < p.n_src && row >= p.row_end[i]) {
        which = i + 1;
        base = p.row_end[i];
      }
    }
    const T* srow = static_cast<const T*>(p.src[which]) + static_cast<long long>(row - base) * p.ld_src[which];
    uint4 w = ld_stream(srow + c);
    if (p.gamma != nullptr) {
      float v[8], g[8];
      unpack8<T>(w, v);
      unpack8<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(p.gamma) + c), g);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= g[e];
      w = pack8<T>(v);
    }
    *reinterpret_cast<uint4*>(static_cast<T*>(p.out) + static_cast<long long>(row) * p.ld_out + c) = w;
  }
}

}  // namespace hb
