// hb_rowwise_program: pointwise chains and row reductions over a [rows, cols] matrix, driven by a
// small op-code program instead of generated source.
//
// The reference emits TileLang source text for such partitions and compiles it at run time:
// pointwise chains (Heddle/heddle/frontend/codegen.py:1457-1498, op table _map_op :1577-1609) and
// softmax-like / sum / mean / max reductions over the last axis (:1246-1455: one pass per reduction
// that recomputes the expression up to it, results kept in fp32, then an output pass).  Here the
// FX lowering linearises the same partition into an accumulator-machine program.  This file holds
// the argument checks and the precompiled kernels that INTERPRET such a program (used when the
// caller asks for it or when NVRTC cannot be loaded); rowprog_jit.cu turns the same program into a
// kernel specialised for it, which is the default path.
//
// Machine, per group of 8 consecutive columns of a row (16 bytes of a 16-bit tensor):
//   acc[8]           the running value (fp32), in registers
//   tmp[4][8]        saved values (HB_EW_STORE_TMP), in shared memory
//   red[4]           row reductions computed by earlier passes (one scalar per row)
// An instruction is `acc = op(acc, operand)`; the operand is a full input tensor (16-byte load), a
// [cols] vector broadcast over rows, a [rows] fp32 vector broadcast over columns, an immediate, a
// temporary or a reduction result.  Unary ops ignore the operand.  The op code is warp-uniform, so
// the switch costs a handful of uniform instructions per 8 elements.
//
// Passes: a program with R reductions runs R + 1 times over the row — pass r executes the prefix
// that ends at the r-th HB_EW_REDUCE_* instruction and reduces acc over the row (warp shuffles, plus
// shared memory when four warps share a row); the last pass executes the whole program and is the
// only one that stores.  Inputs are re-read per pass (from L1/L2: a row is a few KB), HBM sees each
// input once.  Without reductions the kernel is a flat grid-stride stream over 16-byte groups.
//
// Rounding: HB_EW_ROUND rounds acc to the tensors' 16-bit type and back, which reproduces the
// intermediate tensors of the eager graph; the lowering decides where it is needed.
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "rowprog_sm100.cuh"

#include <algorithm>
#include <cstring>
#include <mutex>

namespace hb {

template <typename T>
__device__ __forceinline__ void rp_unpack8(const uint4& w, float (&f)[8]);
template <>
__device__ __forceinline__ void rp_unpack8<__nv_bfloat16>(const uint4& w, float (&f)[8]) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void rp_unpack8<__half>(const uint4& w, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 rp_pack8(const float (&f)[8]) {
  uint4 w;
  w.x = Pack2<T>::pack(f[0], f[1]);
  w.y = Pack2<T>::pack(f[2], f[3]);
  w.z = Pack2<T>::pack(f[4], f[5]);
  w.w = Pack2<T>::pack(f[6], f[7]);
  return w;
}

// exp, reciprocal and friends through the MUFU: the results are rounded to 16 bits, for which the
// approximate units (2 ulp of fp32) are exact enough, and an interpreter that has to stay under the
// HBM roofline cannot afford the multi-instruction accurate versions.
__device__ __forceinline__ float rp_exp(float x) { return fast_exp2(x * 1.4426950408889634f); }
__device__ __forceinline__ float rp_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rp_sigmoid(float x) { return rp_rcp(1.0f + fast_exp2(x * -1.4426950408889634f)); }
__device__ __forceinline__ float rp_tanh(float x) {
  // 1 - 2 / (1 + exp(2x)); saturates correctly for large |x| (exp -> inf gives 1, exp -> 0 gives -1)
  return fmaf(-2.0f, rp_rcp(1.0f + fast_exp2(x * 2.8853900817779268f)), 1.0f);
}

// Register state of the machine: kG groups of 8 columns are interpreted together, so that one
// decode serves 16 elements and a thread keeps several 16-byte loads in flight.
constexpr int kG = 2;
constexpr int kE = 8 * kG;
constexpr int kRpThreads = 128;
// The accumulator lives in registers; the temporaries, which are touched far less often and are
// selected by a run-time index, live in shared memory ([slot][element][thread]: conflict-free).
struct RowProgState {
  float acc[kE];
  float* tmp;  // this thread's column of the shared temporaries
};
__device__ __forceinline__ float& rp_tmp(const RowProgState& s, int slot, int e) { return s.tmp[(slot * kE + e) * kRpThreads]; }

// Executes instructions [0, end) for kG groups of 8 columns: group g covers columns col[g].. of
// row[g] (`ok[g]` false = past the end: nothing is loaded or stored for it).  `red` holds the
// reductions of earlier passes; `store` is true in the last pass only.
template <typename T>
__device__ __forceinline__ void rowprog_run(const RowProgParams& p, int end, const long long (&row)[kG], const int (&col)[kG],
                                            const bool (&ok)[kG], const float (&red)[4], bool store, RowProgState& s) {
#pragma unroll 1
  for (int pc = 0; pc < end; ++pc) {
    const hb_ew_inst inst = p.prog[pc];
    float v[kE];
    // ---- operand
    switch (inst.src) {
      case HB_SRC_INPUT: {
        const T* base = static_cast<const T*>(p.in[inst.index]);
        const long long ld = p.ld_in[inst.index];
        uint4 w[kG];
#pragma unroll
        for (int g = 0; g < kG; ++g) w[g] = ok[g] ? *reinterpret_cast<const uint4*>(base + row[g] * ld + col[g]) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int g = 0; g < kG; ++g) rp_unpack8<T>(w[g], *reinterpret_cast<float(*)[8]>(&v[8 * g]));
        break;
      }
      case HB_SRC_ROWVEC: {
        const T* base = static_cast<const T*>(p.rowvec[inst.index]);
#pragma unroll
        for (int g = 0; g < kG; ++g) {
          const uint4 w = ok[g] ? *reinterpret_cast<const uint4*>(base + col[g]) : make_uint4(0, 0, 0, 0);
          rp_unpack8<T>(w, *reinterpret_cast<float(*)[8]>(&v[8 * g]));
        }
        break;
      }
      case HB_SRC_ROWSCALAR: {
#pragma unroll
        for (int g = 0; g < kG; ++g) {
          const float x = ok[g] ? p.rowscalar[inst.index][row[g]] : 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) v[8 * g + e] = x;
        }
        break;
      }
      case HB_SRC_TMP:
#pragma unroll
        for (int e = 0; e < kE; ++e) v[e] = rp_tmp(s, inst.index, e);
        break;
      case HB_SRC_REDUCED: {
        const float x = inst.index == 0 ? red[0] : inst.index == 1 ? red[1] : inst.index == 2 ? red[2] : red[3];
#pragma unroll
        for (int e = 0; e < kE; ++e) v[e] = x;
        break;
      }
      case HB_SRC_IMM:
#pragma unroll
        for (int e = 0; e < kE; ++e) v[e] = inst.imm;
        break;
      default:  // HB_SRC_NONE: unary ops, stores and reductions read no operand
        break;
    }
    // ---- operation (formulas: Heddle/heddle/frontend/codegen.py:1577-1609)
    float (&a)[kE] = s.acc;
#define HB_RP_EACH(expr)              \
  _Pragma("unroll") for (int e = 0; e < kE; ++e) { a[e] = (expr); } \
  break
    switch (inst.op) {
      case HB_EW_LOAD: HB_RP_EACH(v[e]);
      case HB_EW_ADD: HB_RP_EACH(a[e] + v[e]);
      case HB_EW_SUB: HB_RP_EACH(a[e] - v[e]);
      case HB_EW_RSUB: HB_RP_EACH(v[e] - a[e]);
      case HB_EW_MUL: HB_RP_EACH(a[e] * v[e]);
      case HB_EW_DIV: HB_RP_EACH(a[e] * rp_rcp(v[e]));
      case HB_EW_RDIV: HB_RP_EACH(v[e] * rp_rcp(a[e]));
      case HB_EW_MAX: HB_RP_EACH(fmaxf(a[e], v[e]));
      case HB_EW_MIN: HB_RP_EACH(fminf(a[e], v[e]));
      case HB_EW_POW: HB_RP_EACH(powf(a[e], v[e]));
      case HB_EW_NEG: HB_RP_EACH(-a[e]);
      case HB_EW_ABS: HB_RP_EACH(fabsf(a[e]));
      case HB_EW_EXP: HB_RP_EACH(rp_exp(a[e]));
      case HB_EW_LOG: HB_RP_EACH(fast_log2(a[e]) * 0.6931471805599453f);
      case HB_EW_LOG2: HB_RP_EACH(fast_log2(a[e]));
      case HB_EW_SQRT: HB_RP_EACH(sqrtf(a[e]));
      case HB_EW_RSQRT: HB_RP_EACH(rsqrtf(a[e]));
      case HB_EW_RECIP: HB_RP_EACH(rp_rcp(a[e]));
      case HB_EW_SIGMOID: HB_RP_EACH(rp_sigmoid(a[e]));
      case HB_EW_SILU: HB_RP_EACH(a[e] * rp_sigmoid(a[e]));
      case HB_EW_RELU: HB_RP_EACH(fmaxf(a[e], 0.0f));
      case HB_EW_GELU_TANH: HB_RP_EACH(a[e] * 0.5f * (1.0f + rp_tanh(0.7978845608f * (a[e] + 0.044715f * a[e] * a[e] * a[e]))));
      case HB_EW_GELU_ERF: HB_RP_EACH(a[e] * 0.5f * (1.0f + erff(a[e] * 0.7071067811865476f)));
      case HB_EW_TANH: HB_RP_EACH(rp_tanh(a[e]));
      case HB_EW_ROUND:
#pragma unroll
        for (int g = 0; g < kG; ++g) {
          float (&ag)[8] = *reinterpret_cast<float(*)[8]>(&a[8 * g]);
          const uint4 w = rp_pack8<T>(ag);
          rp_unpack8<T>(w, ag);
        }
        break;
      case HB_EW_STORE_TMP:
#pragma unroll
        for (int e = 0; e < kE; ++e) rp_tmp(s, inst.index, e) = a[e];
        break;
      case HB_EW_STORE_OUT:
        if (store) {
          T* base = static_cast<T*>(p.out[inst.index]);
          const long long ld = p.ld_out[inst.index];
#pragma unroll
          for (int g = 0; g < kG; ++g) {
            if (ok[g]) *reinterpret_cast<uint4*>(base + row[g] * ld + col[g]) = rp_pack8<T>(*reinterpret_cast<float(*)[8]>(&a[8 * g]));
          }
        }
        break;
      default:  // HB_EW_REDUCE_*: a no-op inside a pass (the pass that ends here reduces acc afterwards)
        break;
    }
#undef HB_RP_EACH
  }
}

// No reductions: a flat stream over the 16-byte groups of the matrix.
template <typename T>
__global__ void __launch_bounds__(kRpThreads) rowprog_stream_kernel(const __grid_constant__ RowProgParams p) {
  extern __shared__ float tmp_s[];  // [temporaries the program uses][kE][threads]
  const unsigned groups = static_cast<unsigned>(p.cols >> 3);
  const unsigned total = static_cast<unsigned>(p.rows) * groups;  // the host checks that this fits 32 bits
  const float red[4] = {0.f, 0.f, 0.f, 0.f};
  // a thread takes kG groups that are one block width apart, so that a warp's loads stay contiguous;
  // 32-bit index arithmetic (a 64-bit division per group would cost more than the program itself)
  const unsigned stride = kRpThreads * kG * gridDim.x;
  for (unsigned g0 = blockIdx.x * (kRpThreads * kG) + threadIdx.x; g0 < total; g0 += stride) {
    long long row[kG];
    int col[kG];
    bool ok[kG];
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const unsigned idx = g0 + kRpThreads * g;
      ok[g] = idx < total && idx >= g0;  // the second test guards the 32-bit wrap of the last batch
      const unsigned r = ok[g] ? idx / groups : 0u;
      row[g] = r;
      col[g] = ok[g] ? static_cast<int>(idx - r * groups) << 3 : 0;
    }
    if (g0 + stride < g0) {  // next index would wrap: this was the last batch of this thread
      RowProgState s;
      s.tmp = tmp_s + threadIdx.x;
      rowprog_run<T>(p, p.n_inst, row, col, ok, red, true, s);
      break;
    }
    RowProgState s;
    s.tmp = tmp_s + threadIdx.x;
    rowprog_run<T>(p, p.n_inst, row, col, ok, red, true, s);
  }
}

// With reductions: kWarpsPerRow warps (1 or 4) own a row; 128-thread CTAs.
template <typename T, int kWarpsPerRow>
__global__ void __launch_bounds__(kRpThreads) rowprog_reduce_kernel(const __grid_constant__ RowProgParams p) {
  constexpr int kThreadsPerRow = 32 * kWarpsPerRow;
  constexpr int kRowsPerCta = 4 / kWarpsPerRow;
  __shared__ float part[4];
  extern __shared__ float tmp_s[];  // [temporaries the program uses][kE][threads]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = kWarpsPerRow == 1 ? (blockIdx.x * static_cast<long long>(kRowsPerCta) + warp) : static_cast<long long>(blockIdx.x);
  const int t = kWarpsPerRow == 1 ? lane : static_cast<int>(threadIdx.x);
  const bool row_ok = row < p.rows;  // warp-uniform; a CTA-wide row is always valid
  const int groups = p.cols >> 3;
  float red[4] = {0.f, 0.f, 0.f, 0.f};

  for (int pass = 0; pass <= p.n_red; ++pass) {
    const bool last = pass == p.n_red;
    const int end = last ? p.n_inst : p.red_pc[pass];
    const int kind = last ? 0 : p.prog[end].op;
    float partial = (kind == HB_EW_REDUCE_MAX) ? -INFINITY : 0.f;
    if (row_ok) {
      for (int g0 = t; g0 < groups; g0 += kThreadsPerRow * kG) {
        long long rows_[kG];
        int col[kG];
        bool ok[kG];
#pragma unroll
        for (int g = 0; g < kG; ++g) {
          const int gi = g0 + kThreadsPerRow * g;
          ok[g] = gi < groups;
          rows_[g] = row;
          col[g] = ok[g] ? gi << 3 : 0;
        }
        RowProgState s;
        s.tmp = tmp_s + threadIdx.x;
        rowprog_run<T>(p, end, rows_, col, ok, red, last, s);
        if (!last) {
#pragma unroll
          for (int g = 0; g < kG; ++g) {
            if (!ok[g]) continue;
#pragma unroll
            for (int e = 0; e < 8; ++e)
              partial = (kind == HB_EW_REDUCE_MAX) ? fmaxf(partial, s.acc[8 * g + e]) : partial + s.acc[8 * g + e];
          }
        }
      }
    }
    if (last) break;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, partial, o);
      partial = (kind == HB_EW_REDUCE_MAX) ? fmaxf(partial, other) : partial + other;
    }
    if constexpr (kWarpsPerRow > 1) {
      __syncthreads();  // the previous pass's readers are done with `part`
      if (lane == 0) part[warp] = partial;
      __syncthreads();
      partial = part[0];
#pragma unroll
      for (int w = 1; w < kWarpsPerRow; ++w) partial = (kind == HB_EW_REDUCE_MAX) ? fmaxf(partial, part[w]) : partial + part[w];
    }
    if (kind == HB_EW_REDUCE_MEAN) partial /= static_cast<float>(p.cols);
    const int slot = p.prog[end].index;
    red[0] = slot == 0 ? partial : red[0];
    red[1] = slot == 1 ? partial : red[1];
    red[2] = slot == 2 ? partial : red[2];
    red[3] = slot == 3 ? partial : red[3];
  }
}

static bool rp_aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

// Checks the arguments and the program and fills the kernel parameters; *n_tmp receives the number
// of temporaries the program uses.
static int rowprog_validate(const hb_rowwise_args* a, RowProgParams& p, int* n_tmp) {
  if (a == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: args is NULL");
  if (a->rows < 0 || a->cols <= 0) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: negative or zero extent");
  if (a->dtype != HB_BF16 && a->dtype != HB_FP16)
    return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: dtype %d not supported (bf16, fp16)", a->dtype);
  if (a->cols % 8 != 0) return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: cols must be a multiple of 8 (got %d)", a->cols);
  if (a->rows > 0x7fffffffLL || a->rows * (a->cols / 8) > 0xffffffffLL)
    return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: too many rows or elements (at most 2^31-1 rows and 2^35 elements)");
  if (a->n_inputs < 0 || a->n_inputs > HB_EW_MAX_INPUTS || a->n_rowvec < 0 || a->n_rowvec > HB_EW_MAX_ROWVEC ||
      a->n_rowscalar < 0 || a->n_rowscalar > HB_EW_MAX_ROWSCALAR || a->n_outputs < 1 || a->n_outputs > HB_EW_MAX_OUTPUTS)
    return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: operand counts out of range");
  if (a->mode < HB_ROWWISE_AUTO || a->mode > HB_ROWWISE_COMPILED)
    return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: unknown mode %d", a->mode);
  if (a->n_inst < 1 || a->n_inst > HB_EW_MAX_INST)
    return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: program length %d not in 1..%d", a->n_inst, HB_EW_MAX_INST);

  memset(&p, 0, sizeof(p));
  for (int i = 0; i < a->n_inputs; ++i) {
    if (a->inputs[i] == nullptr || !rp_aligned16(a->inputs[i]) || a->ld_in[i] < a->cols || a->ld_in[i] % 8 != 0)
      return set_error(HB_ERR_ALIGN, "hb_rowwise_program: input %d needs a non-NULL 16-byte aligned pointer and a row stride >= cols that is a multiple of 8", i);
    p.in[i] = a->inputs[i];
    p.ld_in[i] = a->ld_in[i];
  }
  for (int i = 0; i < a->n_rowvec; ++i) {
    if (a->rowvec[i] == nullptr || !rp_aligned16(a->rowvec[i]))
      return set_error(HB_ERR_ALIGN, "hb_rowwise_program: row vector %d needs a non-NULL 16-byte aligned pointer", i);
    p.rowvec[i] = a->rowvec[i];
  }
  for (int i = 0; i < a->n_rowscalar; ++i) {
    if (a->rowscalar[i] == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: per-row vector %d is NULL", i);
    p.rowscalar[i] = a->rowscalar[i];
  }
  for (int i = 0; i < a->n_outputs; ++i) {
    if (a->outputs[i] == nullptr || !rp_aligned16(a->outputs[i]) || a->ld_out[i] < a->cols || a->ld_out[i] % 8 != 0)
      return set_error(HB_ERR_ALIGN, "hb_rowwise_program: output %d needs a non-NULL 16-byte aligned pointer and a row stride >= cols that is a multiple of 8", i);
    p.out[i] = a->outputs[i];
    p.ld_out[i] = a->ld_out[i];
  }
  // program check: every index in range, values defined before use, at least one store
  bool acc_defined = false, tmp_defined[HB_EW_MAX_TMP] = {}, red_defined[HB_EW_MAX_RED] = {}, stored[HB_EW_MAX_OUTPUTS] = {};
  for (int pc = 0; pc < a->n_inst; ++pc) {
    const hb_ew_inst& in = a->program[pc];
    const bool binary = in.op >= HB_EW_LOAD && in.op <= HB_EW_POW;
    const bool unary = in.op >= HB_EW_NEG && in.op <= HB_EW_ROUND;
    const bool reduce = in.op >= HB_EW_REDUCE_SUM && in.op <= HB_EW_REDUCE_MEAN;
    if (!binary && !unary && !reduce && in.op != HB_EW_STORE_TMP && in.op != HB_EW_STORE_OUT)
      return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: instruction %d has unknown op %d", pc, in.op);
    if (binary) {
      int limit = 0;
      switch (in.src) {
        case HB_SRC_INPUT: limit = a->n_inputs; break;
        case HB_SRC_ROWVEC: limit = a->n_rowvec; break;
        case HB_SRC_ROWSCALAR: limit = a->n_rowscalar; break;
        case HB_SRC_TMP: limit = HB_EW_MAX_TMP; break;
        case HB_SRC_REDUCED: limit = HB_EW_MAX_RED; break;
        case HB_SRC_IMM: limit = 1; break;
        default:
          return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: instruction %d needs an operand", pc);
      }
      if (in.src != HB_SRC_IMM && (in.index < 0 || in.index >= limit))
        return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: instruction %d: operand index %d out of range", pc, in.index);
      if (in.src == HB_SRC_TMP && !tmp_defined[in.index])
        return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: instruction %d reads temporary %d before it is stored", pc, in.index);
      if (in.src == HB_SRC_REDUCED && !red_defined[in.index])
        return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: instruction %d reads reduction %d before it is computed", pc, in.index);
      if (in.op != HB_EW_LOAD && !acc_defined)
        return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: instruction %d uses the accumulator before a LOAD", pc);
      acc_defined = true;
    } else {
      if (!acc_defined) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: instruction %d uses the accumulator before a LOAD", pc);
      if (in.op == HB_EW_STORE_TMP) {
        if (in.index < 0 || in.index >= HB_EW_MAX_TMP) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: temporary index %d out of range", in.index);
        tmp_defined[in.index] = true;
      } else if (in.op == HB_EW_STORE_OUT) {
        if (in.index < 0 || in.index >= a->n_outputs) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: output index %d out of range", in.index);
        stored[in.index] = true;
      } else if (reduce) {
        if (in.index < 0 || in.index >= HB_EW_MAX_RED) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: reduction slot %d out of range", in.index);
        if (p.n_red >= HB_EW_MAX_RED) return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: more than %d reductions", HB_EW_MAX_RED);
        red_defined[in.index] = true;
        p.red_pc[p.n_red++] = pc;
      }
    }
    p.prog[pc] = in;
  }
  for (int i = 0; i < a->n_outputs; ++i)
    if (!stored[i]) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: output %d is never stored", i);
  p.rows = a->rows;
  p.cols = a->cols;
  p.n_inst = a->n_inst;
  *n_tmp = 0;
  for (int k = 0; k < HB_EW_MAX_TMP; ++k)
    if (tmp_defined[k]) *n_tmp = k + 1;
  return HB_OK;
}

static int rowprog_impl(const hb_rowwise_args* a) {
  RowProgParams p;
  int n_tmp = 0;
  const int vrc = rowprog_validate(a, p, &n_tmp);
  if (vrc != HB_OK) return vrc;
  if (a->rows == 0) return HB_OK;

  DeviceState* st = nullptr;
  const int rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  const bool bf16 = a->dtype == HB_BF16;
  if (a->mode != HB_ROWWISE_INTERPRET) {
    const int jit = rowprog_jit_launch(p, bf16, *st, stream);
    if (jit == kJitLaunched) return HB_OK;
    if (jit == kJitError) return HB_ERR_CUDA;  // the message is set
    if (a->mode == HB_ROWWISE_COMPILED)
      return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: the run-time compiler (libnvrtc) cannot be loaded in this process");
  }
  // dynamic shared memory: only the temporaries the program uses (16 KB each)
  const size_t smem = (size_t)n_tmp * kE * kRpThreads * sizeof(float);
  {
    static std::mutex mu;
    static bool configured[64] = {};
    std::lock_guard<std::mutex> lock(mu);
    if (!configured[st->device & 63]) {
      const int max_smem = HB_EW_MAX_TMP * kE * kRpThreads * (int)sizeof(float);
      HB_CUDA_CHECK(cudaFuncSetAttribute(rowprog_stream_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      HB_CUDA_CHECK(cudaFuncSetAttribute(rowprog_stream_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      HB_CUDA_CHECK(cudaFuncSetAttribute(rowprog_reduce_kernel<__nv_bfloat16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      HB_CUDA_CHECK(cudaFuncSetAttribute(rowprog_reduce_kernel<__half, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      HB_CUDA_CHECK(cudaFuncSetAttribute(rowprog_reduce_kernel<__nv_bfloat16, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      HB_CUDA_CHECK(cudaFuncSetAttribute(rowprog_reduce_kernel<__half, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      configured[st->device & 63] = true;
    }
  }
  if (p.n_red == 0) {
    const long long groups = a->rows * (a->cols / 8);
    const long long per_block = 1ll * kRpThreads * kG;
    const unsigned grid = static_cast<unsigned>(std::min<long long>((groups + per_block - 1) / per_block, 48ll * st->sm_count));
    if (bf16) rowprog_stream_kernel<__nv_bfloat16><<<grid, kRpThreads, smem, stream>>>(p);
    else rowprog_stream_kernel<__half><<<grid, kRpThreads, smem, stream>>>(p);
  } else if (a->cols <= 1024) {
    const unsigned grid = static_cast<unsigned>((a->rows + 3) / 4);
    if (bf16) rowprog_reduce_kernel<__nv_bfloat16, 1><<<grid, 128, smem, stream>>>(p);
    else rowprog_reduce_kernel<__half, 1><<<grid, 128, smem, stream>>>(p);
  } else {
    const unsigned grid = static_cast<unsigned>(a->rows);
    if (bf16) rowprog_reduce_kernel<__nv_bfloat16, 4><<<grid, 128, smem, stream>>>(p);
    else rowprog_reduce_kernel<__half, 4><<<grid, 128, smem, stream>>>(p);
  }
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

}  // namespace hb

extern "C" int hb_rowwise_compiler_available(void) { return hb::rowprog_jit_available(); }

extern "C" int hb_debug_rowwise_compile(const hb_rowwise_args* args, char* source, int64_t capacity) {
  hb::clear_error();
  hb::RowProgParams p;
  int n_tmp = 0;
  const int rc = hb::rowprog_validate(args, p, &n_tmp);
  if (rc != HB_OK) return rc;
  return hb::rowprog_jit_compile_only(p, args->dtype == HB_BF16, source, capacity);
}

extern "C" int hb_rowwise_program(const hb_rowwise_args* args) {
  hb::clear_error();
  return hb::rowprog_impl(args);
}
