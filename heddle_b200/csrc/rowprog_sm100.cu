// hb_rowwise_program: pointwise chains and row reductions over a [rows, cols] matrix, driven by a
// small op-code program instead of generated source.
//
// The reference emits TileLang source text for such partitions and compiles it at run time:
// pointwise chains (Heddle/heddle/frontend/codegen.py:1457-1498, op table _map_op :1577-1609) and
// softmax-like / sum / mean / max reductions over the last axis (:1246-1455: one pass per reduction
// that recomputes the expression up to it, results kept in fp32, then an output pass).  Here the
// FX lowering linearises the same partition into an accumulator-machine program that one
// precompiled kernel interprets: nothing is compiled at run time.
//
// Machine, per group of 8 consecutive columns of a row (16 bytes of a 16-bit tensor):
//   acc[8]           the running value (fp32)
//   tmp[4][8]        saved values (HB_EW_STORE_TMP)
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

#include <algorithm>
#include <cstring>

namespace hb {

struct alignas(16) RowProgParams {
  const void* in[HB_EW_MAX_INPUTS];
  long long ld_in[HB_EW_MAX_INPUTS];
  const void* rowvec[HB_EW_MAX_ROWVEC];
  const float* rowscalar[HB_EW_MAX_ROWSCALAR];
  void* out[HB_EW_MAX_OUTPUTS];
  long long ld_out[HB_EW_MAX_OUTPUTS];
  long long rows;
  int cols;
  int n_inst;
  int n_red;
  int red_pc[HB_EW_MAX_RED];  // position of the r-th reduction instruction
  hb_ew_inst prog[HB_EW_MAX_INST];
};

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

// Register state of the machine for one group of 8 columns.
struct RowProgState {
  float acc[8];
  float t0[8], t1[8], t2[8], t3[8];
};

// Executes instructions [0, end) for the 8 columns starting at `col` of `row`.  `red` holds the
// reductions of earlier passes; `store` is true in the last pass only.
template <typename T>
__device__ __forceinline__ void rowprog_run(const RowProgParams& p, int end, long long row, int col, const float (&red)[4],
                                            bool store, RowProgState& s) {
#pragma unroll 1
  for (int pc = 0; pc < end; ++pc) {
    const hb_ew_inst inst = p.prog[pc];
    float v[8];
    // ---- operand
    switch (inst.src) {
      case HB_SRC_INPUT:
        rp_unpack8<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(p.in[inst.index]) + row * p.ld_in[inst.index] + col), v);
        break;
      case HB_SRC_ROWVEC:
        rp_unpack8<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(p.rowvec[inst.index]) + col), v);
        break;
      case HB_SRC_ROWSCALAR: {
        const float x = p.rowscalar[inst.index][row];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = x;
        break;
      }
      case HB_SRC_TMP:
#pragma unroll
        for (int e = 0; e < 8; ++e)
          v[e] = inst.index == 0 ? s.t0[e] : inst.index == 1 ? s.t1[e] : inst.index == 2 ? s.t2[e] : s.t3[e];
        break;
      case HB_SRC_REDUCED: {
        const float x = inst.index == 0 ? red[0] : inst.index == 1 ? red[1] : inst.index == 2 ? red[2] : red[3];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = x;
        break;
      }
      default:  // HB_SRC_IMM, HB_SRC_NONE
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = inst.imm;
        break;
    }
    // ---- operation (formulas: Heddle/heddle/frontend/codegen.py:1577-1609)
    float (&a)[8] = s.acc;
    switch (inst.op) {
      case HB_EW_LOAD:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = v[e];
        break;
      case HB_EW_ADD:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] + v[e];
        break;
      case HB_EW_SUB:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] - v[e];
        break;
      case HB_EW_RSUB:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = v[e] - a[e];
        break;
      case HB_EW_MUL:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] * v[e];
        break;
      case HB_EW_DIV:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] / v[e];
        break;
      case HB_EW_RDIV:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = v[e] / a[e];
        break;
      case HB_EW_MAX:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = fmaxf(a[e], v[e]);
        break;
      case HB_EW_MIN:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = fminf(a[e], v[e]);
        break;
      case HB_EW_POW:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = powf(a[e], v[e]);
        break;
      case HB_EW_NEG:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = -a[e];
        break;
      case HB_EW_ABS:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = fabsf(a[e]);
        break;
      case HB_EW_EXP:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = expf(a[e]);
        break;
      case HB_EW_LOG:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = logf(a[e]);
        break;
      case HB_EW_LOG2:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = log2f(a[e]);
        break;
      case HB_EW_SQRT:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = sqrtf(a[e]);
        break;
      case HB_EW_RSQRT:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = 1.0f / sqrtf(a[e]);
        break;
      case HB_EW_RECIP:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = 1.0f / a[e];
        break;
      case HB_EW_SIGMOID:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = 1.0f / (1.0f + expf(-a[e]));
        break;
      case HB_EW_SILU:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] * (1.0f / (1.0f + expf(-a[e])));
        break;
      case HB_EW_RELU:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = fmaxf(a[e], 0.0f);
        break;
      case HB_EW_GELU_TANH:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] * 0.5f * (1.0f + tanhf(0.7978845608f * (a[e] + 0.044715f * a[e] * a[e] * a[e])));
        break;
      case HB_EW_GELU_ERF:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] * 0.5f * (1.0f + erff(a[e] * 0.7071067811865476f));
        break;
      case HB_EW_TANH:
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = tanhf(a[e]);
        break;
      case HB_EW_ROUND: {
        const uint4 w = rp_pack8<T>(a);
        rp_unpack8<T>(w, a);
        break;
      }
      case HB_EW_STORE_TMP:
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          if (inst.index == 0) s.t0[e] = a[e];
          else if (inst.index == 1) s.t1[e] = a[e];
          else if (inst.index == 2) s.t2[e] = a[e];
          else s.t3[e] = a[e];
        }
        break;
      case HB_EW_STORE_OUT:
        if (store)
          *reinterpret_cast<uint4*>(static_cast<T*>(p.out[inst.index]) + row * p.ld_out[inst.index] + col) = rp_pack8<T>(a);
        break;
      default:  // HB_EW_REDUCE_*: a no-op inside a pass (the pass that ends here reduces acc afterwards)
        break;
    }
  }
}

// No reductions: a flat stream over the 16-byte groups of the matrix.
template <typename T>
__global__ void __launch_bounds__(256) rowprog_stream_kernel(const __grid_constant__ RowProgParams p) {
  const int groups = p.cols >> 3;
  const long long total = p.rows * groups;
  const float red[4] = {0.f, 0.f, 0.f, 0.f};
  for (long long g = blockIdx.x * 256ll + threadIdx.x; g < total; g += 256ll * gridDim.x) {
    const long long row = g / groups;
    const int col = static_cast<int>(g - row * groups) << 3;
    RowProgState s;
    rowprog_run<T>(p, p.n_inst, row, col, red, true, s);
  }
}

// With reductions: kWarpsPerRow warps (1 or 4) own a row; 128-thread CTAs.
template <typename T, int kWarpsPerRow>
__global__ void __launch_bounds__(128) rowprog_reduce_kernel(const __grid_constant__ RowProgParams p) {
  constexpr int kThreadsPerRow = 32 * kWarpsPerRow;
  constexpr int kRowsPerCta = 4 / kWarpsPerRow;
  __shared__ float part[4];
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
      for (int g = t; g < groups; g += kThreadsPerRow) {
        RowProgState s;
        rowprog_run<T>(p, end, row, g << 3, red, last, s);
        if (!last) {
#pragma unroll
          for (int e = 0; e < 8; ++e) partial = (kind == HB_EW_REDUCE_MAX) ? fmaxf(partial, s.acc[e]) : partial + s.acc[e];
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

static int rowprog_impl(const hb_rowwise_args* a) {
  if (a == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: args is NULL");
  if (a->rows < 0 || a->cols <= 0) return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: negative or zero extent");
  if (a->dtype != HB_BF16 && a->dtype != HB_FP16)
    return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: dtype %d not supported (bf16, fp16)", a->dtype);
  if (a->cols % 8 != 0) return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: cols must be a multiple of 8 (got %d)", a->cols);
  if (a->rows > 0x7fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: too many rows");
  if (a->n_inputs < 0 || a->n_inputs > HB_EW_MAX_INPUTS || a->n_rowvec < 0 || a->n_rowvec > HB_EW_MAX_ROWVEC ||
      a->n_rowscalar < 0 || a->n_rowscalar > HB_EW_MAX_ROWSCALAR || a->n_outputs < 1 || a->n_outputs > HB_EW_MAX_OUTPUTS)
    return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: operand counts out of range");
  if (a->n_inst < 1 || a->n_inst > HB_EW_MAX_INST)
    return set_error(HB_ERR_BAD_ARG, "hb_rowwise_program: program length %d not in 1..%d", a->n_inst, HB_EW_MAX_INST);

  RowProgParams p;
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
  if (a->rows == 0) return HB_OK;
  p.rows = a->rows;
  p.cols = a->cols;
  p.n_inst = a->n_inst;

  DeviceState* st = nullptr;
  const int rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  const bool bf16 = a->dtype == HB_BF16;
  if (p.n_red == 0) {
    const long long groups = a->rows * (a->cols / 8);
    const unsigned grid = static_cast<unsigned>(std::min<long long>((groups + 255) / 256, 32ll * st->sm_count));
    if (bf16) rowprog_stream_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
    else rowprog_stream_kernel<__half><<<grid, 256, 0, stream>>>(p);
  } else if (a->cols <= 1024) {
    const unsigned grid = static_cast<unsigned>((a->rows + 3) / 4);
    if (bf16) rowprog_reduce_kernel<__nv_bfloat16, 1><<<grid, 128, 0, stream>>>(p);
    else rowprog_reduce_kernel<__half, 1><<<grid, 128, 0, stream>>>(p);
  } else {
    const unsigned grid = static_cast<unsigned>(a->rows);
    if (bf16) rowprog_reduce_kernel<__nv_bfloat16, 4><<<grid, 128, 0, stream>>>(p);
    else rowprog_reduce_kernel<__half, 4><<<grid, 128, 0, stream>>>(p);
  }
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

}  // namespace hb

extern "C" int hb_rowwise_program(const hb_rowwise_args* args) {
  hb::clear_error();
  return hb::rowprog_impl(args);
}
