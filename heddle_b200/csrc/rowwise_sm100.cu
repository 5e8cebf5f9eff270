// hb_row_softmax: y = softmax(scale * x) over the last dimension of a [rows, cols] matrix.
//
// The reference lowers softmax-like partitions (max, exp, sum, divide over the last axis) to a
// generated TileLang kernel with one 32-thread CTA per row, exp2 and a block-wise online merge
// (Heddle/heddle/frontend/codegen.py:1246-1400).  Here a row is read from HBM once, kept in
// registers in fp32, and written once: one warp per row up to 2048 columns, one
// 256-thread CTA per row up to 16384.  fp32 arithmetic, exp2 with log2(e) folded into the scale.
#include "host_common.h"
#include "ptx_sm100.cuh"

#include <algorithm>

namespace hb {

template <typename T>
__device__ __forceinline__ void rs_unpack8(const uint4& w, float (&f)[8]);
template <>
__device__ __forceinline__ void rs_unpack8<__nv_bfloat16>(const uint4& w, float (&f)[8]) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void rs_unpack8<__half>(const uint4& w, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 rs_pack8(const float (&f)[8]) {
  uint4 w;
  w.x = Pack2<T>::pack(f[0], f[1]);
  w.y = Pack2<T>::pack(f[2], f[3]);
  w.z = Pack2<T>::pack(f[4], f[5]);
  w.w = Pack2<T>::pack(f[6], f[7]);
  return w;
}

// kChunks 16-byte chunks per thread; kWarpsPerRow warps cooperate on a row (1 or 8).
template <typename T, int kChunks, int kWarpsPerRow>
__global__ void __launch_bounds__(256) row_softmax_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows,
                                                          int cols, long long ld_x, long long ld_y, float scale_log2) {
  constexpr int kThreadsPerRow = 32 * kWarpsPerRow;
  __shared__ float red[2][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = kWarpsPerRow == 1 ? (blockIdx.x * 8ll + warp) : static_cast<long long>(blockIdx.x);
  const int t = kWarpsPerRow == 1 ? lane : static_cast<int>(threadIdx.x);
  const bool row_ok = row < rows;
  float f[kChunks][8];  // the row's slice in fp32: scaled scores, then exponentials
  float mx = -INFINITY;
#pragma unroll
  for (int k = 0; k < kChunks; ++k) {
    const int c = (k * kThreadsPerRow + t) * 8;
    if (row_ok && c < cols) {
      rs_unpack8<T>(*reinterpret_cast<const uint4*>(x + row * ld_x + c), f[k]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        f[k][e] *= scale_log2;
        mx = fmaxf(mx, f[k][e]);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if constexpr (kWarpsPerRow > 1) {
    if (lane == 0) red[0][warp] = mx;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < kWarpsPerRow; ++w) mx = fmaxf(mx, red[0][w]);
  }
  const float ref = (mx == -INFINITY) ? 0.f : mx;  // a row of -inf stays finite arithmetic (and yields NaN like torch)
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < kChunks; ++k) {
    const int c = (k * kThreadsPerRow + t) * 8;
    if (row_ok && c < cols) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        f[k][e] = fast_exp2(f[k][e] - ref);
        sum += f[k][e];
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if constexpr (kWarpsPerRow > 1) {
    if (lane == 0) red[1][warp] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsPerRow; ++w) sum += red[1][w];
  }
  const float inv = 1.0f / sum;
#pragma unroll
  for (int k = 0; k < kChunks; ++k) {
    const int c = (k * kThreadsPerRow + t) * 8;
    if (row_ok && c < cols) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[k][e] *= inv;
      *reinterpret_cast<uint4*>(y + row * ld_y + c) = rs_pack8<T>(f[k]);
    }
  }
}

template <typename T>
static int launch_row_softmax(const T* x, T* y, long long rows, int cols, long long ld_x, long long ld_y, float scale_log2,
                              cudaStream_t stream) {
  const int chunks = (cols + 7) / 8;  // 16-byte chunks per row
  if (chunks <= 32 * 8) {
    const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
    if (chunks <= 32 * 2)
      row_softmax_kernel<T, 2, 1><<<grid, 256, 0, stream>>>(x, y, rows, cols, ld_x, ld_y, scale_log2);
    else if (chunks <= 32 * 4)
      row_softmax_kernel<T, 4, 1><<<grid, 256, 0, stream>>>(x, y, rows, cols, ld_x, ld_y, scale_log2);
    else
      row_softmax_kernel<T, 8, 1><<<grid, 256, 0, stream>>>(x, y, rows, cols, ld_x, ld_y, scale_log2);
  } else {
    const unsigned grid = static_cast<unsigned>(rows);
    if (chunks <= 256 * 2)
      row_softmax_kernel<T, 2, 8><<<grid, 256, 0, stream>>>(x, y, rows, cols, ld_x, ld_y, scale_log2);
    else if (chunks <= 256 * 4)
      row_softmax_kernel<T, 4, 8><<<grid, 256, 0, stream>>>(x, y, rows, cols, ld_x, ld_y, scale_log2);
    else
      row_softmax_kernel<T, 8, 8><<<grid, 256, 0, stream>>>(x, y, rows, cols, ld_x, ld_y, scale_log2);
  }
  HB_CUDA_CHECK(cudaGetLastError());
  return HB_OK;
}

}  // namespace hb

extern "C" int hb_row_softmax(const void* x, void* y, int64_t rows, int32_t cols, int64_t ld_x, int64_t ld_y, float scale,
                              int32_t dtype, void* stream) {
  using namespace hb;
  if (rows < 0 || cols <= 0) return set_error(HB_ERR_BAD_ARG, "hb_row_softmax: negative or zero extent");
  if (dtype != HB_BF16 && dtype != HB_FP16)
    return set_error(HB_ERR_UNSUPPORTED, "hb_row_softmax: dtype %d not supported (bf16, fp16)", dtype);
  if (cols % 8 != 0 || cols > 16384)
    return set_error(HB_ERR_UNSUPPORTED, "hb_row_softmax: cols must be a multiple of 8, at most 16384 (got %d)", cols);
  if (rows == 0) return HB_OK;
  if (rows > 0x7fffffffLL) return set_error(HB_ERR_UNSUPPORTED, "hb_row_softmax: too many rows");
  if (x == nullptr || y == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_row_softmax: x and y must be non-NULL");
  if (ld_x < cols || ld_y < cols || ld_x % 8 != 0 || ld_y % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(y) & 15) != 0)
    return set_error(HB_ERR_ALIGN, "hb_row_softmax: 16-byte alignment and row strides that are multiples of 8 are required");
  DeviceState* st = nullptr;
  const int rc = get_device_state(&st);
  if (rc != HB_OK) return rc;
  const float scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == HB_BF16)
    return launch_row_softmax<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rows, cols,
                                             ld_x, ld_y, scale_log2, s);
  return launch_row_softmax<__half>(static_cast<const __half*>(x), static_cast<__half*>(y), rows, cols, ld_x, ld_y, scale_log2, s);
}
