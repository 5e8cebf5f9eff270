// hb_debug_wait_timeout: exercises the bounded-wait / abort path of the kernels without a
// fault or a hang.  One CTA: warp 0 waits on an mbarrier that nothing ever arrives on, with a short
// limit; when the limit runs out it raises the CTA's abort flag and records a status code, exactly
// as a role of the attention or GEMM kernels would.  Warp 1 waits on a second barrier with a long
// limit and must leave as soon as it sees the flag.  The kernel then ends normally; the status goes
// to a scratch word of its own, so the device status word of the library stays untouched.
#include "host_common.h"
#include "ptx_sm100.cuh"

namespace hb {

static __device__ uint32_t g_probe_status;

__global__ void __launch_bounds__(64) wait_timeout_probe_kernel(uint64_t limit_ns, uint32_t* status, unsigned long long* out) {
  __shared__ uint64_t bar[2];
  __shared__ uint32_t abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    fence_mbar_init();
  }
  __syncthreads();
  AbortCtx ctx{&abort_flag, status, warp == 0 ? limit_ns : limit_ns * 1000ull};
  const uint64_t t0 = global_timer_ns();
  const bool ok = mbar_wait_warp(&bar[warp], 0, ctx, 0x70u + static_cast<uint32_t>(warp));
  const uint64_t t1 = global_timer_ns();
  if (lane == 0) {
    out[warp * 2] = ok ? 1ull : 0ull;
    out[warp * 2 + 1] = t1 - t0;
  }
}

}  // namespace hb

extern "C" int hb_debug_wait_timeout(uint32_t limit_us, uint32_t* status_out, uint64_t* result4) {
  using namespace hb;
  if (status_out == nullptr || result4 == nullptr) return set_error(HB_ERR_BAD_ARG, "hb_debug_wait_timeout: NULL output");
  if (limit_us == 0 || limit_us > 100000) return set_error(HB_ERR_BAD_ARG, "hb_debug_wait_timeout: limit must be 1..100000 us");
  uint32_t* d_status = nullptr;
  HB_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&d_status), g_probe_status));
  HB_CUDA_CHECK(cudaMemset(d_status, 0, sizeof(uint32_t)));
  unsigned long long* d_out = nullptr;
  HB_CUDA_CHECK(cudaMalloc(&d_out, 4 * sizeof(unsigned long long)));
  wait_timeout_probe_kernel<<<1, 64>>>(static_cast<uint64_t>(limit_us) * 1000ull, d_status, d_out);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(status_out, d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(result4, d_out, 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  cudaFree(d_out);
  if (e != cudaSuccess) return set_error(HB_ERR_CUDA, "hb_debug_wait_timeout: %s", cudaGetErrorString(e));
  return HB_OK;
}
