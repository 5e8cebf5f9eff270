// Host-side plumbing shared by the C-ABI entry points: thread-local error text,
// per-device state (status word), and TMA descriptor encoding through the driver
// entry point (fetched at run time, so the library has no link-time dependency on
// libcuda and loads on a machine without a GPU driver).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/heddle_b200.h"

namespace hb {

int set_error(int code, const char* fmt, ...);
void clear_error();

// Human-readable form of a device status word (0x100 | role: a bounded wait of that role ran out;
// 0x200: shared memory base misaligned).  Returns a pointer to a thread-local buffer.
const char* describe_status(uint32_t word);

#define HB_CUDA_CHECK(expr)                                                                   \
  do {                                                                                        \
    cudaError_t err__ = (expr);                                                               \
    if (err__ != cudaSuccess)                                                                 \
      return hb::set_error(HB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));   \
  } while (0)

struct DeviceState {
  int device = -1;
  int sm_count = 0;
  int smem_optin = 0;
  int cc = 0;
  uint32_t* status_word = nullptr;  // device memory, zero-initialised
};

// Lazily created state of the CURRENT device (mutex-guarded).  Returns an hb_status.
int get_device_state(DeviceState** out);

// Device facts for entry points that must not allocate: attribute queries and the
// driver entry point only (no cudaMalloc, no per-device state is created).
struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int smem_optin = 0;
  int cc = 0;
};
int get_device_info_noalloc(DeviceInfo* out);

// 2-D .. 4-D tiled tensor map with 128-byte swizzle, zero fill out of bounds.
//   dims[i]     extent of dimension i in elements (dimension 0 is contiguous)
//   strides[i]  byte stride of dimension i+1
//   box[i]      tile extent of dimension i in elements
int encode_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);

inline size_t dtype_size(int dtype) { return dtype == HB_FP8_E4M3 ? 1 : 2; }

}  // namespace hb
