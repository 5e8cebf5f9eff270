// Kernel parameters of hb_rowwise_program, shared by the interpreter kernels (rowprog_sm100.cu)
// and by the run-time specialised kernels (rowprog_jit.cu).
#pragma once

#include "host_common.h"

namespace hb {

// Operand pointers and extents: everything a specialised kernel needs (its program is in its code).
struct alignas(16) RowProgHead {
  const void* in[HB_EW_MAX_INPUTS];
  long long ld_in[HB_EW_MAX_INPUTS];
  const void* rowvec[HB_EW_MAX_ROWVEC];
  const float* rowscalar[HB_EW_MAX_ROWSCALAR];
  void* out[HB_EW_MAX_OUTPUTS];
  long long ld_out[HB_EW_MAX_OUTPUTS];
  long long rows;
  int cols;
};

struct alignas(16) RowProgParams : RowProgHead {
  int n_inst;
  int n_red;
  int red_pc[HB_EW_MAX_RED];  // position of the r-th reduction instruction
  hb_ew_inst prog[HB_EW_MAX_INST];
};

// Result of the specialised path: launched, not available on this machine (no run-time compiler:
// the caller falls back to the interpreter), or an error that hb_last_error() describes.
enum { kJitLaunched = 0, kJitUnavailable = 1, kJitError = 2 };
int rowprog_jit_launch(const RowProgParams& p, bool bf16, const DeviceState& st, cudaStream_t stream);
// Generates and compiles the specialised kernel without loading or launching it (no device needed);
// the generated source is copied to `source` (capacity bytes, NUL-terminated) when it is not NULL.
int rowprog_jit_compile_only(const RowProgParams& p, bool bf16, char* source, int64_t capacity);
// 1 when the run-time compiler can be loaded in this process, else 0 (no device needed).
int rowprog_jit_available();

}  // namespace hb
