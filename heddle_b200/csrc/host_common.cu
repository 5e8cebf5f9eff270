// Error text, per-device state, driver entry point for TMA descriptors, and the
// small informational entry points of the C ABI.
#include "host_common.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace hb {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { g_err[0] = '\0'; }

const char* describe_status(uint32_t word) {
  static thread_local char buf[160];
  if (word == 0) {
    snprintf(buf, sizeof(buf), "status word 0 (no bounded wait gave up)");
  } else if ((word & 0xf00u) == 0x100u) {
    // role ids: attention forward 1..5, GEMM 0x21.., H2O 0x31.., attention backward 0x41.., probes 0x70
    const uint32_t role = word & 0xffu;
    const char* kernel = role < 0x20 ? "attention forward" : role < 0x30 ? "GEMM" : role < 0x40 ? "H2O score"
                         : role < 0x50 ? "attention backward" : "probe";
    static const char* const kFa[] = {"?", "softmax", "correction", "MMA issuer", "TMA producer", "drain"};
    static const char* const kOther[] = {"?", "TMA producer", "MMA issuer", "consumer", "drain"};
    const char* name = role < 6 ? kFa[role] : ((role & 0xfu) < 5 && role < 0x50) ? kOther[role & 0xfu] : "?";
    snprintf(buf, sizeof(buf),
             "status word 0x%x: a bounded wait of the %s kernel gave up (role 0x%x, %s); that launch's outputs are incomplete",
             word, kernel, role, name);
  } else if (word == 0x200u) {
    snprintf(buf, sizeof(buf), "status word 0x200: dynamic shared memory base was not 1024-byte aligned");
  } else {
    snprintf(buf, sizeof(buf), "status word 0x%x", word);
  }
  return buf;
}

static std::mutex g_mutex;
static constexpr int kMaxDevices = 64;
static DeviceState g_devices[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

int get_device_state(DeviceState** out) {
  int dev = -1;
  HB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return set_error(HB_ERR_CUDA, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_devices[dev];
  if (st.device != dev) {
    int major = 0, minor = 0;
    HB_CUDA_CHECK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    HB_CUDA_CHECK(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
    HB_CUDA_CHECK(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
    HB_CUDA_CHECK(cudaDeviceGetAttribute(&st.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    st.cc = major * 10 + minor;
    if (st.cc != 100) {
      return set_error(HB_ERR_UNSUPPORTED,
                       "device %d has compute capability %d.%d; this library is built for sm_100a only", dev, major,
                       minor);
    }
    HB_CUDA_CHECK(cudaMalloc(&st.status_word, sizeof(uint32_t)));
    HB_CUDA_CHECK(cudaMemset(st.status_word, 0, sizeof(uint32_t)));
    st.device = dev;
  }
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    HB_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr)
      return set_error(HB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = &st;
  return HB_OK;
}

int get_device_info_noalloc(DeviceInfo* out) {
  int dev = -1;
  HB_CUDA_CHECK(cudaGetDevice(&dev));
  int major = 0, minor = 0;
  HB_CUDA_CHECK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  HB_CUDA_CHECK(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
  HB_CUDA_CHECK(cudaDeviceGetAttribute(&out->sm_count, cudaDevAttrMultiProcessorCount, dev));
  HB_CUDA_CHECK(cudaDeviceGetAttribute(&out->smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  out->device = dev;
  out->cc = major * 10 + minor;
  if (out->cc != 100)
    return set_error(HB_ERR_UNSUPPORTED, "device %d has compute capability %d.%d; this library is built for sm_100a only",
                     dev, major, minor);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    HB_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr)
      return set_error(HB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  return HB_OK;
}

int encode_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  if (g_encode == nullptr) return set_error(HB_ERR_CUDA, "tensor-map encoder not initialised");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return set_error(HB_ERR_ALIGN, "tensor base %p is not 16-byte aligned", base);
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) {
    if ((strides_bytes[i] & 15u) != 0)
      return set_error(HB_ERR_ALIGN, "stride %llu bytes of dimension %d is not a multiple of 16",
                       (unsigned long long)strides_bytes[i], i + 1);
    gstr[i] = strides_bytes[i];
  }
  CUresult r = g_encode(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(HB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_version(void) { return HB_VERSION; }

const char* hb_last_error(void) { return hb::g_err; }

int hb_status_word(uint32_t* out) {
  hb::clear_error();
  if (out == nullptr) return hb::set_error(HB_ERR_BAD_ARG, "hb_status_word: out is NULL");
  hb::DeviceState* st = nullptr;
  int rc = hb::get_device_state(&st);
  if (rc != HB_OK) return rc;
  HB_CUDA_CHECK(cudaDeviceSynchronize());
  HB_CUDA_CHECK(cudaMemcpy(out, st->status_word, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (*out != 0) return hb::set_error(HB_ERR_TIMEOUT, "hb_status_word: %s", hb::describe_status(*out));
  return HB_OK;
}

int hb_shutdown(void) {
  std::lock_guard<std::mutex> lock(hb::g_mutex);
  int prev = -1;
  cudaGetDevice(&prev);
  for (int d = 0; d < hb::kMaxDevices; ++d) {
    hb::DeviceState& st = hb::g_devices[d];
    if (st.device == d && st.status_word != nullptr) {
      cudaSetDevice(d);
      cudaFree(st.status_word);
    }
    st = hb::DeviceState();
  }
  if (prev >= 0) cudaSetDevice(prev);
  return HB_OK;
}

}  // extern "C"
