// Run-time specialisation of hb_rowwise_program: the op-code program is turned into straight-line
// CUDA source, compiled for sm_100a with NVRTC, and cached per (device, dtype, program).
//
// The reference compiles every fused pointwise / reduction partition at run time as well
// (Heddle/heddle/frontend/codegen.py:1457-1498 for pointwise chains, :1246-1455 for row
// reductions, compiled through tilelang.compile).  The interpreter in rowprog_sm100.cu spends most
// of its issue slots on decode and operand moves; with the program known at compile time the
// compiler hoists all loads of a group to the top (every input's 16-byte loads are in flight
// together), keeps temporaries in registers and emits only the program's own arithmetic, which puts
// a pointwise chain on the HBM roofline.
//
// NVRTC is loaded with dlopen on first use; on a machine without it the caller falls back to the
// interpreter kernels (same results: both use the same formulas).  The generated kernels follow the
// interpreter's structure one to one:
//   * no reductions: a grid-stride stream over groups of 8 columns, kG groups per thread;
//   * reductions: one row per warp (cols <= 1024) or per 128-thread CTA, R + 1 passes, pass r runs
//     the program up to the r-th reduction and reduces the accumulator over the row.
#include "rowprog_sm100.cuh"

#include <dlfcn.h>
#include <nvrtc.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace hb {
namespace {

// ---- NVRTC through dlopen ---------------------------------------------------------------------
struct Nvrtc {
  void* handle = nullptr;
  nvrtcResult (*create)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  nvrtcResult (*compile)(nvrtcProgram, int, const char* const*) = nullptr;
  nvrtcResult (*cubin_size)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*cubin)(nvrtcProgram, char*) = nullptr;
  nvrtcResult (*log_size)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*log)(nvrtcProgram, char*) = nullptr;
  nvrtcResult (*destroy)(nvrtcProgram*) = nullptr;
  bool tried = false;
  bool ok = false;
};
Nvrtc g_nvrtc;
std::mutex g_jit_mutex;

template <typename F>
bool bind(void* h, const char* name, F* out) {
  *out = reinterpret_cast<F>(dlsym(h, name));
  return *out != nullptr;
}

// Callers hold g_jit_mutex.
bool load_nvrtc() {
  if (g_nvrtc.tried) return g_nvrtc.ok;
  g_nvrtc.tried = true;
  const char* off = getenv("HEDDLE_B200_ROWWISE_JIT");
  if (off != nullptr && strcmp(off, "0") == 0) return false;
  std::vector<std::string> names;
  if (const char* user = getenv("HEDDLE_B200_NVRTC")) names.push_back(user);
  names.push_back("libnvrtc.so.12");
  names.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
  names.push_back("libnvrtc.so");
  for (const std::string& n : names) {
    g_nvrtc.handle = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (g_nvrtc.handle != nullptr) break;
  }
  if (g_nvrtc.handle == nullptr) return false;
  void* h = g_nvrtc.handle;
  g_nvrtc.ok = bind(h, "nvrtcCreateProgram", &g_nvrtc.create) && bind(h, "nvrtcCompileProgram", &g_nvrtc.compile) &&
               bind(h, "nvrtcGetCUBINSize", &g_nvrtc.cubin_size) && bind(h, "nvrtcGetCUBIN", &g_nvrtc.cubin) &&
               bind(h, "nvrtcGetProgramLogSize", &g_nvrtc.log_size) && bind(h, "nvrtcGetProgramLog", &g_nvrtc.log) &&
               bind(h, "nvrtcDestroyProgram", &g_nvrtc.destroy);
  return g_nvrtc.ok;
}

// ---- driver entry points (module load and launch) -----------------------------------------------
struct Driver {
  CUresult (*module_load)(CUmodule*, const void*) = nullptr;
  CUresult (*get_function)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*launch)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
  bool ok = false;
};
Driver g_driver;

int load_driver() {
  if (g_driver.ok) return HB_OK;
  struct {
    const char* name;
    void** slot;
  } wanted[] = {{"cuModuleLoadData", reinterpret_cast<void**>(&g_driver.module_load)},
                {"cuModuleGetFunction", reinterpret_cast<void**>(&g_driver.get_function)},
                {"cuLaunchKernel", reinterpret_cast<void**>(&g_driver.launch)}};
  for (auto& w : wanted) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    HB_CUDA_CHECK(cudaGetDriverEntryPoint(w.name, &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return set_error(HB_ERR_CUDA, "%s is not available from this driver", w.name);
    *w.slot = fn;
  }
  g_driver.ok = true;
  return HB_OK;
}

// ---- source generation --------------------------------------------------------------------------
constexpr int kJitG = 2;         // groups of 8 columns per thread and iteration
constexpr int kJitThreads = 128;

// Helpers and kernels that do not depend on the program.  HB_T_BF16 (0/1), HB_NRED, HB_WARPS_PER_ROW
// and the function rp_body() are put in front of / between these pieces by generate().
const char* kPrelude = R"SRC(
typedef unsigned int u32;
struct __align__(16) Head {
  const void* in[6]; long long ld_in[6]; const void* rowvec[4]; const float* rowscalar[4];
  void* out[2]; long long ld_out[2]; long long rows; int cols;
};
static_assert(sizeof(Head) == 208, "must match the host's RowProgHead");
constexpr int G = HB_G;
constexpr int E = 8 * G;
constexpr int THREADS = 128;

__device__ __forceinline__ void unpack8(const uint4& w, float* f) {
  const u32 u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#if HB_T_BF16
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
#else
    asm("{.reg .b16 l, h; mov.b32 {l, h}, %2; cvt.f32.f16 %0, l; cvt.f32.f16 %1, h;}" : "=f"(f[2 * i]), "=f"(f[2 * i + 1]) : "r"(u[i]));
#endif
  }
}
__device__ __forceinline__ u32 pack2(float lo, float hi) {
  u32 r;
#if HB_T_BF16
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
#else
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
#endif
  return r;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 w;
  w.x = pack2(f[0], f[1]); w.y = pack2(f[2], f[3]); w.z = pack2(f[4], f[5]); w.w = pack2(f[6], f[7]);
  return w;
}
__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float lg2(float x) { float y; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcp(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float f_exp(float x) { return ex2(x * 1.4426950408889634f); }
__device__ __forceinline__ float f_sigmoid(float x) { return rcp(1.0f + ex2(x * -1.4426950408889634f)); }
__device__ __forceinline__ float f_tanh(float x) { return fmaf(-2.0f, rcp(1.0f + ex2(x * 2.8853900817779268f)), 1.0f); }

__device__ __forceinline__ void ld_in(const void* base, long long ld, const long long* row, const int* col, const bool* ok, float* v) {
  uint4 w[G];
#pragma unroll
  for (int g = 0; g < G; ++g)
    w[g] = ok[g] ? *reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(base) + row[g] * ld + col[g]) : make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int g = 0; g < G; ++g) unpack8(w[g], v + 8 * g);
}
__device__ __forceinline__ void ld_rowvec(const void* base, const int* col, const bool* ok, float* v) {
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 w = ok[g] ? *reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(base) + col[g]) : make_uint4(0, 0, 0, 0);
    unpack8(w, v + 8 * g);
  }
}
__device__ __forceinline__ void ld_rowscalar(const float* base, const long long* row, const bool* ok, float* v) {
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float x = ok[g] ? base[row[g]] : 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) v[8 * g + e] = x;
  }
}
__device__ __forceinline__ void st_out(void* base, long long ld, const long long* row, const int* col, const bool* ok, const float* a) {
#pragma unroll
  for (int g = 0; g < G; ++g)
    if (ok[g]) *reinterpret_cast<uint4*>(static_cast<unsigned short*>(base) + row[g] * ld + col[g]) = pack8(a + 8 * g);
}
__device__ __forceinline__ void round16(float* a) {
#pragma unroll
  for (int g = 0; g < G; ++g) { const uint4 w = pack8(a + 8 * g); unpack8(w, a + 8 * g); }
}
#define EACH(expr) _Pragma("unroll") for (int e = 0; e < E; ++e) { a[e] = (expr); }
)SRC";

const char* kStreamKernel = R"SRC(
extern "C" __global__ void __launch_bounds__(THREADS) rowprog_jit(const __grid_constant__ Head p) {
  const unsigned groups = static_cast<unsigned>(p.cols >> 3);
  const unsigned total = static_cast<unsigned>(p.rows) * groups;
  const float red[4] = {0.f, 0.f, 0.f, 0.f};
  const unsigned stride = THREADS * G * gridDim.x;
  for (unsigned g0 = blockIdx.x * (THREADS * G) + threadIdx.x; g0 < total; g0 += stride) {
    long long row[G]; int col[G]; bool ok[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const unsigned idx = g0 + THREADS * g;
      ok[g] = idx < total && idx >= g0;
      const unsigned r = ok[g] ? idx / groups : 0u;
      row[g] = r;
      col[g] = ok[g] ? static_cast<int>(idx - r * groups) << 3 : 0;
    }
    float a[E];
    rp_body(p, 0, row, col, ok, red, a);
    if (g0 + stride < g0) break;  // the next index would wrap 32 bits: this was the last batch
  }
}
)SRC";

const char* kReduceKernel = R"SRC(
extern "C" __global__ void __launch_bounds__(THREADS) rowprog_jit(const __grid_constant__ Head p) {
  constexpr int W = HB_WARPS_PER_ROW;
  constexpr int TPR = 32 * W;
  __shared__ float part[4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = W == 1 ? (blockIdx.x * 4ll + warp) : static_cast<long long>(blockIdx.x);
  const int t = W == 1 ? lane : static_cast<int>(threadIdx.x);
  const bool row_ok = row < p.rows;
  const int groups = p.cols >> 3;
  float red[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int pass = 0; pass <= HB_NRED; ++pass) {
    const bool last = pass == HB_NRED;
    const int kind = last ? 0 : RED_KIND(pass);
    float partial = (kind == 1) ? __int_as_float(0xff800000) : 0.f;
    if (row_ok) {
      for (int g0 = t; g0 < groups; g0 += TPR * G) {
        long long rows_[G]; int col[G]; bool ok[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int gi = g0 + TPR * g;
          ok[g] = gi < groups;
          rows_[g] = row;
          col[g] = ok[g] ? gi << 3 : 0;
        }
        float a[E];
        rp_body(p, pass, rows_, col, ok, red, a);
        if (!last) {
#pragma unroll
          for (int g = 0; g < G; ++g) {
            if (!ok[g]) continue;
#pragma unroll
            for (int e = 0; e < 8; ++e) partial = (kind == 1) ? fmaxf(partial, a[8 * g + e]) : partial + a[8 * g + e];
          }
        }
      }
    }
    if (last) break;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, partial, o);
      partial = (kind == 1) ? fmaxf(partial, other) : partial + other;
    }
    if (W > 1) {
      __syncthreads();
      if (lane == 0) part[warp] = partial;
      __syncthreads();
      partial = part[0];
#pragma unroll
      for (int w = 1; w < W; ++w) partial = (kind == 1) ? fmaxf(partial, part[w]) : partial + part[w];
    }
    if (kind == 2) partial /= static_cast<float>(p.cols);
    const int slot = RED_SLOT(pass);
    red[0] = slot == 0 ? partial : red[0];
    red[1] = slot == 1 ? partial : red[1];
    red[2] = slot == 2 ? partial : red[2];
    red[3] = slot == 3 ? partial : red[3];
  }
}
)SRC";

std::string fmt_float(float x) {
  // exact round trip through the bit pattern (also covers inf / nan immediates)
  uint32_t bits;
  memcpy(&bits, &x, 4);
  char buf[48];
  snprintf(buf, sizeof(buf), "__uint_as_float(0x%08xu)", bits);
  return buf;
}

// One line of rp_body per instruction; the formulas are those of the interpreter's op switch.
std::string generate(const RowProgParams& p, bool bf16, int warps_per_row) {
  std::string s;
  char line[256];
  snprintf(line, sizeof(line), "#define HB_T_BF16 %d\n#define HB_G %d\n#define HB_NRED %d\n#define HB_WARPS_PER_ROW %d\n", bf16 ? 1 : 0, kJitG,
           p.n_red, warps_per_row);
  s += line;
  s += kPrelude;
  if (p.n_red > 0) {
    // kind: 0 sum, 1 max, 2 mean
    std::string kinds = "#define RED_KIND(pass) (", slots = "#define RED_SLOT(pass) (";
    for (int r = 0; r < p.n_red; ++r) {
      const int op = p.prog[p.red_pc[r]].op;
      const std::string sel = "(pass) == " + std::to_string(r) + " ? ";
      kinds += sel + std::to_string(op == HB_EW_REDUCE_MAX ? 1 : op == HB_EW_REDUCE_MEAN ? 2 : 0) + " : ";
      slots += sel + std::to_string(p.prog[p.red_pc[r]].index) + " : ";
    }
    s += kinds + "0)\n" + slots + "0)\n";
  }
  s += "__device__ __forceinline__ void rp_body(const Head& p, int pass, const long long* row, const int* col, const bool* ok,\n"
       "                                        const float* red, float* a) {\n  float v[E];\n";
  bool tmp_used[HB_EW_MAX_TMP] = {};
  for (int pc = 0; pc < p.n_inst; ++pc)
    if (p.prog[pc].op == HB_EW_STORE_TMP) tmp_used[p.prog[pc].index] = true;
  for (int k = 0; k < HB_EW_MAX_TMP; ++k)
    if (tmp_used[k]) s += "  float t" + std::to_string(k) + "[E];\n";
  int reductions_seen = 0;
  for (int pc = 0; pc < p.n_inst; ++pc) {
    const hb_ew_inst& in = p.prog[pc];
    const std::string idx = std::to_string(in.index);
    const bool binary = in.op >= HB_EW_LOAD && in.op <= HB_EW_POW;
    if (binary) {
      switch (in.src) {
        case HB_SRC_INPUT: s += "  ld_in(p.in[" + idx + "], p.ld_in[" + idx + "], row, col, ok, v);\n"; break;
        case HB_SRC_ROWVEC: s += "  ld_rowvec(p.rowvec[" + idx + "], col, ok, v);\n"; break;
        case HB_SRC_ROWSCALAR: s += "  ld_rowscalar(p.rowscalar[" + idx + "], row, ok, v);\n"; break;
        case HB_SRC_TMP: s += "  _Pragma(\"unroll\") for (int e = 0; e < E; ++e) v[e] = t" + idx + "[e];\n"; break;
        case HB_SRC_REDUCED: s += "  _Pragma(\"unroll\") for (int e = 0; e < E; ++e) v[e] = red[" + idx + "];\n"; break;
        default: s += "  _Pragma(\"unroll\") for (int e = 0; e < E; ++e) v[e] = " + fmt_float(in.imm) + ";\n"; break;
      }
    }
    const char* expr = nullptr;
    switch (in.op) {
      case HB_EW_LOAD: expr = "v[e]"; break;
      case HB_EW_ADD: expr = "a[e] + v[e]"; break;
      case HB_EW_SUB: expr = "a[e] - v[e]"; break;
      case HB_EW_RSUB: expr = "v[e] - a[e]"; break;
      case HB_EW_MUL: expr = "a[e] * v[e]"; break;
      case HB_EW_DIV: expr = "a[e] * rcp(v[e])"; break;
      case HB_EW_RDIV: expr = "v[e] * rcp(a[e])"; break;
      case HB_EW_MAX: expr = "fmaxf(a[e], v[e])"; break;
      case HB_EW_MIN: expr = "fminf(a[e], v[e])"; break;
      case HB_EW_POW: expr = "powf(a[e], v[e])"; break;
      case HB_EW_NEG: expr = "-a[e]"; break;
      case HB_EW_ABS: expr = "fabsf(a[e])"; break;
      case HB_EW_EXP: expr = "f_exp(a[e])"; break;
      case HB_EW_LOG: expr = "lg2(a[e]) * 0.6931471805599453f"; break;
      case HB_EW_LOG2: expr = "lg2(a[e])"; break;
      case HB_EW_SQRT: expr = "sqrtf(a[e])"; break;
      case HB_EW_RSQRT: expr = "rsqrtf(a[e])"; break;
      case HB_EW_RECIP: expr = "rcp(a[e])"; break;
      case HB_EW_SIGMOID: expr = "f_sigmoid(a[e])"; break;
      case HB_EW_SILU: expr = "a[e] * f_sigmoid(a[e])"; break;
      case HB_EW_RELU: expr = "fmaxf(a[e], 0.0f)"; break;
      case HB_EW_GELU_TANH: expr = "a[e] * 0.5f * (1.0f + f_tanh(0.7978845608f * (a[e] + 0.044715f * a[e] * a[e] * a[e])))"; break;
      case HB_EW_GELU_ERF: expr = "a[e] * 0.5f * (1.0f + erff(a[e] * 0.7071067811865476f))"; break;
      case HB_EW_TANH: expr = "f_tanh(a[e])"; break;
      default: break;
    }
    if (expr != nullptr) {
      s += std::string("  EACH(") + expr + ")\n";
    } else if (in.op == HB_EW_ROUND) {
      s += "  round16(a);\n";
    } else if (in.op == HB_EW_STORE_TMP) {
      s += "  _Pragma(\"unroll\") for (int e = 0; e < E; ++e) t" + idx + "[e] = a[e];\n";
    } else if (in.op == HB_EW_STORE_OUT) {
      s += "  if (pass == HB_NRED) st_out(p.out[" + idx + "], p.ld_out[" + idx + "], row, col, ok, a);\n";
    } else {  // a reduction: the pass that ends here returns with the accumulator to reduce
      s += "  if (pass == " + std::to_string(reductions_seen) + ") return;\n";
      ++reductions_seen;
    }
  }
  s += "}\n";
  s += p.n_red > 0 ? kReduceKernel : kStreamKernel;
  return s;
}

// ---- cache ------------------------------------------------------------------------------------
std::map<std::string, CUfunction> g_cache;

// Compiles `src` to device code for sm_100a.  Callers hold g_jit_mutex and have loaded NVRTC.
int compile_image(const std::string& src, std::vector<char>* image) {
  nvrtcProgram prog = nullptr;
  if (g_nvrtc.create(&prog, src.c_str(), "rowprog_jit.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
    return set_error(HB_ERR_CUDA, "hb_rowwise_program: nvrtcCreateProgram failed");
  const char* opts[] = {"--gpu-architecture=sm_100a", "-std=c++17", "-lineinfo"};
  const nvrtcResult rc = g_nvrtc.compile(prog, 3, opts);
  if (rc != NVRTC_SUCCESS) {
    size_t n = 0;
    g_nvrtc.log_size(prog, &n);
    std::string log(n + 1, '\0');
    if (n > 0) g_nvrtc.log(prog, &log[0]);
    g_nvrtc.destroy(&prog);
    return set_error(HB_ERR_CUDA, "hb_rowwise_program: run-time compilation failed (%d): %.600s", (int)rc, log.c_str());
  }
  size_t n = 0;
  if (g_nvrtc.cubin_size(prog, &n) != NVRTC_SUCCESS || n == 0) {
    g_nvrtc.destroy(&prog);
    return set_error(HB_ERR_CUDA, "hb_rowwise_program: the run-time compiler produced no device code");
  }
  image->resize(n);
  g_nvrtc.cubin(prog, image->data());
  g_nvrtc.destroy(&prog);
  return HB_OK;
}

int compile(const std::string& src, CUfunction* out) {
  std::vector<char> image;
  const int rc = compile_image(src, &image);
  if (rc != HB_OK) return rc;
  CUmodule mod = nullptr;  // kept for the life of the process (the cache owns the function)
  CUresult cr = g_driver.module_load(&mod, image.data());
  if (cr != CUDA_SUCCESS) return set_error(HB_ERR_CUDA, "hb_rowwise_program: cuModuleLoadData failed (%d)", (int)cr);
  cr = g_driver.get_function(out, mod, "rowprog_jit");
  if (cr != CUDA_SUCCESS) return set_error(HB_ERR_CUDA, "hb_rowwise_program: cuModuleGetFunction failed (%d)", (int)cr);
  return HB_OK;
}

}  // namespace

int rowprog_jit_available() {
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  return load_nvrtc() ? 1 : 0;
}

int rowprog_jit_compile_only(const RowProgParams& p, bool bf16, char* source, int64_t capacity) {
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  if (!load_nvrtc()) return set_error(HB_ERR_UNSUPPORTED, "hb_rowwise_program: the run-time compiler (libnvrtc) cannot be loaded in this process");
  const std::string src = generate(p, bf16, p.n_red == 0 ? 0 : (p.cols <= 1024 ? 1 : 4));
  if (source != nullptr && capacity > 0) {
    const size_t n = std::min<size_t>(src.size(), static_cast<size_t>(capacity) - 1);
    memcpy(source, src.data(), n);
    source[n] = '\0';
  }
  std::vector<char> image;
  return compile_image(src, &image);
}

int rowprog_jit_launch(const RowProgParams& p, bool bf16, const DeviceState& st, cudaStream_t stream) {
  static_assert(sizeof(RowProgHead) == 208, "the generated source restates this struct");
  const int warps_per_row = p.n_red == 0 ? 0 : (p.cols <= 1024 ? 1 : 4);
  CUfunction fn = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_jit_mutex);
    if (!load_nvrtc()) return kJitUnavailable;
    if (load_driver() != HB_OK) return kJitError;
    std::string key(reinterpret_cast<const char*>(p.prog), sizeof(hb_ew_inst) * p.n_inst);
    key += static_cast<char>(bf16 ? 1 : 0);
    key += static_cast<char>(warps_per_row);
    key += static_cast<char>(st.device);
    auto it = g_cache.find(key);
    if (it == g_cache.end()) {
      // the primary context of the current device must be current for the module load
      if (cudaFree(nullptr) != cudaSuccess) {
        set_error(HB_ERR_CUDA, "hb_rowwise_program: no CUDA context");
        return kJitError;
      }
      if (compile(generate(p, bf16, warps_per_row), &fn) != HB_OK) return kJitError;
      g_cache.emplace(std::move(key), fn);
    } else {
      fn = it->second;
    }
  }
  unsigned grid;
  if (p.n_red == 0) {
    const long long groups = p.rows * (p.cols / 8);
    const long long per_block = 1ll * kJitThreads * kJitG;
    grid = static_cast<unsigned>(std::min<long long>((groups + per_block - 1) / per_block, 64ll * st.sm_count));
  } else if (warps_per_row == 1) {
    grid = static_cast<unsigned>((p.rows + 3) / 4);
  } else {
    grid = static_cast<unsigned>(p.rows);
  }
  RowProgHead head = p;
  void* params[] = {&head};
  const CUresult cr = g_driver.launch(fn, grid, 1, 1, kJitThreads, 1, 1, 0, stream, params, nullptr);
  if (cr != CUDA_SUCCESS) {
    set_error(HB_ERR_CUDA, "hb_rowwise_program: cuLaunchKernel failed (%d)", (int)cr);
    return kJitError;
  }
  return kJitLaunched;
}

}  // namespace hb
