// Shared device/host helpers for the policy-forward kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/bsrl.h"

namespace bsrl {

constexpr int kT = BSRL_N_TOKENS;      // 29 tokens per env
constexpr int kLead = BSRL_N_LEAD;     // 5 lead tokens
constexpr int kSlots = BSRL_N_SLOTS;   // 24 entity slots
constexpr int kObs = BSRL_OBS_DIM;     // 630 obs lanes
constexpr int kActHeads = BSRL_N_ACT_HEADS;
constexpr float kMaskBias = 16384.0f;  // additive key mask magnitude
constexpr float kMaskedLogit = -1e9f;  // fill of lanes past a head's gear count

// Quotient and remainder of a row or element index (0 <= i) by a small positive divisor.  64-bit integer
// division is a long software routine on the GPU (~150 cycles per call where a thread needs it before it can do
// anything else); indices that fit 32 bits -- all of them at the sizes these kernels see -- take the 32-bit
// unsigned division instead.
__host__ __device__ __forceinline__ int64_t div_index(int64_t i, int d, int* rem) {
  if (!((uint64_t)i >> 32)) {
    const uint32_t q = (uint32_t)i / (uint32_t)d;
    *rem = (int)((uint32_t)i - q * (uint32_t)d);
    return (int64_t)q;
  }
  *rem = (int)(i % d);
  return i / d;
}

// Row remapping of a (rows, ld) matrix: logical row r lives at physical row
// (r / group) * stride + first + (r % group).  Identity: group = INT_MAX, stride = 0, first = 0.
struct RowMap {
  int group;
  int stride;
  int first;
  __host__ __device__ inline int64_t operator()(int64_t r) const {
    if (r < (int64_t)group) return (int64_t)first + r;      // identity maps and every first group: no division
    int rem;
    const int64_t q = div_index(r, group, &rem);
    return q * (int64_t)stride + first + rem;
  }
  // the same map as the plain formula, for cold paths of kernels whose code generation should not move
  __host__ __device__ inline int64_t plain(int64_t r) const {
    return (r / group) * (int64_t)stride + first + (r % group);
  }
};
inline RowMap identity_map() { return RowMap{0x7fffffff, 0, 0}; }

// thread-local error message (host)
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define BSRL_CUDA_OK(expr)                                   \
  do {                                                       \
    cudaError_t e__ = (expr);                                \
    if (e__ != cudaSuccess) return ::bsrl::cuda_fail(e__, #expr); \
  } while (0)

#define BSRL_LAUNCH_OK(what)                                 \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return ::bsrl::cuda_fail(e__, what); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

int sm_count();  // multiprocessors of the current device (cached per device)

// One-time set-up per device (raising a kernel's dynamic shared-memory limit, resolving a device
// symbol): run(what, fn) calls fn() -> cudaError_t once for the CURRENT device, whichever host
// thread gets there first, and returns BSRL_OK or the failure of that first run.  The cached result
// belongs to the device's primary context: it does not survive cudaDeviceReset.
constexpr int kMaxDevices = 64;
class DeviceOnce {
 public:
  template <typename Fn>
  int run(const char* what, Fn&& fn) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) {
      set_error("%s: device ordinal %d not supported (at most %d devices)", what, dev, kMaxDevices);
      return BSRL_ERR_UNSUPPORTED;
    }
    std::call_once(flag_[dev], [&] { err_[dev] = fn(); });
    if (err_[dev] != cudaSuccess) return cuda_fail(err_[dev], what);
    return BSRL_OK;
  }

 private:
  std::once_flag flag_[kMaxDevices];
  cudaError_t err_[kMaxDevices] = {};
};

// ----------------------------------------------------------------------------- device
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  int n = pred ? 16 : 0;  // src-size 0 => zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8, f32) += A(16x16, f16 row) * B(16x8, f16 col)
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// erf-based GELU, 0.5 x (1 + erf(x / sqrt 2)): torch.nn.GELU() with its default approximate='none'.
// erf by the rational-exponential form 1 - (a1 t + ... + a5 t^5) exp(-z^2), t = 1 / (1 + p z), whose absolute
// error is below 1.5e-7 (Abramowitz & Stegun 7.1.26) -- float rounding level, three orders under the fp16
// rounding of the hidden activations this feeds -- in one branch-free sequence with two special-function
// instructions; it runs inside GEMM epilogues, 1024 times per token row and block.
__device__ __forceinline__ float gelu_exact(float x) {
  const float z = fabsf(x) * 0.70710678118654752f;
  float t, ex;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.f)));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(-1.4426950408889634f * z * z));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float e = poly * t * ex;                                   // 1 - erf(z), z >= 0
  // 0.5 x (1 + sign(x) (1 - e)) = x >= 0 ? x - 0.5 x e : 0.5 x e
  const float he = 0.5f * x * e;
  return x >= 0.f ? x - he : he;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace bsrl
