// Row LayerNorm: fp32 rows in, fp16 rows out, fp32 statistics; one warp per row.
//
// Stands in for FusedLayerNorm.forward (python/fused_ln.py:126-138) and its kernels
// ln_fwd_kernel / ln_fwd_h_kernel (python/beat_arena_env/csrc/layer_norm.cu:58-89, :147-201).
// The statistics are two-pass (mean, then centred variance) on register-resident rows.
// Pure streaming kernel: 4*d bytes read + 2*d bytes written per row.
#include "kernels.cuh"

namespace bsrl {
namespace {
constexpr int kMaxVec = 8;  // float4 per lane => rows up to 1024 wide

__global__ void __launch_bounds__(256) layernorm_kernel(const float* __restrict__ x, int64_t ldx,
                                                       RowMap xmap, const float* __restrict__ gamma,
                                                       const float* __restrict__ beta, float eps,
                                                       int64_t rows, int d, __half* __restrict__ y,
                                                       int64_t ldy) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int nvec = d >> 2;
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += warps) {
    const float4* xr = reinterpret_cast<const float4*>(x + xmap(row) * ldx);
    float4 v[kMaxVec];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int c = lane + i * 32;
      if (c < nvec) {
        v[i] = xr[c];
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    const float mean = warp_sum(s) / d;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int c = lane + i * 32;
      if (c < nvec) {
        float a = v[i].x - mean, b = v[i].y - mean, e = v[i].z - mean, f = v[i].w - mean;
        q += (a * a + b * b) + (e * e + f * f);
      }
    }
    const float rstd = rsqrtf(warp_sum(q) / d + eps);
    uint2* yr = reinterpret_cast<uint2*>(y + row * ldy);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int c = lane + i * 32;
      if (c < nvec) {
        float4 g = reinterpret_cast<const float4*>(gamma)[c];
        float4 b = reinterpret_cast<const float4*>(beta)[c];
        uint2 o;
        o.x = pack_half2((v[i].x - mean) * rstd * g.x + b.x, (v[i].y - mean) * rstd * g.y + b.y);
        o.y = pack_half2((v[i].z - mean) * rstd * g.z + b.z, (v[i].w - mean) * rstd * g.w + b.w);
        yr[c] = o;
      }
    }
  }
}
}  // namespace

int layernorm_rows(const float* x, int64_t ldx, RowMap xmap, const float* gamma, const float* beta,
                   float eps, int64_t rows, int d, __half* y, int64_t ldy, cudaStream_t stream) {
  if (!x || !gamma || !beta || !y) {
    set_error("layernorm: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (d <= 0 || d % 4 != 0 || d > kMaxVec * 128 || rows < 0) {
    set_error("layernorm: width %d unsupported (need d %% 4 == 0, d <= 1024)", d);
    return BSRL_ERR_SHAPE;
  }
  if (!aligned16(x) || !aligned16(gamma) || !aligned16(beta) || (ldx % 4) || (ldy % 4) ||
      (reinterpret_cast<uintptr_t>(y) & 7)) {
    set_error("layernorm: rows must be 16-byte (in) / 8-byte (out) aligned");
    return BSRL_ERR_ALIGN;
  }
  if (rows == 0) return BSRL_OK;
  int64_t blocks = (rows + 7) / 8;
  int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  layernorm_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(x, ldx, xmap, gamma, beta, eps,
                                                                     rows, d, y, ldy);
  BSRL_LAUNCH_OK("layernorm_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
