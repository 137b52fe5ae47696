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

// RPW rows per warp are in flight together: the kernel is latency-bound on its loads, and a second
// (third, fourth) independent row per warp multiplies the bytes in flight.
// F32: the output rows are fp32 (y points at floats) instead of fp16.
template <int RPW, bool F32>
__global__ void __launch_bounds__(256, RPW > 1 ? 4 : 1) layernorm_kernel(const float* __restrict__ x, int64_t ldx,
                                                       RowMap xmap, const float* __restrict__ gamma,
                                                       const float* __restrict__ beta, float eps,
                                                       int64_t rows, int d, __half* __restrict__ y,
                                                       int64_t ldy) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int nvec = d >> 2;
  constexpr int NV = kMaxVec / RPW;                // float4 per lane and row: rows up to 1024 / 512 / 256 wide
  for (int64_t row0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW; row0 < rows;
       row0 += warps * RPW) {
    float4 v[RPW][NV];
    float s[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      s[r] = 0.f;
      const int64_t row = row0 + r;
      if (row < rows) {
        const float4* xr = reinterpret_cast<const float4*>(x + xmap(row) * ldx);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c = lane + i * 32;
          if (c < nvec) v[r][i] = xr[c];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (lane + i * 32 < nvec && row0 + r < rows) s[r] += (v[r][i].x + v[r][i].y) + (v[r][i].z + v[r][i].w);
    float mean[RPW], rstd[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) mean[r] = warp_sum(s[r]) / d;
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (lane + i * 32 < nvec && row0 + r < rows) {
          const float a = v[r][i].x - mean[r], b = v[r][i].y - mean[r], e = v[r][i].z - mean[r], f = v[r][i].w - mean[r];
          q += (a * a + b * b) + (e * e + f * f);
        }
      rstd[r] = rsqrtf(warp_sum(q) / d + eps);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        const float4 g = reinterpret_cast<const float4*>(gamma)[c];
        const float4 b = reinterpret_cast<const float4*>(beta)[c];
#pragma unroll
        for (int r = 0; r < RPW; ++r)
          if (row0 + r < rows) {
            const float o0 = (v[r][i].x - mean[r]) * rstd[r] * g.x + b.x, o1 = (v[r][i].y - mean[r]) * rstd[r] * g.y + b.y;
            const float o2 = (v[r][i].z - mean[r]) * rstd[r] * g.z + b.z, o3 = (v[r][i].w - mean[r]) * rstd[r] * g.w + b.w;
            if (F32) {
              reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + (row0 + r) * ldy)[c] = make_float4(o0, o1, o2, o3);
            } else {
              uint2 o;
              o.x = pack_half2(o0, o1);
              o.y = pack_half2(o2, o3);
              reinterpret_cast<uint2*>(y + (row0 + r) * ldy)[c] = o;
            }
          }
      }
    }
  }
}
}  // namespace

namespace {
template <bool F32>
int launch_layernorm(const float* x, int64_t ldx, RowMap xmap, const float* gamma, const float* beta,
                     float eps, int64_t rows, int d, __half* y, int64_t ldy, cudaStream_t stream);
}
int layernorm_rows(const float* x, int64_t ldx, RowMap xmap, const float* gamma, const float* beta,
                   float eps, int64_t rows, int d, __half* y, int64_t ldy, cudaStream_t stream) {
  return launch_layernorm<false>(x, ldx, xmap, gamma, beta, eps, rows, d, y, ldy, stream);
}
// fp32 rows out (may be in place: every row is read completely before it is written)
int layernorm_rows_f32(const float* x, int64_t ldx, const float* gamma, const float* beta, float eps,
                       int64_t rows, int d, float* y, int64_t ldy, cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(y) & 15) || (ldy % 4)) {
    set_error("layernorm: fp32 output rows must be 16-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  return launch_layernorm<true>(x, ldx, identity_map(), gamma, beta, eps, rows, d, reinterpret_cast<__half*>(y), ldy, stream);
}
namespace {
template <bool F32>
int launch_layernorm(const float* x, int64_t ldx, RowMap xmap, const float* gamma, const float* beta,
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
  const int64_t cap = (int64_t)sm_count() * 16;
  const int rpw = rows < cap * 8 * 4 ? 1 : d <= 256 ? 4 : d <= 512 ? 2 : 1;   // long inputs: several rows per warp
  int64_t blocks = (rows + 8 * rpw - 1) / (8 * rpw);
  if (blocks > cap) blocks = cap;
  const unsigned nb = static_cast<unsigned>(blocks);
  if (rpw == 4) layernorm_kernel<4, F32><<<nb, 256, 0, stream>>>(x, ldx, xmap, gamma, beta, eps, rows, d, y, ldy);
  else if (rpw == 2) layernorm_kernel<2, F32><<<nb, 256, 0, stream>>>(x, ldx, xmap, gamma, beta, eps, rows, d, y, ldy);
  else layernorm_kernel<1, F32><<<nb, 256, 0, stream>>>(x, ldx, xmap, gamma, beta, eps, rows, d, y, ldy);
  BSRL_LAUNCH_OK("layernorm_kernel");
  return BSRL_OK;
}
}  // namespace

// ---- SimBaV2 trunk row operations (NotePolicy._trunk_v2, python/policy.py:1140-1155), warp per row ----
// l2n(v) = v / max(|v|, 1e-6) (F.normalize).  mode 0: x = l2n(in * s) -> x (fp32, in place allowed) and
// x16.  mode 1: y = l2n(in); x = l2n(x + alpha c_alpha (y - x)); out16 = sqrt(d) x.
namespace {
__global__ void __launch_bounds__(256) simba2_rows_kernel(int mode, const float* in, float* x,
                                                         const float* __restrict__ vec, float c_alpha,
                                                         int64_t rows, int d, __half* __restrict__ out16,
                                                         int64_t ld16) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int nvec = d >> 2;
  const float4* v4 = reinterpret_cast<const float4*>(vec);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    const float4* ir = reinterpret_cast<const float4*>(in + row * d);
    float4* xr = reinterpret_cast<float4*>(x + row * d);
    float4 a[kMaxVec], b[kMaxVec];
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        a[i] = ir[c];
        if (mode == 0) {
          const float4 s = v4[c];
          a[i].x *= s.x; a[i].y *= s.y; a[i].z *= s.z; a[i].w *= s.w;
        }
        q += (a[i].x * a[i].x + a[i].y * a[i].y) + (a[i].z * a[i].z + a[i].w * a[i].w);
      }
    }
    const float inv = 1.f / fmaxf(sqrtf(warp_sum(q)), 1e-6f);
    if (mode == 0) {
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int c = lane + i * 32;
        if (c < nvec) {
          const float4 o = make_float4(a[i].x * inv, a[i].y * inv, a[i].z * inv, a[i].w * inv);
          xr[c] = o;
          reinterpret_cast<uint2*>(out16 + row * ld16)[c] = make_uint2(pack_half2(o.x, o.y), pack_half2(o.z, o.w));
        }
      }
      continue;
    }
    float q2 = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        const float4 xv = xr[c], al = v4[c];
        b[i].x = xv.x + al.x * c_alpha * (a[i].x * inv - xv.x);
        b[i].y = xv.y + al.y * c_alpha * (a[i].y * inv - xv.y);
        b[i].z = xv.z + al.z * c_alpha * (a[i].z * inv - xv.z);
        b[i].w = xv.w + al.w * c_alpha * (a[i].w * inv - xv.w);
        q2 += (b[i].x * b[i].x + b[i].y * b[i].y) + (b[i].z * b[i].z + b[i].w * b[i].w);
      }
    }
    const float sc = sqrtf((float)d) / fmaxf(sqrtf(warp_sum(q2)), 1e-6f);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec)
        reinterpret_cast<uint2*>(out16 + row * ld16)[c] =
            make_uint2(pack_half2(b[i].x * sc, b[i].y * sc), pack_half2(b[i].z * sc, b[i].w * sc));
    }
  }
}

// out16 = relu(in * s), elementwise on (rows, n) fp32 -> fp16
__global__ void scale_relu_kernel(const float* __restrict__ in, const float* __restrict__ s, int64_t rows, int n,
                                  __half* __restrict__ out16) {
  const int per_row = n >> 2;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (int64_t)gridDim.x * blockDim.x) {
    int c;
    div_index(i, per_row, &c);
    const float4 v = reinterpret_cast<const float4*>(in)[i], sv = reinterpret_cast<const float4*>(s)[c];
    reinterpret_cast<uint2*>(out16)[i] = make_uint2(pack_half2(fmaxf(v.x * sv.x, 0.f), fmaxf(v.y * sv.y, 0.f)),
                                                   pack_half2(fmaxf(v.z * sv.z, 0.f), fmaxf(v.w * sv.w, 0.f)));
  }
}
}  // namespace

int simba2_rows(int mode, const float* in, float* x, const float* vec, float c_alpha, int64_t rows, int d,
                __half* out16, int64_t ld16, cudaStream_t stream) {
  if (!in || !x || !vec || !out16) {
    set_error("simba2_rows: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (d <= 0 || d % 4 != 0 || d > kMaxVec * 128 || (ld16 % 4) || !aligned16(in) || !aligned16(x) || !aligned16(vec) ||
      (reinterpret_cast<uintptr_t>(out16) & 7)) {
    set_error("simba2_rows: width %d / alignment unsupported", d);
    return BSRL_ERR_SHAPE;
  }
  if (rows == 0) return BSRL_OK;
  int64_t blocks = (rows + 7) / 8;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  simba2_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(mode, in, x, vec, c_alpha, rows, d, out16, ld16);
  BSRL_LAUNCH_OK("simba2_rows_kernel");
  return BSRL_OK;
}

int scale_relu_rows(const float* in, const float* s, int64_t rows, int n, __half* out16, cudaStream_t stream) {
  if (!in || !s || !out16 || (n % 4) || !aligned16(in) || !aligned16(s) || (reinterpret_cast<uintptr_t>(out16) & 7)) {
    set_error("scale_relu_rows: bad operand");
    return BSRL_ERR_SHAPE;
  }
  if (rows == 0) return BSRL_OK;
  int64_t blocks = (rows * (n >> 2) + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  scale_relu_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(in, s, rows, n, out16);
  BSRL_LAUNCH_OK("scale_relu_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
