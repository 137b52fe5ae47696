// Backward kernels of the forward's A/B options: the value residual (python/policy.py:604-615, _VMix) and the
// SimBaV2 readout trunk (python/policy.py:1140-1155).  Row kernels, one warp per row where a row statistic is
// needed; parameter gradients that sum over rows collect per block in shared memory and leave as one atomic per
// column and block.  Activation gradients arrive and leave multiplied by the caller's loss scale (everything here
// is linear in them).
#include "kernels.cuh"

namespace bsrl {
namespace {

constexpr int kMaxVec = 8;   // float4 per lane: rows up to 1024 wide

int64_t blocks_for_rows(int64_t rows, int rows_per_block) {
  int64_t b = (rows + rows_per_block - 1) / rows_per_block;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (b > cap) b = cap;
  return b < 1 ? 1 : b;
}

// v' = a v + b v0  =>  g_v = a g', g_v0 += b g', g_a += sum g' v, g_b += sum g' v0.
// g: fp16 gradient of the mixed values, rewritten in place as the gradient of the block's own values.
__global__ void __launch_bounds__(256) vres_bwd_kernel(__half* __restrict__ g, int64_t ldg, const __half* __restrict__ v_own,
                                                       const __half* __restrict__ v0, const float* __restrict__ ab,
                                                       float* __restrict__ g_v0, float* __restrict__ g_a, float* __restrict__ g_b,
                                                       int64_t rows, int d) {
  const float a = ab[0], b = ab[1];
  const int per_row = d >> 3;
  float sa = 0.f, sb = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row; i += (int64_t)gridDim.x * blockDim.x) {
    int piece;
    const int64_t row = div_index(i, per_row, &piece);
    const int c = piece * 8;
    uint4 gv = *reinterpret_cast<const uint4*>(g + row * ldg + c);
    const uint4 ov = *reinterpret_cast<const uint4*>(v_own + row * d + c);
    const uint4 zv = *reinterpret_cast<const uint4*>(v0 + row * d + c);
    uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
    const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, zw[4] = {zv.x, zv.y, zv.z, zv.w};
    float acc[8];
    const float4 p0 = *reinterpret_cast<const float4*>(g_v0 + row * d + c), p1 = *reinterpret_cast<const float4*>(g_v0 + row * d + c + 4);
    acc[0] = p0.x; acc[1] = p0.y; acc[2] = p0.z; acc[3] = p0.w; acc[4] = p1.x; acc[5] = p1.y; acc[6] = p1.z; acc[7] = p1.w;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 gg = __half22float2(*reinterpret_cast<const __half2*>(&gw[e]));
      const float2 oo = __half22float2(*reinterpret_cast<const __half2*>(&ow[e]));
      const float2 zz = __half22float2(*reinterpret_cast<const __half2*>(&zw[e]));
      sa += gg.x * oo.x + gg.y * oo.y;
      sb += gg.x * zz.x + gg.y * zz.y;
      acc[2 * e] += b * gg.x;
      acc[2 * e + 1] += b * gg.y;
      gw[e] = pack_half2(a * gg.x, a * gg.y);
    }
    *reinterpret_cast<uint4*>(g + row * ldg + c) = make_uint4(gw[0], gw[1], gw[2], gw[3]);
    *reinterpret_cast<float4*>(g_v0 + row * d + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(g_v0 + row * d + c + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  __shared__ float red[2][8];
  sa = warp_sum(sa);
  sb = warp_sum(sb);
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = sa;
    red[1][threadIdx.x >> 5] = sb;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float ta = 0.f, tb = 0.f;
    for (int w = 0; w < 8; ++w) {
      ta += red[0][w];
      tb += red[1][w];
    }
    if (g_a) atomicAdd(g_a, ta);
    if (g_b) atomicAdd(g_b, tb);
  }
}

// g16[r, c] += fp16(acc32[r, c]) (fp32 arithmetic, rounded once)
__global__ void __launch_bounds__(256) add_f32_into_f16_kernel(__half* __restrict__ g, int64_t ldg, const float* __restrict__ acc,
                                                               int64_t rows, int d) {
  const int per_row = d >> 2;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row; i += (int64_t)gridDim.x * blockDim.x) {
    int piece;
    const int64_t row = div_index(i, per_row, &piece);
    const int c = piece * 4;
    const float4 a = *reinterpret_cast<const float4*>(acc + row * d + c);
    uint2 gv = *reinterpret_cast<const uint2*>(g + row * ldg + c);
    const float2 g0 = __half22float2(*reinterpret_cast<const __half2*>(&gv.x)), g1 = __half22float2(*reinterpret_cast<const __half2*>(&gv.y));
    gv.x = pack_half2(g0.x + a.x, g0.y + a.y);
    gv.y = pack_half2(g1.x + a.z, g1.y + a.w);
    *reinterpret_cast<uint2*>(g + row * ldg + c) = gv;
  }
}

// per-block partial sums of a per-column parameter gradient: add this lane's float4 pieces, then one atomic per column
template <int NV>
__device__ __forceinline__ void flush_column_sums(float* s_part, const float4 (&acc)[NV], int d, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (lane + i * 32) * 4;
    if (c < d) {
      atomicAdd(&s_part[c], acc[i].x); atomicAdd(&s_part[c + 1], acc[i].y);
      atomicAdd(&s_part[c + 2], acc[i].z); atomicAdd(&s_part[c + 3], acc[i].w);
    }
  }
  __syncthreads();
  if (out)
    for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(&out[i], s_part[i]);
}

// SimBaV2 output side.  Forward: y = l2n(t2); w = x0 + a (y - x0), a = alpha c_alpha; x1 = l2n(w); h = sqrt(D) x1.
// Given g_h: g_x0 (partial, fp32) = g_w (1 - a); g_t2 (fp16) = l2n backward of g_y = g_w a; g_alpha += sum g_w c_alpha (y - x0).
__global__ void __launch_bounds__(256) simba2_out_bwd_kernel(const float* __restrict__ x0, const float* __restrict__ t2,
                                                             const float* __restrict__ alpha, float c_alpha,
                                                             const float* __restrict__ g_h, float* __restrict__ g_x0,
                                                             __half* __restrict__ g_t2, float* __restrict__ g_alpha,
                                                             int64_t rows, int d) {
  extern __shared__ float s_part[];
  for (int i = threadIdx.x; i < d; i += blockDim.x) s_part[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, nvec = d >> 2;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const float sqrt_d = sqrtf((float)d);
  float4 acc[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    float4 xv[kMaxVec], yv[kMaxVec], gv[kMaxVec], av[kMaxVec];
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        xv[i] = reinterpret_cast<const float4*>(x0 + row * d)[c];
        yv[i] = reinterpret_cast<const float4*>(t2 + row * d)[c];
        gv[i] = reinterpret_cast<const float4*>(g_h + row * d)[c];
        av[i] = reinterpret_cast<const float4*>(alpha)[c];
        av[i].x *= c_alpha; av[i].y *= c_alpha; av[i].z *= c_alpha; av[i].w *= c_alpha;
        q += (yv[i].x * yv[i].x + yv[i].y * yv[i].y) + (yv[i].z * yv[i].z + yv[i].w * yv[i].w);
      }
    }
    const float inv_t = 1.f / fmaxf(sqrtf(warp_sum(q)), 1e-6f);
    float q2 = 0.f;
    float4 wv[kMaxVec];
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
      if (lane + i * 32 < nvec) {
        yv[i].x *= inv_t; yv[i].y *= inv_t; yv[i].z *= inv_t; yv[i].w *= inv_t;          // y
        wv[i].x = xv[i].x + av[i].x * (yv[i].x - xv[i].x); wv[i].y = xv[i].y + av[i].y * (yv[i].y - xv[i].y);
        wv[i].z = xv[i].z + av[i].z * (yv[i].z - xv[i].z); wv[i].w = xv[i].w + av[i].w * (yv[i].w - xv[i].w);
        q2 += (wv[i].x * wv[i].x + wv[i].y * wv[i].y) + (wv[i].z * wv[i].z + wv[i].w * wv[i].w);
      }
    const float inv_w = 1.f / fmaxf(sqrtf(warp_sum(q2)), 1e-6f);
    float dot = 0.f;      // x1 . g_x1, with g_x1 = sqrt(D) g_h and x1 = w inv_w
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
      if (lane + i * 32 < nvec) {
        wv[i].x *= inv_w; wv[i].y *= inv_w; wv[i].z *= inv_w; wv[i].w *= inv_w;          // x1
        gv[i].x *= sqrt_d; gv[i].y *= sqrt_d; gv[i].z *= sqrt_d; gv[i].w *= sqrt_d;      // g_x1
        dot += (wv[i].x * gv[i].x + wv[i].y * gv[i].y) + (wv[i].z * gv[i].z + wv[i].w * gv[i].w);
      }
    dot = warp_sum(dot);
    float dot_y = 0.f;    // y . g_y
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        // g_w = (g_x1 - x1 (x1 . g_x1)) / |w|
        float4 gw = make_float4((gv[i].x - wv[i].x * dot) * inv_w, (gv[i].y - wv[i].y * dot) * inv_w,
                                (gv[i].z - wv[i].z * dot) * inv_w, (gv[i].w - wv[i].w * dot) * inv_w);
        acc[i].x += gw.x * c_alpha * (yv[i].x - xv[i].x); acc[i].y += gw.y * c_alpha * (yv[i].y - xv[i].y);
        acc[i].z += gw.z * c_alpha * (yv[i].z - xv[i].z); acc[i].w += gw.w * c_alpha * (yv[i].w - xv[i].w);
        reinterpret_cast<float4*>(g_x0 + row * d)[c] =
            make_float4(gw.x * (1.f - av[i].x), gw.y * (1.f - av[i].y), gw.z * (1.f - av[i].z), gw.w * (1.f - av[i].w));
        gv[i] = make_float4(gw.x * av[i].x, gw.y * av[i].y, gw.z * av[i].z, gw.w * av[i].w);       // g_y
        dot_y += (yv[i].x * gv[i].x + yv[i].y * gv[i].y) + (yv[i].z * gv[i].z + yv[i].w * gv[i].w);
      }
    }
    dot_y = warp_sum(dot_y);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec)
        reinterpret_cast<uint2*>(g_t2 + row * d)[c] =
            make_uint2(pack_half2((gv[i].x - yv[i].x * dot_y) * inv_t, (gv[i].y - yv[i].y * dot_y) * inv_t),
                       pack_half2((gv[i].z - yv[i].z * dot_y) * inv_t, (gv[i].w - yv[i].w * dot_y) * inv_t));
    }
  }
  flush_column_sums<kMaxVec>(s_part, acc, d, g_alpha);
}

// SimBaV2 input side.  Forward: ts = t0 s; x0 = l2n(ts).  g_x0 = g_a + g_b (two fp32 contributions);
// g_ts = (g_x0 - x0 (x0 . g_x0)) / |ts|; g_t0 (fp16) = g_ts s; g_s += sum g_ts t0.
__global__ void __launch_bounds__(256) simba2_in_bwd_kernel(const float* __restrict__ t0, const float* __restrict__ s,
                                                            const float* __restrict__ g_a, const float* __restrict__ g_b,
                                                            __half* __restrict__ g_t0, float* __restrict__ g_s, int64_t rows, int d) {
  extern __shared__ float s_part[];
  for (int i = threadIdx.x; i < d; i += blockDim.x) s_part[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, nvec = d >> 2;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  float4 acc[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    float4 tv[kMaxVec], xs[kMaxVec], gv[kMaxVec], sv[kMaxVec];
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        tv[i] = reinterpret_cast<const float4*>(t0 + row * d)[c];
        sv[i] = reinterpret_cast<const float4*>(s)[c];
        const float4 ga = reinterpret_cast<const float4*>(g_a + row * d)[c], gb = reinterpret_cast<const float4*>(g_b + row * d)[c];
        gv[i] = make_float4(ga.x + gb.x, ga.y + gb.y, ga.z + gb.z, ga.w + gb.w);
        xs[i] = make_float4(tv[i].x * sv[i].x, tv[i].y * sv[i].y, tv[i].z * sv[i].z, tv[i].w * sv[i].w);
        q += (xs[i].x * xs[i].x + xs[i].y * xs[i].y) + (xs[i].z * xs[i].z + xs[i].w * xs[i].w);
      }
    }
    const float inv = 1.f / fmaxf(sqrtf(warp_sum(q)), 1e-6f);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
      if (lane + i * 32 < nvec) {
        xs[i].x *= inv; xs[i].y *= inv; xs[i].z *= inv; xs[i].w *= inv;                  // x0
        dot += (xs[i].x * gv[i].x + xs[i].y * gv[i].y) + (xs[i].z * gv[i].z + xs[i].w * gv[i].w);
      }
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        const float4 gt = make_float4((gv[i].x - xs[i].x * dot) * inv, (gv[i].y - xs[i].y * dot) * inv,
                                      (gv[i].z - xs[i].z * dot) * inv, (gv[i].w - xs[i].w * dot) * inv);
        acc[i].x += gt.x * tv[i].x; acc[i].y += gt.y * tv[i].y; acc[i].z += gt.z * tv[i].z; acc[i].w += gt.w * tv[i].w;
        reinterpret_cast<uint2*>(g_t0 + row * d)[c] =
            make_uint2(pack_half2(gt.x * sv[i].x, gt.y * sv[i].y), pack_half2(gt.z * sv[i].z, gt.w * sv[i].w));
      }
    }
  }
  flush_column_sums<kMaxVec>(s_part, acc, d, g_s);
}

// r = relu(t s): g_t (fp16, in place on g_r) = g_r s [t s > 0]; g_s += sum g_r t [t s > 0].  One warp per row.
__global__ void __launch_bounds__(256) scale_relu_bwd_kernel(__half* __restrict__ g, const float* __restrict__ t,
                                                             const float* __restrict__ s, float* __restrict__ g_s, int64_t rows, int n) {
  extern __shared__ float s_part[];
  for (int i = threadIdx.x; i < n; i += blockDim.x) s_part[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, nvec = n >> 2;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  float4 acc[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        const float4 tv = reinterpret_cast<const float4*>(t + row * n)[c], sv = reinterpret_cast<const float4*>(s)[c];
        uint2 gr = reinterpret_cast<const uint2*>(g + row * n)[c];
        const float2 g0 = __half22float2(*reinterpret_cast<const __half2*>(&gr.x)), g1 = __half22float2(*reinterpret_cast<const __half2*>(&gr.y));
        const float gx = tv.x * sv.x > 0.f ? g0.x : 0.f, gy = tv.y * sv.y > 0.f ? g0.y : 0.f;
        const float gz = tv.z * sv.z > 0.f ? g1.x : 0.f, gw = tv.w * sv.w > 0.f ? g1.y : 0.f;
        acc[i].x += gx * tv.x; acc[i].y += gy * tv.y; acc[i].z += gz * tv.z; acc[i].w += gw * tv.w;
        gr.x = pack_half2(gx * sv.x, gy * sv.y);
        gr.y = pack_half2(gz * sv.z, gw * sv.w);
        reinterpret_cast<uint2*>(g + row * n)[c] = gr;
      }
    }
  }
  flush_column_sums<kMaxVec>(s_part, acc, n, g_s);
}

}  // namespace

int vres_bwd(__half* g, int64_t ldg, const __half* v_own, const __half* v0, const float* ab, float* g_v0, float* g_a, float* g_b,
             int64_t rows, int d, cudaStream_t stream) {
  if (!g || !v_own || !v0 || !ab || !g_v0 || (d % 8) || (ldg % 8) || !aligned16(g) || !aligned16(v_own) || !aligned16(v0) ||
      !aligned16(g_v0)) {
    set_error("vres_bwd: bad operand");
    return BSRL_ERR_SHAPE;
  }
  if (rows == 0) return BSRL_OK;
  vres_bwd_kernel<<<(unsigned)blocks_for_rows(rows * (d >> 3), 256), 256, 0, stream>>>(g, ldg, v_own, v0, ab, g_v0, g_a, g_b, rows, d);
  BSRL_LAUNCH_OK("vres_bwd_kernel");
  return BSRL_OK;
}

int add_f32_into_f16(__half* g, int64_t ldg, const float* acc, int64_t rows, int d, cudaStream_t stream) {
  if (!g || !acc || (d % 4) || (ldg % 4) || !aligned16(acc) || (reinterpret_cast<uintptr_t>(g) & 7)) {
    set_error("add_f32_into_f16: bad operand");
    return BSRL_ERR_SHAPE;
  }
  if (rows == 0) return BSRL_OK;
  add_f32_into_f16_kernel<<<(unsigned)blocks_for_rows(rows * (d >> 2), 256), 256, 0, stream>>>(g, ldg, acc, rows, d);
  BSRL_LAUNCH_OK("add_f32_into_f16_kernel");
  return BSRL_OK;
}

static bool row_ok(int d) { return d > 0 && d % 4 == 0 && d <= kMaxVec * 128; }

int simba2_out_bwd(const float* x0, const float* t2, const float* alpha, float c_alpha, const float* g_h, float* g_x0, __half* g_t2,
                   float* g_alpha, int64_t rows, int d, cudaStream_t stream) {
  if (!x0 || !t2 || !alpha || !g_h || !g_x0 || !g_t2 || !row_ok(d)) {
    set_error("simba2_out_bwd: bad operand (width %d)", d);
    return BSRL_ERR_SHAPE;
  }
  if (rows == 0) return BSRL_OK;
  simba2_out_bwd_kernel<<<(unsigned)blocks_for_rows(rows, 8), 256, d * sizeof(float), stream>>>(x0, t2, alpha, c_alpha, g_h, g_x0, g_t2,
                                                                                             g_alpha, rows, d);
  BSRL_LAUNCH_OK("simba2_out_bwd_kernel");
  return BSRL_OK;
}

int simba2_in_bwd(const float* t0, const float* s, const float* g_a, const float* g_b, __half* g_t0, float* g_s, int64_t rows, int d,
                  cudaStream_t stream) {
  if (!t0 || !s || !g_a || !g_b || !g_t0 || !row_ok(d)) {
    set_error("simba2_in_bwd: bad operand (width %d)", d);
    return BSRL_ERR_SHAPE;
  }
  if (rows == 0) return BSRL_OK;
  simba2_in_bwd_kernel<<<(unsigned)blocks_for_rows(rows, 8), 256, d * sizeof(float), stream>>>(t0, s, g_a, g_b, g_t0, g_s, rows, d);
  BSRL_LAUNCH_OK("simba2_in_bwd_kernel");
  return BSRL_OK;
}

int scale_relu_bwd(__half* g, const float* t, const float* s, float* g_s, int64_t rows, int n, cudaStream_t stream) {
  if (!g || !t || !s || !row_ok(n)) {
    set_error("scale_relu_bwd: bad operand (width %d)", n);
    return BSRL_ERR_SHAPE;
  }
  if (rows == 0) return BSRL_OK;
  scale_relu_bwd_kernel<<<(unsigned)blocks_for_rows(rows, 8), 256, n * sizeof(float), stream>>>(g, t, s, g_s, rows, n);
  BSRL_LAUNCH_OK("scale_relu_bwd_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
