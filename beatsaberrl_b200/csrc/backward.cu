// Row and element kernels of the backward pass of the policy forward (the PPO update's recompute):
// LayerNorm backward with the residual gradient folded in, bias gradients (column sums), the ReLU mask,
// fp32 -> fp16 casts with row gathers, tiled transposes (the weight-gradient GEMMs reduce over token
// rows, so both of their operands are transposed into K-major form first), and the backward of the
// head tail (log-softmax / log-prob / entropy / HL-Gauss value).
//
// Counterparts in the reference: ln_bwd* (python/beat_arena_env/csrc/layer_norm.cu:289-519;
// python/fused_ln.py:58-107), relu_bwd / wgrad_bgrad / dgrad_drelu
// (python/beat_arena_env/csrc/fp16_gemm.cu:129-187, :252-373, :499-518) and autograd through
// python/policy.py:1473-1516.  Gradients of activations travel as fp16 GEMM operands multiplied by a
// loss scale chosen by the caller; the residual-stream gradient, LayerNorm arithmetic and every
// parameter gradient are fp32.
#include "kernels.cuh"

namespace bsrl {
namespace {

constexpr int kMaxVecAll = 8;   // float4 per lane: rows up to 1024 wide

// dx = rstd (gy g - mean(gy g) - xhat mean(gy g xhat)); gx_out = (gres ? gres : 0) + dx; gx16 = fp16(gx_out) if asked;
// ggamma += sum_rows gy xhat, gbeta += sum_rows gy.  One warp per row; per-block partial sums of the
// parameter gradients in shared memory, then one atomic per column per block.
template <bool GY_F32, int kMaxVec>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const float* __restrict__ x, int64_t ldx, RowMap xmap,
                                                     const float* __restrict__ gamma, float eps, const void* __restrict__ gy,
                                                     int64_t ldgy, const float* gres, float* gx_out, int64_t ldg, RowMap gmap,
                                                     __half* __restrict__ gx16, int64_t ldg16,
                                                     float* __restrict__ ggamma, float* __restrict__ gbeta, int64_t rows, int d) {
  extern __shared__ float s_part[];                  // [2][d]
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) s_part[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int nvec = d >> 2;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  float4 acc_g[kMaxVec], acc_b[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) acc_g[i] = acc_b[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    const float4* xr = reinterpret_cast<const float4*>(x + xmap(row) * ldx);
    float4 v[kMaxVec], g[kMaxVec];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        v[i] = xr[c];
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        if (GY_F32) {
          g[i] = reinterpret_cast<const float4*>(static_cast<const float*>(gy) + row * ldgy)[c];
        } else {
          const uint2 raw = reinterpret_cast<const uint2*>(static_cast<const __half*>(gy) + row * ldgy)[c];
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
          const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
          g[i] = make_float4(a.x, a.y, b.x, b.y);
        }
      }
    }
    const float mean = warp_sum(s) / d;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
      if (lane + i * 32 < nvec) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      }
    const float rstd = rsqrtf(warp_sum(q) / d + eps);
    float s1 = 0.f, s2 = 0.f;                         // sum(gy g), sum(gy g xhat)
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        const float4 gm = reinterpret_cast<const float4*>(gamma)[c];
        v[i].x *= rstd; v[i].y *= rstd; v[i].z *= rstd; v[i].w *= rstd;         // xhat
        acc_g[i].x += g[i].x * v[i].x; acc_g[i].y += g[i].y * v[i].y; acc_g[i].z += g[i].z * v[i].z; acc_g[i].w += g[i].w * v[i].w;
        acc_b[i].x += g[i].x; acc_b[i].y += g[i].y; acc_b[i].z += g[i].z; acc_b[i].w += g[i].w;
        g[i].x *= gm.x; g[i].y *= gm.y; g[i].z *= gm.z; g[i].w *= gm.w;         // gy g
        s1 += (g[i].x + g[i].y) + (g[i].z + g[i].w);
        s2 += (g[i].x * v[i].x + g[i].y * v[i].y) + (g[i].z * v[i].z + g[i].w * v[i].w);
      }
    }
    s1 = warp_sum(s1) / d;
    s2 = warp_sum(s2) / d;
    const int64_t go = gmap(row) * ldg;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float4 o = make_float4(rstd * (g[i].x - s1 - v[i].x * s2), rstd * (g[i].y - s1 - v[i].y * s2),
                               rstd * (g[i].z - s1 - v[i].z * s2), rstd * (g[i].w - s1 - v[i].w * s2));
        if (gres) {
          const float4 r = reinterpret_cast<const float4*>(gres + go)[c];
          o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
        }
        reinterpret_cast<float4*>(gx_out + go)[c] = o;
        if (gx16)      // the same gradient as the fp16 operand of the products that follow (dense rows)
          reinterpret_cast<uint2*>(gx16 + row * ldg16)[c] = make_uint2(pack_half2(o.x, o.y), pack_half2(o.z, o.w));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (lane + i * 32) * 4;
    if (c < d) {
      atomicAdd(&s_part[c], acc_g[i].x); atomicAdd(&s_part[c + 1], acc_g[i].y);
      atomicAdd(&s_part[c + 2], acc_g[i].z); atomicAdd(&s_part[c + 3], acc_g[i].w);
      atomicAdd(&s_part[d + c], acc_b[i].x); atomicAdd(&s_part[d + c + 1], acc_b[i].y);
      atomicAdd(&s_part[d + c + 2], acc_b[i].z); atomicAdd(&s_part[d + c + 3], acc_b[i].w);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    if (ggamma) atomicAdd(&ggamma[i], s_part[i]);
    if (gbeta) atomicAdd(&gbeta[i], s_part[d + i]);
  }
}

// out[c] += sum_r in[r, c] (fp16 rows): bias gradients.  A warp covers 256 consecutive columns of a row with
// 16-byte loads, the 8 warps of a block take rows in turn (four in flight each); partial sums meet in shared
// memory and leave as one atomic per column and block.  n % 8 == 0, ld % 8 == 0, 16-byte aligned base.
__global__ void __launch_bounds__(256) colsum_kernel(const __half* __restrict__ in, int64_t ld, int64_t rows, int n,
                                                     int64_t chunk, float* __restrict__ out) {
  __shared__ float part[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 256 + lane * 8;
  const int64_t r0 = (int64_t)blockIdx.y * chunk, r1 = r0 + chunk < rows ? r0 + chunk : rows;
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c < n) {
    int64_t r = r0 + warp;
    for (; r + 24 < r1; r += 32) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(in + (r + 8 * u) * ld + c);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const __half2* h = reinterpret_cast<const __half2*>(&v[u]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __half22float2(h[k]);
          s[2 * k] += f.x;
          s[2 * k + 1] += f.y;
        }
      }
    }
    for (; r < r1; r += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(in + r * ld + c);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(h[k]);
        s[2 * k] += f.x;
        s[2 * k + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) part[warp][lane * 8 + k] = s[k];
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < n && r1 > r0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += part[w][threadIdx.x];
    atomicAdd(&out[col], t);
  }
}
// any shape: one thread per column
__global__ void __launch_bounds__(256) colsum_slow_kernel(const __half* __restrict__ in, int64_t ld, int64_t rows, int n,
                                                          int64_t chunk, float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  const int64_t r0 = (int64_t)blockIdx.y * chunk, r1 = r0 + chunk < rows ? r0 + chunk : rows;
  float s = 0.f;
  for (int64_t r = r0; r < r1; ++r) s += __half2float(in[r * ld + c]);
  if (r1 > r0) atomicAdd(&out[c], s);
}

// g <- (act > 0) ? g : 0, fp16 rows of n columns (n % 8 == 0)
__global__ void __launch_bounds__(256) relu_mask_kernel(__half* __restrict__ g, int64_t ldg, const __half* __restrict__ act,
                                                        int64_t lda, int64_t rows, int n) {
  const int nv = n >> 3;
  const int64_t total = rows * nv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int piece;
    const int64_t r = div_index(i, nv, &piece);
    const int c = piece * 8;
    uint4 gv = *reinterpret_cast<const uint4*>(g + r * ldg + c);
    const uint4 av = *reinterpret_cast<const uint4*>(act + r * lda + c);
    __half* gh = reinterpret_cast<__half*>(&gv);
    const __half* ah = reinterpret_cast<const __half*>(&av);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (!(__half2float(ah[k]) > 0.f)) gh[k] = __float2half_rn(0.f);
    *reinterpret_cast<uint4*>(g + r * ldg + c) = gv;
  }
}

// out16[r, :] = fp16(in32[map(r), :] * scale)
__global__ void __launch_bounds__(256) cast_rows16_kernel(const float* __restrict__ in, int64_t ldi, RowMap imap, float scale,
                                                          __half* __restrict__ out, int64_t ldo, int64_t rows, int n) {
  const int nv = n >> 2;
  const int64_t total = rows * nv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int piece;
    const int64_t r = div_index(i, nv, &piece);
    const int c = piece * 4;
    const float4 v = *reinterpret_cast<const float4*>(in + imap(r) * ldi + c);
    uint2 o;
    o.x = pack_half2(v.x * scale, v.y * scale);
    o.y = pack_half2(v.z * scale, v.w * scale);
    *reinterpret_cast<uint2*>(out + r * ldo + c) = o;
  }
}

// dst[map(r), :] (+)= src[r, :] (fp32 rows)
__global__ void __launch_bounds__(256) add_rows_kernel(const float* __restrict__ src, int64_t lds, float* __restrict__ dst,
                                                       int64_t ldd, RowMap dmap, int64_t rows, int n, int accumulate) {
  const int nv = n >> 2;
  const int64_t total = rows * nv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int piece;
    const int64_t r = div_index(i, nv, &piece);
    const int c = piece * 4;
    float4 v = *reinterpret_cast<const float4*>(src + r * lds + c);
    float4* o = reinterpret_cast<float4*>(dst + dmap(r) * ldd + c);
    if (accumulate) {
      const float4 w = *o;
      v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    *o = v;
  }
}

// out (cols, ldo) = in (rows, ldi)^T, fp16, 64 x 64 tiles through shared memory, 16-byte accesses on both
// sides; rows [rows, rows_pad) of the input read as zero, so the padded K range of the following GEMM
// contributes nothing.  With colsum, the column sums of the input (a Linear's bias gradient, when the input is
// dL/dy) are accumulated on the way: per-tile partial sums, one atomic per column and tile.
// Requires cols % 8 == 0, ldi % 8 == 0, ldo % 8 == 0 and 16-byte aligned bases.
__global__ void __launch_bounds__(256) transpose16_kernel(const __half* __restrict__ in, int64_t ldi, RowMap imap, int64_t rows,
                                                          int cols, __half* __restrict__ out, int64_t ldo, int64_t rows_pad,
                                                          float* __restrict__ colsum) {
  __shared__ __align__(16) __half tile[64][72];      // 144-byte rows: column reads of 8 rows hit 8 bank groups
  const int64_t r0 = (int64_t)blockIdx.x * 64;
  const int c0 = blockIdx.y * 64;
  const int t = threadIdx.x;
#pragma unroll
  for (int i = 0; i < 2; ++i) {                      // 64 rows x 8 chunks of 8 columns
    const int r = (t >> 3) + 32 * i, ch = t & 7;
    const int64_t row = r0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows && c0 + ch * 8 < cols) v = *reinterpret_cast<const uint4*>(in + imap(row) * ldi + c0 + ch * 8);
    *reinterpret_cast<uint4*>(&tile[r][ch * 8]) = v;
  }
  __syncthreads();
  if (colsum && t < 64 && c0 + t < cols) {
    float sum = 0.f;
#pragma unroll 8
    for (int r = 0; r < 64; ++r) sum += __half2float(tile[r][t]);
    atomicAdd(&colsum[c0 + t], sum);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {                      // 64 output rows (input columns) x 8 chunks of 8 input rows
    const int c = (t >> 3) + 32 * i, ch = t & 7;
    if (c0 + c < cols && r0 + ch * 8 < rows_pad) {
      __half v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = tile[ch * 8 + k][c];
      *reinterpret_cast<uint4*>(out + (int64_t)(c0 + c) * ldo + r0 + ch * 8) = *reinterpret_cast<const uint4*>(v);
    }
  }
}

// small-shape fallback of the transpose (any cols / alignment), element-wise
__global__ void __launch_bounds__(256) transpose16_slow_kernel(const __half* __restrict__ in, int64_t ldi, RowMap imap, int64_t rows,
                                                               int cols, __half* __restrict__ out, int64_t ldo, int64_t rows_pad,
                                                               float* __restrict__ colsum) {
  __shared__ __half tile[64][66];
  const int64_t r0 = (int64_t)blockIdx.x * 64;
  const int c0 = blockIdx.y * 64;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int r = i >> 6, c = i & 63;
    const int64_t row = r0 + r;
    tile[r][c] = (row < rows && c0 + c < cols) ? in[imap(row) * ldi + c0 + c] : __float2half_rn(0.f);
  }
  __syncthreads();
  if (colsum && threadIdx.x < 64 && c0 + threadIdx.x < cols) {
    float sum = 0.f;
    for (int r = 0; r < 64; ++r) sum += __half2float(tile[r][threadIdx.x]);
    atomicAdd(&colsum[c0 + threadIdx.x], sum);
  }
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int c = i >> 6, r = i & 63;
    if (c0 + c < cols && r0 + r < rows_pad) out[(int64_t)(c0 + c) * ldo + r0 + r] = tile[r][c];
  }
}

__device__ __forceinline__ int load_action(const void* a, int dtype, int64_t idx) {
  switch (dtype) {
    case BSRL_U8: return static_cast<const uint8_t*>(a)[idx];
    case BSRL_I32: return static_cast<const int32_t*>(a)[idx];
    default: return static_cast<int>(static_cast<const int64_t*>(a)[idx]);
  }
}

// Backward of the head tail, one warp per env.  With p = softmax(z) of a head's live lanes,
//   d logprob / dz_i = [i == a] - p_i,      d entropy / dz_i = -p_i (log p_i + H)
// and for the value  v = sum_i softmax(u)_i c_i:   dv / du_i = softmax(u)_i (c_i - v).
__global__ void __launch_bounds__(256) head_tail_bwd_kernel(HeadTailArgs p, const float* __restrict__ g_logprob,
                                                            const float* __restrict__ g_entropy, const float* __restrict__ g_value,
                                                            const float* __restrict__ g_vlogits, const float* __restrict__ g_logits,
                                                            float scale, __half* __restrict__ g_raw, int ldg_raw,
                                                            __half* __restrict__ g_vraw, int ldg_v) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t env = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); env < p.n_envs; env += warps) {
    for (int c = lane + p.first[kActHeads - 1] + p.gears[kActHeads - 1]; c < ldg_raw; c += 32)
      g_raw[env * (int64_t)ldg_raw + c] = __float2half_rn(0.f);   // padding columns of the packed head matrix
    if (lane < kActHeads) {
      const int k = p.gears[lane];
      const float* src = p.raw + env * p.ld_raw + p.first[lane];
      float v[7], mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 7; ++i) {
        v[i] = i < k ? src[i] : -INFINITY;
        mx = fmaxf(mx, v[i]);
      }
      float se = 0.f;
#pragma unroll
      for (int i = 0; i < 7; ++i)
        if (i < k) se += expf(v[i] - mx);
      const float lse = mx + logf(se);
      float ent = 0.f;
#pragma unroll
      for (int i = 0; i < 7; ++i)
        if (i < k) {
          const float ls = v[i] - lse;
          ent -= expf(ls) * ls;
        }
      const int a = p.actions ? min(max(load_action(p.actions, p.act_dtype, env * kActHeads + lane), 0), p.k_max - 1) : -1;
      const float glp = g_logprob ? g_logprob[env] : 0.f, gen = g_entropy ? g_entropy[env] : 0.f;
#pragma unroll
      for (int i = 0; i < 7; ++i)
        if (i < k) {
          const float ls = v[i] - lse, pi = expf(ls);
          float g = glp * ((i == a ? 1.f : 0.f) - pi) - gen * pi * (ls + ent);
          if (g_logits) g += g_logits[(env * kActHeads + lane) * p.k_max + i];
          g_raw[env * (int64_t)ldg_raw + p.first[lane] + i] = __float2half_rn(g * scale);
        }
    }
    const float* vr = p.vraw + env * p.ld_v;
    float mx = -INFINITY;
    for (int i = lane; i < p.bins; i += 32) mx = fmaxf(mx, vr[i]);
    mx = warp_max(mx);
    const float step = 2.f * p.vmax / (p.bins - 1);
    float se = 0.f, sc = 0.f;
    for (int i = lane; i < p.bins; i += 32) {
      const float e = expf(vr[i] - mx);
      const float c = i < p.bins / 2 ? -p.vmax + step * i : p.vmax - step * (p.bins - 1 - i);
      se += e;
      sc += e * c;
    }
    se = warp_sum(se);
    sc = warp_sum(sc);
    const float val = sc / se, gv = g_value ? g_value[env] : 0.f;
    for (int i = lane; i < ldg_v; i += 32) {
      float g = 0.f;
      if (i < p.bins) {
        const float c = i < p.bins / 2 ? -p.vmax + step * i : p.vmax - step * (p.bins - 1 - i);
        g = gv * (expf(vr[i] - mx) / se) * (c - val);
        if (g_vlogits) g += g_vlogits[env * p.bins + i];
      }
      g_vraw[env * (int64_t)ldg_v + i] = __float2half_rn(g * scale);
    }
  }
}

int64_t grid_for(int64_t work_items, int per_block) {
  int64_t blocks = (work_items + per_block - 1) / per_block;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : blocks;
}

}  // namespace

int layernorm_bwd(const float* x, int64_t ldx, RowMap xmap, const float* gamma, float eps, const void* gy, int gy_f32,
                  int64_t ldgy, const float* gres, float* gx_out, int64_t ldg, RowMap gmap, float* ggamma, float* gbeta,
                  int64_t rows, int d, cudaStream_t stream, __half* gx16, int64_t ldg16) {
  if (!x || !gamma || !gy || !gx_out) {
    set_error("layernorm_bwd: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (d % 4 != 0 || d > 128 * kMaxVecAll || (ldx % 4) || (ldg % 4) || (ldgy % 4) || (gx16 && (ldg16 % 4))) {
    set_error("layernorm_bwd: d = %d unsupported (d %% 4 == 0, d <= 1024, aligned pitches)", d);
    return BSRL_ERR_SHAPE;
  }
  if (rows == 0) return BSRL_OK;
  const int blocks = (int)grid_for(rows, 8 * 4);
  const size_t smem = 2 * d * sizeof(float);
#define BSRL_LN_BWD(F32, NV) \
  ln_bwd_kernel<F32, NV><<<blocks, 256, smem, stream>>>(x, ldx, xmap, gamma, eps, gy, ldgy, gres, gx_out, ldg, gmap, gx16, ldg16, ggamma, gbeta, rows, d)
  const int nv = (d + 127) / 128;          // float4 per lane actually needed: fewer registers, more rows in flight
  if (gy_f32) {
    if (nv <= 2) BSRL_LN_BWD(true, 2); else if (nv <= 4) BSRL_LN_BWD(true, 4); else BSRL_LN_BWD(true, 8);
  } else {
    if (nv <= 2) BSRL_LN_BWD(false, 2); else if (nv <= 4) BSRL_LN_BWD(false, 4); else BSRL_LN_BWD(false, 8);
  }
#undef BSRL_LN_BWD
  BSRL_LAUNCH_OK("ln_bwd_kernel");
  return BSRL_OK;
}

int colsum16(const __half* in, int64_t ld, int64_t rows, int n, float* out, cudaStream_t stream) {
  if (rows == 0 || n == 0 || !out) return BSRL_OK;
  const int col_blocks = (n + 255) / 256;
  // enough row chunks to fill the machine a few times over, at least 64 rows each
  int64_t chunks = (int64_t)sm_count() * 8 / col_blocks;
  if (chunks < 1) chunks = 1;
  if (chunks > (rows + 63) / 64) chunks = (rows + 63) / 64;
  const int64_t chunk = (rows + chunks - 1) / chunks;
  chunks = (rows + chunk - 1) / chunk;
  const dim3 grid((unsigned)col_blocks, (unsigned)chunks);
  if (n % 8 == 0 && ld % 8 == 0 && aligned16(in)) colsum_kernel<<<grid, 256, 0, stream>>>(in, ld, rows, n, chunk, out);
  else colsum_slow_kernel<<<grid, 256, 0, stream>>>(in, ld, rows, n, chunk, out);
  BSRL_LAUNCH_OK("colsum_kernel");
  return BSRL_OK;
}

int relu_mask16(__half* g, int64_t ldg, const __half* act, int64_t lda, int64_t rows, int n, cudaStream_t stream) {
  if (rows == 0) return BSRL_OK;
  relu_mask_kernel<<<(unsigned)grid_for(rows * (n >> 3), 256), 256, 0, stream>>>(g, ldg, act, lda, rows, n);
  BSRL_LAUNCH_OK("relu_mask_kernel");
  return BSRL_OK;
}

int cast_rows16(const float* in, int64_t ldi, RowMap imap, float scale, __half* out, int64_t ldo, int64_t rows, int n,
                cudaStream_t stream) {
  if (rows == 0) return BSRL_OK;
  cast_rows16_kernel<<<(unsigned)grid_for(rows * (n >> 2), 256), 256, 0, stream>>>(in, ldi, imap, scale, out, ldo, rows, n);
  BSRL_LAUNCH_OK("cast_rows16_kernel");
  return BSRL_OK;
}

int add_rows32(const float* src, int64_t lds, float* dst, int64_t ldd, RowMap dmap, int64_t rows, int n, int accumulate,
               cudaStream_t stream) {
  if (rows == 0) return BSRL_OK;
  add_rows_kernel<<<(unsigned)grid_for(rows * (n >> 2), 256), 256, 0, stream>>>(src, lds, dst, ldd, dmap, rows, n, accumulate);
  BSRL_LAUNCH_OK("add_rows_kernel");
  return BSRL_OK;
}

int transpose16(const __half* in, int64_t ldi, RowMap imap, int64_t rows, int cols, __half* out, int64_t ldo,
                int64_t rows_pad, cudaStream_t stream, float* colsum) {
  if (rows_pad == 0 || cols == 0) return BSRL_OK;
  const int64_t bx = (rows_pad + 63) / 64;
  if (bx > 0x7fffffff) {
    set_error("transpose16: too many rows");
    return BSRL_ERR_SHAPE;
  }
  const dim3 grid((unsigned)bx, (cols + 63) / 64);
  const bool fast = cols % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && rows_pad % 8 == 0 && aligned16(in) && aligned16(out);
  if (fast) transpose16_kernel<<<grid, 256, 0, stream>>>(in, ldi, imap, rows, cols, out, ldo, rows_pad, colsum);
  else transpose16_slow_kernel<<<grid, 256, 0, stream>>>(in, ldi, imap, rows, cols, out, ldo, rows_pad, colsum);
  BSRL_LAUNCH_OK("transpose16_kernel");
  return BSRL_OK;
}

int head_tail_bwd(const HeadTailArgs& a, const float* g_logprob, const float* g_entropy, const float* g_value,
                  const float* g_vlogits, const float* g_logits, float scale, __half* g_raw, int ldg_raw, __half* g_vraw,
                  int ldg_v, cudaStream_t stream) {
  if (!a.raw || !a.vraw || !g_raw || !g_vraw) {
    set_error("head_tail_bwd: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (a.n_envs == 0) return BSRL_OK;
  head_tail_bwd_kernel<<<(unsigned)grid_for(a.n_envs, 8), 256, 0, stream>>>(a, g_logprob, g_entropy, g_value, g_vlogits,
                                                                            g_logits, scale, g_raw, ldg_raw, g_vraw, ldg_v);
  BSRL_LAUNCH_OK("head_tail_bwd_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
