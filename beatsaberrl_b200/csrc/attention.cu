// Masked multi-head self-attention over the tokens of one environment (29 in the reference's layout;
// any count up to 96 for the single-body-token layouts of 17 / 33 / 65 tokens).
//
// One warp owns one (env, head) pair: it stages that head's q, k, v slices (tokens x head_dim
// fp16 each) in its private shared-memory tile, computes a 16-row strip of the score matrix with
// m16n8k16 MMAs, runs the softmax in fp32 on the accumulator fragments (row statistics by
// quad shuffles) and feeds the probabilities straight back as the A operand of the P V MMAs.
// Scores never leave registers.  The additive key bias (0 or -16384) makes masked keys'
// probabilities exactly 0; the pad keys (up to the next multiple of 32) are forced to -inf.
//
// Reference: attn29_fwd_kernel (python/beat_arena_env/csrc/small_attn.cu:228-332) and the
// fp32 arithmetic it is checked against, softmax(q k^T / sqrt(dh) + bias) v
// (python/policy.py:686-690).  The kernel is not tied to (T, d, H) = (29, 192, 4): head_dim
// 32, 48 or 64, any head count.
#include "kernels.cuh"

namespace bsrl {
namespace {
// KG: groups of 32 keys (tokens padded to 32 KG rows: two 16-row MMA tiles / four 8-key tiles per group);
// WARPS: warps per block, fewer where the per-warp tile is large
template <int DH, int KG, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) attn29_kernel(const __half* __restrict__ qkv, int ld,
                                                           const float* __restrict__ key_bias,
                                                           int64_t n_pairs, int tokens, int d, int n_heads,
                                                           int q_first, int n_q,
                                                           __half* __restrict__ out, int ldo) {
  constexpr int kWarps = WARPS, kRows = 32 * KG, NT = 4 * KG;   // NT: 8-key tiles
  constexpr int LDS = DH + 8;          // padded row (halfs): ldmatrix rows land in distinct banks
  constexpr int CH = DH / 8;           // 16-byte chunks per row
  extern __shared__ __align__(16) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __half* sq = reinterpret_cast<__half*>(smem) + (size_t)warp * 3 * kRows * LDS;
  __half* sk = sq + kRows * LDS;
  __half* sv = sk + kRows * LDS;
  const uint32_t sq_u = smem_u32(sq), sk_u = smem_u32(sk), sv_u = smem_u32(sv);
  const float scale = rsqrtf(static_cast<float>(DH));
  const int g = lane >> 2, tig = lane & 3;
  const int m_tiles = (n_q + 15) >> 4;

  for (int64_t pair = (int64_t)blockIdx.x * kWarps + warp; pair < n_pairs;
       pair += (int64_t)gridDim.x * kWarps) {
    int head;
    const int64_t env = div_index(pair, n_heads, &head);
    const __half* base = qkv + env * tokens * (int64_t)ld + head * DH;
    __syncwarp();
    // stage q (query rows), k, v; rows past the live range are zero
    for (int c = lane; c < kRows * CH; c += 32) {
      int row = c / CH, ch = c % CH;
      uint4 zq = make_uint4(0, 0, 0, 0), zk = zq, zv = zq;
      if (row < n_q)
        zq = *reinterpret_cast<const uint4*>(base + (int64_t)(q_first + row) * ld + ch * 8);
      if (row < tokens) {
        const __half* r = base + (int64_t)row * ld + ch * 8;
        zk = *reinterpret_cast<const uint4*>(r + d);
        zv = *reinterpret_cast<const uint4*>(r + 2 * d);
      }
      *reinterpret_cast<uint4*>(sq + row * LDS + ch * 8) = zq;
      *reinterpret_cast<uint4*>(sk + row * LDS + ch * 8) = zk;
      *reinterpret_cast<uint4*>(sv + row * LDS + ch * 8) = zv;
    }
    // key bias of the 8 key columns this lane sees: keys nt*8 + tig*2 + {0,1}
    float kb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        int key = nt * 8 + tig * 2 + e;
        kb[nt][e] = key < tokens ? key_bias[env * tokens + key] : -INFINITY;
      }
    __syncwarp();

    for (int mt = 0; mt < m_tiles; ++mt) {
      float s[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DH / 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, sq_u + ((mt * 16 + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
        for (int j = 0; j < 2 * KG; ++j) {
          uint32_t b[4];
          int row = j * 16 + (lane & 7) + ((lane >> 4) << 3);
          ldmatrix_x4(b, sk_u + (row * LDS + ks * 16 + ((lane >> 3) & 1) * 8) * 2);
          mma_f16(s[2 * j], a, b[0], b[1]);
          mma_f16(s[2 * j + 1], a, b[2], b[3]);
        }
      }
      // softmax over keys for rows g (e = 0,1) and g + 8 (e = 2,3)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] = s[nt][e] * scale + kb[nt][e & 1];
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] = expf(s[nt][e] - mx[e >> 1]);
          sum[e >> 1] += s[nt][e];
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        sum[r] = 1.f / sum[r];
      }
      // P (normalised, fp16) as the A operand of P V
      uint32_t pa[2 * KG][4];
#pragma unroll
      for (int ks = 0; ks < 2 * KG; ++ks) {
        pa[ks][0] = pack_half2(s[2 * ks][0] * sum[0], s[2 * ks][1] * sum[0]);
        pa[ks][1] = pack_half2(s[2 * ks][2] * sum[1], s[2 * ks][3] * sum[1]);
        pa[ks][2] = pack_half2(s[2 * ks + 1][0] * sum[0], s[2 * ks + 1][1] * sum[0]);
        pa[ks][3] = pack_half2(s[2 * ks + 1][2] * sum[1], s[2 * ks + 1][3] * sum[1]);
      }
      float o[DH / 8][4];
#pragma unroll
      for (int nt = 0; nt < DH / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 2 * KG; ++ks) {
#pragma unroll
        for (int j = 0; j < DH / 16; ++j) {
          uint32_t b[4];
          int row = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(b, sv_u + (row * LDS + j * 16 + (lane >> 4) * 8) * 2);
          mma_f16(o[2 * j], pa[ks], b[0], b[1]);
          mma_f16(o[2 * j + 1], pa[ks], b[2], b[3]);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        int qrow = mt * 16 + g + r * 8;
        if (qrow < n_q) {
          __half* orow = out + (env * n_q + qrow) * (int64_t)ldo + head * DH + tig * 2;
#pragma unroll
          for (int nt = 0; nt < DH / 8; ++nt)
            *reinterpret_cast<uint32_t*>(orow + nt * 8) = pack_half2(o[nt][r * 2], o[nt][r * 2 + 1]);
        }
      }
    }
  }
}

// Token counts of the form 1 + 16 k (the single-body-token layouts: 17 / 33 / 65): the object tokens fill
// whole 16-row MMA tiles, and only the body token (row 0 of the env) would force a padded tile on both the
// query and the key side -- at 33 tokens the padded problem is 48 x 64 against 32 x 32, three times the MMAs.
// So the MMAs run over the object tokens alone and the body token is folded in on the CUDA cores:
//   * its key: one extra score column s0[i] = q_i . k_0 (a dot product per query row) joins the row's softmax,
//     and its probability adds p0[i] v_0 to the row's output;
//   * its query row: 1 x tokens scores, a warp-wide softmax and a tokens-long weighted sum of the v rows.
// n_q = tokens (every row) or 1 (the body row only: the last block's readout).  Same arithmetic as
// attn29_kernel: fp32 scores and softmax, masked keys exactly 0, probabilities rounded to fp16 only where
// they enter an MMA.
template <int DH, int NOBJ, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) attn_body_kernel(const __half* __restrict__ qkv, int ld,
                                                              const float* __restrict__ key_bias, int64_t n_pairs,
                                                              int d, int n_heads, int n_q, __half* __restrict__ out, int ldo) {
  constexpr int T = NOBJ + 1, NT = NOBJ / 8, KS = NOBJ / 16, MT = NOBJ / 16;
  constexpr int LDS = DH + 8, CH = DH / 8;
  constexpr int PER = (NOBJ + 31) / 32;              // object rows per lane in the lane-per-row passes
  extern __shared__ __align__(16) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // per warp: q, k, v of the object tokens (NOBJ rows each), then q0 | k0 | v0, then the extra score column
  constexpr int kWarpHalfs = 3 * NOBJ * LDS + 3 * LDS;
  __half* sq = reinterpret_cast<__half*>(smem) + (size_t)warp * kWarpHalfs;
  __half* sk = sq + NOBJ * LDS;
  __half* sv = sk + NOBJ * LDS;
  __half* s0 = sv + NOBJ * LDS;                      // q0 at [0, DH), k0 at [LDS, ..), v0 at [2 LDS, ..)
  float* sx = reinterpret_cast<float*>(smem + (size_t)WARPS * kWarpHalfs * 2) + warp * NOBJ;
  const uint32_t sq_u = smem_u32(sq), sk_u = smem_u32(sk), sv_u = smem_u32(sv);
  const float scale = rsqrtf(static_cast<float>(DH));
  const int g = lane >> 2, tig = lane & 3;
  const bool all_rows = n_q == T;

  for (int64_t pair = (int64_t)blockIdx.x * WARPS + warp; pair < n_pairs; pair += (int64_t)gridDim.x * WARPS) {
    int head;
    const int64_t env = div_index(pair, n_heads, &head);
    const __half* base = qkv + env * T * (int64_t)ld + head * DH;
    __syncwarp();
    for (int c = lane; c < NOBJ * CH; c += 32) {
      const int row = c / CH, ch = c % CH;
      const __half* r = base + (int64_t)(row + 1) * ld + ch * 8;
      if (all_rows) *reinterpret_cast<uint4*>(sq + row * LDS + ch * 8) = *reinterpret_cast<const uint4*>(r);
      *reinterpret_cast<uint4*>(sk + row * LDS + ch * 8) = *reinterpret_cast<const uint4*>(r + d);
      *reinterpret_cast<uint4*>(sv + row * LDS + ch * 8) = *reinterpret_cast<const uint4*>(r + 2 * d);
    }
    if (lane < 3 * CH) {
      const int which = lane / CH, ch = lane % CH;
      *reinterpret_cast<uint4*>(s0 + which * LDS + ch * 8) = *reinterpret_cast<const uint4*>(base + which * d + ch * 8);
    }
    const float kb0 = key_bias[env * T];
    __syncwarp();

    // ---- body query row: lane j scores object keys j, j + 32
    {
      float sc[PER], s00 = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) sc[i] = 0.f;
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        const uint4 qv = *reinterpret_cast<const uint4*>(s0 + ch * 8);
        const uint4 k0v = *reinterpret_cast<const uint4*>(s0 + LDS + ch * 8);
        const __half2* qh = reinterpret_cast<const __half2*>(&qv);
        const __half2* k0h = reinterpret_cast<const __half2*>(&k0v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = __half22float2(qh[e]), b = __half22float2(k0h[e]);
          s00 = fmaf(a.x, b.x, fmaf(a.y, b.y, s00));
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          const int j = lane + 32 * i;
          if (j < NOBJ) {
            const uint4 kv = *reinterpret_cast<const uint4*>(sk + j * LDS + ch * 8);
            const __half2* kh = reinterpret_cast<const __half2*>(&kv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 a = __half22float2(qh[e]), b = __half22float2(kh[e]);
              sc[i] = fmaf(a.x, b.x, fmaf(a.y, b.y, sc[i]));
            }
          }
        }
      }
      s00 = s00 * scale + kb0;
      float mx = s00;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int j = lane + 32 * i;
        sc[i] = j < NOBJ ? sc[i] * scale + key_bias[env * T + 1 + j] : -INFINITY;
        mx = fmaxf(mx, sc[i]);
      }
      mx = warp_max(mx);
      const float p00 = expf(s00 - mx);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        sc[i] = expf(sc[i] - mx);              // exp(-inf) = 0 for the lanes past NOBJ
        sum += sc[i];
      }
      sum = warp_sum(sum) + p00;
      const float inv = 1.f / sum;
      // o0[c] = p00 v0[c] + sum_j p_j v_j[c]; lane owns columns lane, lane + 32
      constexpr int CPL = (DH + 31) / 32;
      float o[CPL];
#pragma unroll
      for (int u = 0; u < CPL; ++u) {
        const int c = lane + 32 * u;
        o[u] = c < DH ? p00 * __half2float(s0[2 * LDS + c]) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < PER; ++i) {
#pragma unroll 8
        for (int jj = 0; jj < 32; ++jj) {
          const int j = jj + 32 * i;
          if (j >= NOBJ) break;
          const float pj = __shfl_sync(0xffffffffu, sc[i], jj);
#pragma unroll
          for (int u = 0; u < CPL; ++u) {
            const int c = lane + 32 * u;
            if (c < DH) o[u] = fmaf(pj, __half2float(sv[j * LDS + c]), o[u]);
          }
        }
      }
      __half* orow = out + env * n_q * (int64_t)ldo + head * DH;
#pragma unroll
      for (int u = 0; u < CPL; ++u) {
        const int c = lane + 32 * u;
        if (c < DH) orow[c] = __float2half_rn(o[u] * inv);
      }
    }
    if (!all_rows) continue;

    // ---- extra score column of the object rows: sx[i] = q_i . k_0 (raw)
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int r = lane + 32 * i;
      if (r < NOBJ) {
        float acc = 0.f;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
          const uint4 qv = *reinterpret_cast<const uint4*>(sq + r * LDS + ch * 8);
          const uint4 k0v = *reinterpret_cast<const uint4*>(s0 + LDS + ch * 8);
          const __half2* qh = reinterpret_cast<const __half2*>(&qv);
          const __half2* k0h = reinterpret_cast<const __half2*>(&k0v);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a = __half22float2(qh[e]), b = __half22float2(k0h[e]);
            acc = fmaf(a.x, b.x, fmaf(a.y, b.y, acc));
          }
        }
        sx[r] = acc;
      }
    }
    float kb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) kb[nt][e] = key_bias[env * T + 1 + nt * 8 + tig * 2 + e];
    __syncwarp();

    // ---- object query rows against the object keys on the tensor cores
#pragma unroll 1
    for (int mt = 0; mt < MT; ++mt) {
      float s[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DH / 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, sq_u + ((mt * 16 + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
        for (int j = 0; j < NT / 2; ++j) {
          uint32_t b[4];
          const int row = j * 16 + (lane & 7) + ((lane >> 4) << 3);
          ldmatrix_x4(b, sk_u + (row * LDS + ks * 16 + ((lane >> 3) & 1) * 8) * 2);
          mma_f16(s[2 * j], a, b[0], b[1]);
          mma_f16(s[2 * j + 1], a, b[2], b[3]);
        }
      }
      float x0[2], mx[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        x0[r] = sx[mt * 16 + g + r * 8] * scale + kb0;
        mx[r] = x0[r];
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] = s[nt][e] * scale + kb[nt][e & 1];
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] = expf(s[nt][e] - mx[e >> 1]);
          sum[e >> 1] += s[nt][e];
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        x0[r] = expf(x0[r] - mx[r]);                 // the body key's share, the same for the four lanes of a row
        sum[r] = 1.f / (sum[r] + x0[r]);
        x0[r] *= sum[r];
      }
      uint32_t pa[KS][4];
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        pa[ks][0] = pack_half2(s[2 * ks][0] * sum[0], s[2 * ks][1] * sum[0]);
        pa[ks][1] = pack_half2(s[2 * ks][2] * sum[1], s[2 * ks][3] * sum[1]);
        pa[ks][2] = pack_half2(s[2 * ks + 1][0] * sum[0], s[2 * ks + 1][1] * sum[0]);
        pa[ks][3] = pack_half2(s[2 * ks + 1][2] * sum[1], s[2 * ks + 1][3] * sum[1]);
      }
      float o[DH / 8][4];
#pragma unroll
      for (int nt = 0; nt < DH / 8; ++nt) {           // start from the body token's contribution p0 v_0
        const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(s0 + 2 * LDS + nt * 8 + tig * 2));
        o[nt][0] = x0[0] * v0.x; o[nt][1] = x0[0] * v0.y;
        o[nt][2] = x0[1] * v0.x; o[nt][3] = x0[1] * v0.y;
      }
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int j = 0; j < DH / 16; ++j) {
          uint32_t b[4];
          const int row = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(b, sv_u + (row * LDS + j * 16 + (lane >> 4) * 8) * 2);
          mma_f16(o[2 * j], pa[ks], b[0], b[1]);
          mma_f16(o[2 * j + 1], pa[ks], b[2], b[3]);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int token = 1 + mt * 16 + g + r * 8;
        __half* orow = out + (env * T + token) * (int64_t)ldo + head * DH + tig * 2;
#pragma unroll
        for (int nt = 0; nt < DH / 8; ++nt)
          *reinterpret_cast<uint32_t*>(orow + nt * 8) = pack_half2(o[nt][r * 2], o[nt][r * 2 + 1]);
      }
    }
  }
}

template <int DH, int NOBJ>
int launch_body(const __half* qkv, int ld, const float* key_bias, int64_t n_envs, int d, int n_heads, int n_q, __half* out,
                int ldo, cudaStream_t stream) {
  constexpr int kWarps = NOBJ <= 32 ? 8 : 4;
  constexpr int smem = kWarps * ((3 * NOBJ + 3) * (DH + 8) * 2 + NOBJ * 4);
  static DeviceOnce once;
  int rc = once.run("attn_body_kernel set-up", [] {
    return cudaFuncSetAttribute(attn_body_kernel<DH, NOBJ, kWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (rc != BSRL_OK) return rc;
  const int64_t pairs = n_envs * n_heads;
  int64_t blocks = (pairs + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  attn_body_kernel<DH, NOBJ, kWarps><<<static_cast<unsigned>(blocks), kWarps * 32, smem, stream>>>(qkv, ld, key_bias, pairs, d,
                                                                                                n_heads, n_q, out, ldo);
  BSRL_LAUNCH_OK("attn_body_kernel");
  return BSRL_OK;
}
template <int DH>
int launch_body_n(const __half* qkv, int ld, const float* key_bias, int64_t n_envs, int tokens, int d, int n_heads, int n_q,
                  __half* out, int ldo, cudaStream_t stream) {
  if (tokens == 17) return launch_body<DH, 16>(qkv, ld, key_bias, n_envs, d, n_heads, n_q, out, ldo, stream);
  if (tokens == 33) return launch_body<DH, 32>(qkv, ld, key_bias, n_envs, d, n_heads, n_q, out, ldo, stream);
  return launch_body<DH, 64>(qkv, ld, key_bias, n_envs, d, n_heads, n_q, out, ldo, stream);
}

template <int DH, int KG>
int launch(const __half* qkv, int ld, const float* key_bias, int64_t n_envs, int tokens, int d, int n_heads,
           int q_first, int n_q, __half* out, int ldo, cudaStream_t stream) {
  constexpr int kWarps = KG == 1 ? 8 : 4;
  constexpr int smem = kWarps * 3 * (32 * KG) * (DH + 8) * 2;
  static DeviceOnce once;
  int rc = once.run("attn29_kernel set-up", [] {
    return cudaFuncSetAttribute(attn29_kernel<DH, KG, kWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (rc != BSRL_OK) return rc;
  int64_t pairs = n_envs * n_heads;
  int64_t blocks = (pairs + kWarps - 1) / kWarps;
  int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  attn29_kernel<DH, KG, kWarps><<<static_cast<unsigned>(blocks), kWarps * 32, smem, stream>>>(
      qkv, ld, key_bias, pairs, tokens, d, n_heads, q_first, n_q, out, ldo);
  BSRL_LAUNCH_OK("attn29_kernel");
  return BSRL_OK;
}
template <int DH>
int launch_kg(const __half* qkv, int ld, const float* key_bias, int64_t n_envs, int tokens, int d, int n_heads,
              int q_first, int n_q, __half* out, int ldo, cudaStream_t stream) {
  if (tokens <= 32) return launch<DH, 1>(qkv, ld, key_bias, n_envs, tokens, d, n_heads, q_first, n_q, out, ldo, stream);
  if (tokens <= 64) return launch<DH, 2>(qkv, ld, key_bias, n_envs, tokens, d, n_heads, q_first, n_q, out, ldo, stream);
  return launch<DH, 3>(qkv, ld, key_bias, n_envs, tokens, d, n_heads, q_first, n_q, out, ldo, stream);
}
}  // namespace

int attention29(const __half* qkv, int ld_qkv, const float* key_bias, int64_t n_envs, int d,
                int n_heads, int q_first, int n_q, __half* out, int ldo, cudaStream_t stream) {
  return attention_tokens(qkv, ld_qkv, key_bias, n_envs, kT, d, n_heads, q_first, n_q, out, ldo, stream);
}

int attention_tokens(const __half* qkv, int ld_qkv, const float* key_bias, int64_t n_envs, int tokens, int d,
                     int n_heads, int q_first, int n_q, __half* out, int ldo, cudaStream_t stream) {
  if (!qkv || !key_bias || !out) {
    set_error("attention: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (tokens < 1 || tokens > 96) {
    set_error("attention: %d tokens per env unsupported (1..96)", tokens);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (n_envs < 0 || n_heads <= 0 || d % n_heads != 0 || q_first < 0 || n_q < 1 ||
      q_first + n_q > tokens || ld_qkv < 3 * d || ldo < d) {
    set_error("attention: bad shape d=%d heads=%d q=[%d,%d)", d, n_heads, q_first, q_first + n_q);
    return BSRL_ERR_SHAPE;
  }
  if (!aligned16(qkv) || !aligned16(out) || (ld_qkv % 8) || (ldo % 8) || (d % 8)) {
    set_error("attention: buffers must be 16-byte aligned, leading dimensions %% 8 == 0");
    return BSRL_ERR_ALIGN;
  }
  if (n_envs == 0) return BSRL_OK;
  const int dh = d / n_heads;
  // one body token + 16 / 32 / 64 object tokens, all rows or the body row only: the body token off the MMA tiles
  if ((tokens == 17 || tokens == 33 || tokens == 65) && q_first == 0 && (n_q == tokens || n_q == 1)) {
    if (dh == 32) return launch_body_n<32>(qkv, ld_qkv, key_bias, n_envs, tokens, d, n_heads, n_q, out, ldo, stream);
    if (dh == 64) return launch_body_n<64>(qkv, ld_qkv, key_bias, n_envs, tokens, d, n_heads, n_q, out, ldo, stream);
  }
  if (dh == 32) return launch_kg<32>(qkv, ld_qkv, key_bias, n_envs, tokens, d, n_heads, q_first, n_q, out, ldo, stream);
  if (dh == 48) return launch_kg<48>(qkv, ld_qkv, key_bias, n_envs, tokens, d, n_heads, q_first, n_q, out, ldo, stream);
  if (dh == 64) return launch_kg<64>(qkv, ld_qkv, key_bias, n_envs, tokens, d, n_heads, q_first, n_q, out, ldo, stream);
  set_error("attention: head_dim %d unsupported (32, 48 or 64)", dh);
  return BSRL_ERR_UNSUPPORTED;
}

// Value residual on the unfused path (python/policy.py:604-615, _VMix): the v columns of the packed
// projection are copied out as the block's own values (v_out) and / or replaced by
// vres[0] * v + vres[1] * v0 (fp32 arithmetic, rounded once).  8 columns per thread.
namespace {
__global__ void vres_mix_kernel(__half* __restrict__ v, int ld, int64_t rows, int d,
                                __half* __restrict__ v_out, const __half* __restrict__ v0,
                                const float* __restrict__ vres) {
  const float a = vres ? vres[0] : 1.f, b = vres ? vres[1] : 0.f;
  const int per_row = d >> 3;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (int64_t)gridDim.x * blockDim.x) {
    int piece;
    const int64_t row = div_index(i, per_row, &piece);
    const int c = piece * 8;
    uint4 w = *reinterpret_cast<const uint4*>(v + row * ld + c);
    if (v_out) *reinterpret_cast<uint4*>(v_out + row * d + c) = w;
    if (v0) {
      const uint4 o = *reinterpret_cast<const uint4*>(v0 + row * d + c);
      uint32_t ww[4] = {w.x, w.y, w.z, w.w};
      const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&ww[e]));
        const float2 y = __half22float2(*reinterpret_cast<const __half2*>(&ow[e]));
        ww[e] = pack_half2(fmaf(a, x.x, b * y.x), fmaf(a, x.y, b * y.y));
      }
      *reinterpret_cast<uint4*>(v + row * ld + c) = make_uint4(ww[0], ww[1], ww[2], ww[3]);
    }
  }
}
}  // namespace

int vres_mix(__half* v, int ld, int64_t rows, int d, __half* v_out, const __half* v0, const float* vres,
             cudaStream_t stream) {
  if (!v || (v0 && !vres)) {
    set_error("vres_mix: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (!aligned16(v) || (ld % 8) || (d % 8) || (v_out && !aligned16(v_out)) || (v0 && !aligned16(v0))) {
    set_error("vres_mix: buffers must be 16-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  if (rows == 0 || (!v_out && !v0)) return BSRL_OK;
  int64_t blocks = (rows * (d >> 3) + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  vres_mix_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(v, ld, rows, d, v_out, v0, vres);
  BSRL_LAUNCH_OK("vres_mix_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
