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
    const int64_t env = pair / n_heads;
    const int head = static_cast<int>(pair % n_heads);
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
    const int64_t row = i / per_row;
    const int c = (int)(i % per_row) * 8;
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
