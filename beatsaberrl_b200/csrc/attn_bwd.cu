// Backward of the masked 29-key attention, one warp per (env, head).
//
//   S = q k^T / sqrt(dh) + key_bias,  P = softmax(S),  O = P v            (forward, recomputed here)
//   dV = P^T dO;  dP = dO v^T;  dS = P (dP - rowsum(P dP));  dQ = dS k / sqrt(dh);  dK = dS^T q / sqrt(dh)
//
// q, k, v come from the packed projection (rows of 3d fp16: [q | k | v]); dO and the three outputs are
// fp16 rows carrying the caller's loss scale.  The probabilities are recomputed in fp32 from q and k, as
// attn29_bwd_kernel of the reference does (python/beat_arena_env/csrc/small_attn.cu:345-463).  The whole
// problem of one (env, head) pair -- at most 29 x 64 values per matrix -- lives in shared memory; the
// arithmetic is plain fp32 FMAs (2 % of the update's FLOPs).
#include "kernels.cuh"

namespace bsrl {
namespace {

constexpr int kWarps = 4;
constexpr int kKeys = 32;      // 29 keys padded to the warp width

template <int DH>
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_kernel(const __half* __restrict__ qkv, int ld, const float* __restrict__ key_bias,
                                                               int64_t n_pairs, int d, int n_heads, int q_first, int n_q,
                                                               const __half* __restrict__ g_out, int ldgo, __half* __restrict__ gq,
                                                               int ldq, __half* __restrict__ gk, int ldk, __half* __restrict__ gv,
                                                               int ldv) {
  constexpr int PITCH = DH + 2;                       // halves per row: an odd number of 32-bit words
  constexpr int PER_WARP = 4 * kT * PITCH * 2 + 2 * kT * kKeys * 4;
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* mine = smem + warp * PER_WARP;
  __half* sQ = reinterpret_cast<__half*>(mine);
  __half* sK = sQ + kT * PITCH;
  __half* sV = sK + kT * PITCH;
  __half* sG = sV + kT * PITCH;
  float* sP = reinterpret_cast<float*>(sG + kT * PITCH);
  float* sD = sP + kT * kKeys;
  const float scale = rsqrtf((float)DH);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  for (int64_t pair = (int64_t)blockIdx.x * kWarps + warp; pair < n_pairs; pair += warps) {
    const int64_t env = pair / n_heads;
    const int head = (int)(pair % n_heads);
    const __half* base = qkv + env * kT * (int64_t)ld + head * DH;
    __syncwarp();
    // stage q (query rows only), k, v, dO: pairs of halves, coalesced along the head's columns
    for (int i = lane; i < kT * (DH / 2); i += 32) {
      const int r = i / (DH / 2), c = (i % (DH / 2)) * 2;
      *reinterpret_cast<__half2*>(sK + r * PITCH + c) = *reinterpret_cast<const __half2*>(base + (int64_t)r * ld + d + c);
      *reinterpret_cast<__half2*>(sV + r * PITCH + c) = *reinterpret_cast<const __half2*>(base + (int64_t)r * ld + 2 * d + c);
      if (r < n_q) {
        *reinterpret_cast<__half2*>(sQ + r * PITCH + c) = *reinterpret_cast<const __half2*>(base + (int64_t)(q_first + r) * ld + c);
        *reinterpret_cast<__half2*>(sG + r * PITCH + c) =
            *reinterpret_cast<const __half2*>(g_out + (env * n_q + r) * (int64_t)ldgo + head * DH + c);
      }
    }
    __syncwarp();
    const float kb = lane < kT ? key_bias[env * kT + lane] : -INFINITY;
    // P and dS, lane = key
    for (int i = 0; i < n_q; ++i) {
      float s = 0.f, dp = 0.f;
      if (lane < kT) {
#pragma unroll 8
        for (int c = 0; c < DH; c += 2) {
          const float2 q = __half22float2(*reinterpret_cast<const __half2*>(sQ + i * PITCH + c));
          const float2 k = __half22float2(*reinterpret_cast<const __half2*>(sK + lane * PITCH + c));
          const float2 g = __half22float2(*reinterpret_cast<const __half2*>(sG + i * PITCH + c));
          const float2 v = __half22float2(*reinterpret_cast<const __half2*>(sV + lane * PITCH + c));
          s = fmaf(q.x, k.x, fmaf(q.y, k.y, s));
          dp = fmaf(g.x, v.x, fmaf(g.y, v.y, dp));
        }
      }
      s = lane < kT ? fmaf(s, scale, kb) : -INFINITY;
      const float mx = warp_max(s);
      const float e = lane < kT ? expf(s - mx) : 0.f;
      const float p = e / warp_sum(e);
      const float dot = warp_sum(p * dp);
      sP[i * kKeys + lane] = p;
      sD[i * kKeys + lane] = p * (dp - dot) * scale;        // dS with the 1 / sqrt(dh) of dQ and dK folded in
    }
    __syncwarp();
    // dV, dK (rows = keys) and dQ (rows = queries), lane = column pair
    for (int c = lane * 2; c < DH; c += 64) {
      for (int j = 0; j < kT; ++j) {
        float2 av = make_float2(0.f, 0.f), ak = make_float2(0.f, 0.f);
        for (int i = 0; i < n_q; ++i) {
          const float p = sP[i * kKeys + j], ds = sD[i * kKeys + j];
          const float2 g = __half22float2(*reinterpret_cast<const __half2*>(sG + i * PITCH + c));
          const float2 q = __half22float2(*reinterpret_cast<const __half2*>(sQ + i * PITCH + c));
          av.x = fmaf(p, g.x, av.x); av.y = fmaf(p, g.y, av.y);
          ak.x = fmaf(ds, q.x, ak.x); ak.y = fmaf(ds, q.y, ak.y);
        }
        const int64_t row = env * kT + j;
        *reinterpret_cast<__half2*>(gv + row * ldv + head * DH + c) = __floats2half2_rn(av.x, av.y);
        *reinterpret_cast<__half2*>(gk + row * ldk + head * DH + c) = __floats2half2_rn(ak.x, ak.y);
      }
      for (int i = 0; i < n_q; ++i) {
        float2 aq = make_float2(0.f, 0.f);
        for (int j = 0; j < kT; ++j) {
          const float ds = sD[i * kKeys + j];
          const float2 k = __half22float2(*reinterpret_cast<const __half2*>(sK + j * PITCH + c));
          aq.x = fmaf(ds, k.x, aq.x); aq.y = fmaf(ds, k.y, aq.y);
        }
        *reinterpret_cast<__half2*>(gq + (env * n_q + i) * (int64_t)ldq + head * DH + c) = __floats2half2_rn(aq.x, aq.y);
      }
    }
  }
}

template <int DH>
int launch(const __half* qkv, int ld, const float* key_bias, int64_t n_envs, int d, int n_heads, int q_first, int n_q,
           const __half* g_out, int ldgo, __half* gq, int ldq, __half* gk, int ldk, __half* gv, int ldv, cudaStream_t stream) {
  constexpr int smem = kWarps * (4 * kT * (DH + 2) * 2 + 2 * kT * kKeys * 4);
  static DeviceOnce once;
  int rc = once.run("attn_bwd_kernel set-up", [] {
    return cudaFuncSetAttribute(attn_bwd_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (rc != BSRL_OK) return rc;
  const int64_t pairs = n_envs * n_heads;
  int64_t blocks = (pairs + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  attn_bwd_kernel<DH><<<(unsigned)blocks, kWarps * 32, smem, stream>>>(qkv, ld, key_bias, pairs, d, n_heads, q_first, n_q, g_out,
                                                                      ldgo, gq, ldq, gk, ldk, gv, ldv);
  BSRL_LAUNCH_OK("attn_bwd_kernel");
  return BSRL_OK;
}
}  // namespace

int attention29_bwd(const __half* qkv, int ld_qkv, const float* key_bias, int64_t n_envs, int d, int n_heads, int q_first,
                    int n_q, const __half* g_out, int ldgo, __half* gq, int ldq, __half* gk, int ldk, __half* gv, int ldv,
                    cudaStream_t stream) {
  if (!qkv || !key_bias || !g_out || !gq || !gk || !gv) {
    set_error("attention_bwd: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (n_heads < 1 || d % n_heads != 0 || q_first < 0 || n_q < 1 || q_first + n_q > kT || (ld_qkv % 2) || (ldgo % 2) ||
      (ldq % 2) || (ldk % 2) || (ldv % 2)) {
    set_error("attention_bwd: bad shape d=%d heads=%d q_first=%d n_q=%d", d, n_heads, q_first, n_q);
    return BSRL_ERR_SHAPE;
  }
  if (n_envs == 0) return BSRL_OK;
  switch (d / n_heads) {
    case 32: return launch<32>(qkv, ld_qkv, key_bias, n_envs, d, n_heads, q_first, n_q, g_out, ldgo, gq, ldq, gk, ldk, gv, ldv, stream);
    case 48: return launch<48>(qkv, ld_qkv, key_bias, n_envs, d, n_heads, q_first, n_q, g_out, ldgo, gq, ldq, gk, ldk, gv, ldv, stream);
    case 64: return launch<64>(qkv, ld_qkv, key_bias, n_envs, d, n_heads, q_first, n_q, g_out, ldgo, gq, ldq, gk, ldk, gv, ldv, stream);
    default:
      set_error("attention_bwd: head_dim %d unsupported (32, 48 or 64)", d / n_heads);
      return BSRL_ERR_UNSUPPORTED;
  }
}

}  // namespace bsrl
