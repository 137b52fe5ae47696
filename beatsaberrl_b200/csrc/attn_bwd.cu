// Backward of the masked 29-key attention, one warp per (env, head).
//
//   S = q k^T / sqrt(dh) + key_bias,  P = softmax(S),  O = P v            (forward, recomputed here)
//   dV = P^T dO;  dP = dO v^T;  dS = P (dP - rowsum(P dP));  dQ = dS k / sqrt(dh);  dK = dS^T q / sqrt(dh)
//
// q, k, v come from the packed projection (rows of 3d fp16: [q | k | v]); dO and the three outputs are
// fp16 rows carrying the caller's loss scale.  The probabilities are recomputed in fp32 from q and k, as
// attn29_bwd_kernel of the reference does (python/beat_arena_env/csrc/small_attn.cu:345-463).  The whole
// problem of one (env, head) pair -- at most 32 x 64 values per matrix -- lives in the warp's shared-memory
// tile; the five products run on m16n8k16 MMAs with fp32 accumulation, P and dS rounded to fp16 as operands.
#include "kernels.cuh"

namespace bsrl {
namespace {

constexpr int kWarps = 4;
constexpr int kKeys = 32;      // 29 keys padded to four 8-key MMA tiles
constexpr int LDP = kKeys + 8; // row pitch (halves) of the P / dS tiles

// One warp per (env, head); MT = 16-row query tiles (2: all 29 queries, 1: the lead rows or the critic's one).
// Five small products on m16n8k16 MMAs: S = q k^T and dP = dO v^T (A rows = queries, B rows = keys);
// dQ = dS k (A = dS from the accumulator registers, B = k with the keys as the reduction dimension);
// dV = P^T dO and dK = dS^T q (A = the transposed P / dS tile, fetched from shared memory with
// ldmatrix.trans; B = dO / q with the queries as the reduction dimension).
template <int DH, int MT>
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_kernel(const __half* __restrict__ qkv, int ld, const float* __restrict__ key_bias,
                                                               int64_t n_pairs, int d, int n_heads, int q_first, int n_q,
                                                               const __half* __restrict__ g_out, int ldgo, __half* __restrict__ gq,
                                                               int ldq, __half* __restrict__ gk, int ldk, __half* __restrict__ gv,
                                                               int ldv) {
  constexpr int LDS = DH + 8;                         // padded row (halves): ldmatrix rows land in distinct banks
  constexpr int CH = DH / 8;
  constexpr int QR = 16 * MT;                         // staged query rows
  constexpr int PER_WARP = (2 * QR + 2 * kKeys) * LDS * 2 + 2 * QR * LDP * 2;
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __half* sq = reinterpret_cast<__half*>(smem + (size_t)warp * PER_WARP);
  __half* sg = sq + QR * LDS;
  __half* sk = sg + QR * LDS;
  __half* sv = sk + kKeys * LDS;
  __half* sp = sv + kKeys * LDS;                      // P  [query][key]
  __half* sd = sp + QR * LDP;                         // dS [query][key]
  const uint32_t sq_u = smem_u32(sq), sg_u = smem_u32(sg), sk_u = smem_u32(sk), sv_u = smem_u32(sv), sp_u = smem_u32(sp),
                 sd_u = smem_u32(sd);
  const float scale = rsqrtf((float)DH);
  const int g = lane >> 2, tig = lane & 3;
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  for (int64_t pair = (int64_t)blockIdx.x * kWarps + warp; pair < n_pairs; pair += warps) {
    int head;
    const int64_t env = div_index(pair, n_heads, &head);
    const __half* base = qkv + env * kT * (int64_t)ld + head * DH;
    __syncwarp();
    // stage q, dO (query rows) and k, v (key rows); rows past the live range are zero
    for (int c = lane; c < kKeys * CH; c += 32) {
      const int row = c / CH, ch = c % CH;
      uint4 zk = make_uint4(0, 0, 0, 0), zv = zk, zq = zk, zg = zk;
      if (row < kT) {
        const __half* r = base + (int64_t)row * ld + ch * 8;
        zk = *reinterpret_cast<const uint4*>(r + d);
        zv = *reinterpret_cast<const uint4*>(r + 2 * d);
      }
      if (row < n_q) {
        zq = *reinterpret_cast<const uint4*>(base + (int64_t)(q_first + row) * ld + ch * 8);
        zg = *reinterpret_cast<const uint4*>(g_out + (env * n_q + row) * (int64_t)ldgo + head * DH + ch * 8);
      }
      *reinterpret_cast<uint4*>(sk + row * LDS + ch * 8) = zk;
      *reinterpret_cast<uint4*>(sv + row * LDS + ch * 8) = zv;
      if (row < QR) {
        *reinterpret_cast<uint4*>(sq + row * LDS + ch * 8) = zq;
        *reinterpret_cast<uint4*>(sg + row * LDS + ch * 8) = zg;
      }
    }
    float kb[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = nt * 8 + tig * 2 + e;
        kb[nt][e] = key < kT ? key_bias[env * kT + key] : -INFINITY;
      }
    __syncwarp();

#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      // ---- S = q k^T and dP = dO v^T for this query tile
      float s[4][4], dp[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = dp[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DH / 16; ++ks) {
        uint32_t a[4], ag[4];
        const uint32_t aoff = ((mt * 16 + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8) * 2;
        ldmatrix_x4(a, sq_u + aoff);
        ldmatrix_x4(ag, sg_u + aoff);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t b[4], bv[4];
          const int row = j * 16 + (lane & 7) + ((lane >> 4) << 3);
          const uint32_t boff = (row * LDS + ks * 16 + ((lane >> 3) & 1) * 8) * 2;
          ldmatrix_x4(b, sk_u + boff);
          ldmatrix_x4(bv, sv_u + boff);
          mma_f16(s[2 * j], a, b[0], b[1]);
          mma_f16(s[2 * j + 1], a, b[2], b[3]);
          mma_f16(dp[2 * j], ag, bv[0], bv[1]);
          mma_f16(dp[2 * j + 1], ag, bv[2], bv[3]);
        }
      }
      // ---- P = softmax(S / sqrt(dh) + bias), dS = P (dP - rowsum(P dP)) / sqrt(dh); rows g (e = 0, 1) and g + 8 (e = 2, 3)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
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
      for (int nt = 0; nt < 4; ++nt)
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
      float dot[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] *= sum[e >> 1];                       // P
          dot[e >> 1] += s[nt][e] * dp[nt][e];
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], 1);
        dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], 2);
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) dp[nt][e] = s[nt][e] * (dp[nt][e] - dot[e >> 1]) * scale;   // dS
      // P and dS tiles to shared memory ([query][key] fp16) for the two transposed products
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int off = (mt * 16 + g + r * 8) * LDP + nt * 8 + tig * 2;
          *reinterpret_cast<uint32_t*>(sp + off) = pack_half2(s[nt][2 * r], s[nt][2 * r + 1]);
          *reinterpret_cast<uint32_t*>(sd + off) = pack_half2(dp[nt][2 * r], dp[nt][2 * r + 1]);
        }
      // ---- dQ = dS k: A = dS from the accumulator registers (as P feeds P v in the forward)
      uint32_t da[2][4];
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        da[ks][0] = pack_half2(dp[2 * ks][0], dp[2 * ks][1]);
        da[ks][1] = pack_half2(dp[2 * ks][2], dp[2 * ks][3]);
        da[ks][2] = pack_half2(dp[2 * ks + 1][0], dp[2 * ks + 1][1]);
        da[ks][3] = pack_half2(dp[2 * ks + 1][2], dp[2 * ks + 1][3]);
      }
      float oq[DH / 8][4];
#pragma unroll
      for (int nt = 0; nt < DH / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) oq[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int j = 0; j < DH / 16; ++j) {
          uint32_t b[4];
          const int row = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(b, sk_u + (row * LDS + j * 16 + (lane >> 4) * 8) * 2);
          mma_f16(oq[2 * j], da[ks], b[0], b[1]);
          mma_f16(oq[2 * j + 1], da[ks], b[2], b[3]);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int qrow = mt * 16 + g + r * 8;
        if (qrow < n_q) {
          __half* orow = gq + (env * n_q + qrow) * (int64_t)ldq + head * DH + tig * 2;
#pragma unroll
          for (int nt = 0; nt < DH / 8; ++nt) *reinterpret_cast<uint32_t*>(orow + nt * 8) = pack_half2(oq[nt][r * 2], oq[nt][r * 2 + 1]);
        }
      }
    }
    __syncwarp();
    // ---- dV = P^T dO and dK = dS^T q: key tiles as rows, the queries as the reduction dimension
#pragma unroll
    for (int kt = 0; kt < 2; ++kt) {
      float ov[DH / 8][4], ok[DH / 8][4];
#pragma unroll
      for (int nt = 0; nt < DH / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) ov[nt][e] = ok[nt][e] = 0.f;
#pragma unroll
      for (int qs = 0; qs < MT; ++qs) {                 // 16 queries per step
        // A fragment (16 keys x 16 queries) of the transposed tile: matrix m of the x4 load covers
        // keys kt * 16 + (m & 1) * 8 .., queries qs * 16 + (m >> 1) * 8 ..; lane l supplies query row l & 7 of matrix l >> 3
        uint32_t ap[4], ad[4];
        const int m = lane >> 3;
        const uint32_t toff = ((qs * 16 + (m >> 1) * 8 + (lane & 7)) * LDP + kt * 16 + (m & 1) * 8) * 2;
        ldmatrix_x4_trans(ap, sp_u + toff);
        ldmatrix_x4_trans(ad, sd_u + toff);
#pragma unroll
        for (int j = 0; j < DH / 16; ++j) {
          uint32_t b[4], bq[4];
          const int row = qs * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const uint32_t boff = (row * LDS + j * 16 + (lane >> 4) * 8) * 2;
          ldmatrix_x4_trans(b, sg_u + boff);
          ldmatrix_x4_trans(bq, sq_u + boff);
          mma_f16(ov[2 * j], ap, b[0], b[1]);
          mma_f16(ov[2 * j + 1], ap, b[2], b[3]);
          mma_f16(ok[2 * j], ad, bq[0], bq[1]);
          mma_f16(ok[2 * j + 1], ad, bq[2], bq[3]);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int key = kt * 16 + g + r * 8;
        if (key < kT) {
          const int64_t row = env * kT + key;
          __half* vrow = gv + row * ldv + head * DH + tig * 2;
          __half* krow = gk + row * ldk + head * DH + tig * 2;
#pragma unroll
          for (int nt = 0; nt < DH / 8; ++nt) {
            *reinterpret_cast<uint32_t*>(vrow + nt * 8) = pack_half2(ov[nt][r * 2], ov[nt][r * 2 + 1]);
            *reinterpret_cast<uint32_t*>(krow + nt * 8) = pack_half2(ok[nt][r * 2], ok[nt][r * 2 + 1]);
          }
        }
      }
    }
  }
}

template <int DH, int MT>
int launch(const __half* qkv, int ld, const float* key_bias, int64_t n_envs, int d, int n_heads, int q_first, int n_q,
           const __half* g_out, int ldgo, __half* gq, int ldq, __half* gk, int ldk, __half* gv, int ldv, cudaStream_t stream) {
  constexpr int smem = kWarps * ((2 * 16 * MT + 2 * kKeys) * (DH + 8) * 2 + 2 * 16 * MT * LDP * 2);
  static DeviceOnce once;
  int rc = once.run("attn_bwd_kernel set-up", [] {
    return cudaFuncSetAttribute(attn_bwd_kernel<DH, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (rc != BSRL_OK) return rc;
  const int64_t pairs = n_envs * n_heads;
  int64_t blocks = (pairs + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  attn_bwd_kernel<DH, MT><<<(unsigned)blocks, kWarps * 32, smem, stream>>>(qkv, ld, key_bias, pairs, d, n_heads, q_first, n_q, g_out,
                                                                          ldgo, gq, ldq, gk, ldk, gv, ldv);
  BSRL_LAUNCH_OK("attn_bwd_kernel");
  return BSRL_OK;
}
template <int DH>
int launch_mt(const __half* qkv, int ld, const float* key_bias, int64_t n_envs, int d, int n_heads, int q_first, int n_q,
              const __half* g_out, int ldgo, __half* gq, int ldq, __half* gk, int ldk, __half* gv, int ldv, cudaStream_t stream) {
  if (n_q > 16) return launch<DH, 2>(qkv, ld, key_bias, n_envs, d, n_heads, q_first, n_q, g_out, ldgo, gq, ldq, gk, ldk, gv, ldv, stream);
  return launch<DH, 1>(qkv, ld, key_bias, n_envs, d, n_heads, q_first, n_q, g_out, ldgo, gq, ldq, gk, ldk, gv, ldv, stream);
}
}  // namespace

int attention29_bwd(const __half* qkv, int ld_qkv, const float* key_bias, int64_t n_envs, int d, int n_heads, int q_first,
                    int n_q, const __half* g_out, int ldgo, __half* gq, int ldq, __half* gk, int ldk, __half* gv, int ldv,
                    cudaStream_t stream) {
  if (!qkv || !key_bias || !g_out || !gq || !gk || !gv) {
    set_error("attention_bwd: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (n_heads < 1 || d % n_heads != 0 || q_first < 0 || n_q < 1 || q_first + n_q > kT || (ld_qkv % 8) || (ldgo % 8) ||
      (ldq % 2) || (ldk % 2) || (ldv % 2) || !aligned16(qkv) || !aligned16(g_out)) {
    set_error("attention_bwd: bad shape d=%d heads=%d q_first=%d n_q=%d", d, n_heads, q_first, n_q);
    return BSRL_ERR_SHAPE;
  }
  if (n_envs == 0) return BSRL_OK;
  switch (d / n_heads) {
    case 32: return launch_mt<32>(qkv, ld_qkv, key_bias, n_envs, d, n_heads, q_first, n_q, g_out, ldgo, gq, ldq, gk, ldk, gv, ldv, stream);
    case 48: return launch_mt<48>(qkv, ld_qkv, key_bias, n_envs, d, n_heads, q_first, n_q, g_out, ldgo, gq, ldq, gk, ldk, gv, ldv, stream);
    case 64: return launch_mt<64>(qkv, ld_qkv, key_bias, n_envs, d, n_heads, q_first, n_q, g_out, ldgo, gq, ldq, gk, ldk, gv, ldv, stream);
    default:
      set_error("attention_bwd: head_dim %d unsupported (32, 48 or 64)", d / n_heads);
      return BSRL_ERR_UNSUPPORTED;
  }
}

}  // namespace bsrl
