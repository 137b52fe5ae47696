// Fused head of one transformer block: packed q|k|v projection on tcgen05 / TMEM and the masked
// 29-key multi-head attention on the projected rows, without the (rows, 3d) round trip through HBM.
//
//   qkv = h [Wq;Wk;Wv]^T + b          (h = LayerNorm rows, fp16)
//   att = softmax(q k^T / sqrt(dh) + key_bias) v, heads concatenated
//
// One tile = 4 environments, each padded from 29 to 32 token rows (a 3-D TMA load zero-fills rows
// 29..31), so that env e of the tile is exactly rows [32 e, 32 e + 32) = TMEM lane quadrant e of the
// 128-row MMA.  The projection runs per HEAD GROUP (two heads: 64 q + 64 k + 64 v = 192 output
// columns, the weight rows regrouped at pack time), so that a group's q, k, v fit in one 50 KB
// shared-memory tile.  The two warps that own a lane quadrant drain THEIR env's rows (half of the
// columns each) and then attend that env's two heads (m16n8k16 MMAs, fp32 softmax in registers): an env
// only ever waits for its own pair of warps (a 64-thread named barrier), never for the whole CTA, while
// the tensor core already projects the next group into the other TMEM buffer.
//
//   warp 0      TMA producer: the h tile (d/64 swizzled chunks, loaded once per tile) and the
//               regrouped weight tiles (192 x 64 or 144 x 64 per stage, 3- or 4-stage ring)
//   warp 1      MMA issuer: tcgen05.mma M = 128, N = 192, K = 16
//   warps 2..9  drain the accumulator (+ bias, fp16) into the q|k|v tile, then attend
//
// HBM traffic per token: read h (2d B), write att (2d B).  Replaces fp16_packed_linear + attn29 /
// packed_sdpa (python/policy.py:586-600, :645-692; python/beat_arena_env/csrc/small_attn.cu).
// With all 29 query rows, an env's output for the group (29 rows x 128 bytes for two heads of 32, x 96 bytes
// for one head of 48) is staged in shared memory and leaves as one TMA store per env.  All waits are
// bounded (tc5.cuh).
#include "kernels.cuh"
#include "tc5.cuh"

namespace bsrl {
namespace {
using namespace tc5;

constexpr int EPT = 4;                  // envs per tile
constexpr int EROWS = 32;               // tile rows per env: 29 tokens + 3 zero rows
constexpr int BM = EPT * EROWS;
constexpr int MAX_STAGES = 4;           // weight ring: 3 stages of 24 KB (head_dim 32) or 4 of 18 KB (head_dim 48), as measured
constexpr int CHUNK_BYTES = BM * 128;   // 16 KB: 128 rows x 64 k-columns
constexpr int WORKERS = 8;
constexpr int THREADS = (2 + WORKERS) * 32;
// Head group of G heads of width DH: 3 G DH projection columns per group -- (32, 2): 192, two heads;
// (48, 1): 144, one head (the reference's production shape, 4 heads of 48); (64, 1): 192, one head (the wide policy).
template <int DH_, int G_>
struct Shape {
  static constexpr int DH = DH_, G = G_, GD = G * DH, NG = 3 * GD;
  // STREAM (head_dim 64, d up to 512): the h tile does not stay resident (128 rows x 512 x 2 B = 128 KB); its
  // 64-column chunks travel through the ring beside the weight chunks, once per head group (from L2 after the first)
  static constexpr bool STREAM = DH == 64;
  static constexpr int STAGES = DH == 48 ? 4 : 3;
  static constexpr int W_BYTES = NG * 128;       // NG weight rows x 64 k-columns (24 KB / 18 KB)
  static constexpr int STAGE_BYTES = W_BYTES + (STREAM ? CHUNK_BYTES : 0);
  static constexpr int A_BYTES = STREAM ? 0 : 4 * CHUNK_BYTES;
  static constexpr int MAX_D = STREAM ? 512 : 256;
  static constexpr int LDQ = NG * 2 + 16;        // row pitch of the q|k|v tile: 400 / 304 bytes, ldmatrix conflict-free
  static constexpr int SQ_BYTES = BM * LDQ;
  static constexpr int SO_BYTES = BM * 128;      // attention output of one group: 128 rows x 128 B, 128-byte swizzle
  static constexpr int BIAS_BYTES = 3 * MAX_D * 4;
  static constexpr int SB_BYTES = EPT * 2 * 3 * 64;   // body-token mode: q0 | k0 | v0 (64 B each) per env and head of the group
  static constexpr int SMEM_BYTES = A_BYTES + STAGES * STAGE_BYTES + SO_BYTES + SQ_BYTES + BIAS_BYTES + SB_BYTES + 1024 + 256;
  static_assert(NG % 16 == 0 && NG <= 256 && STAGE_BYTES % 1024 == 0 && W_BYTES % 1024 == 0, "group width");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};
constexpr int KERNEL_ID = 3;

struct Shared {
  uint64_t w_full[MAX_STAGES], w_empty[MAX_STAGES], a_full[4], a_free[4], acc_full[2], acc_empty[2], attn_done[2], mma_done;
  uint32_t tmem_base;
  int abort;
  int quit[EPT];   // abort flag as sampled by one thread of an env's warp pair before their barrier, so both leave together
};

struct Params {
  int d, n_heads, q_first, n_q;
  int64_t n_envs;
  int n_tiles;
  const float* bias;       // regrouped q|k|v bias (3d)
  const float* key_bias;   // (n_envs, 29)
  __half* out;             // (n_envs * n_q, ldo)
  int ldo;
  __half* v_out;           // value residual: own values out / block 0's values in + the two mix scalars
  const __half* v0;
  const float* vres;
  int out_tma;             // the group's output leaves as one TMA store from shared memory (all 29 query rows, two heads of 32)
  // single-body-token layout (BODY kernels): envs of `tokens` = 33 rows; rows 1..32 (the object tokens) are the env's
  // 32 tile rows, row 0 (the body token) comes projected from qkv0 (n_envs, 3d: q | k | v in the plain column
  // order) and is folded in beside the MMA tiles; body_only: only the body token's output row is wanted
  int tokens, tok0, body_only;
  const __half* qkv0;
  int* status;
};

__device__ __forceinline__ void give_up(Shared* sh, int* status, int role) {
  atomicCAS(status, 0, KERNEL_ID * 16 + role);
  sh->abort = 1;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Attention of one (env, head) pair from the shared q|k|v tile; one warp.  q, k, v are byte
// addresses (shared window) of the pair's first row / first column; rows are LDQ bytes apart.
// The MT 16-row query tiles are processed side by side: two independent dependency chains per warp
// (the kernel is latency-bound here) and each K / V fragment is fetched once for both.
// OB: bytes per row of the staged group output (128: two heads of 32, swizzled; 96: one head of 48, dense)
// BODY: one more key outside the tile (the body token): x_lane = q_row . k_0 for row `lane` (raw), kb0 its
// base-2 key bias, v0 its DH values (shared memory, generic pointer); its score joins each row's softmax and its
// probability times v_0 starts the row's output.
template <int MT, int DH, int LDQ, int OB, bool BODY = false>
__device__ __forceinline__ void attend_pair(uint32_t sq, uint32_t sk, uint32_t sv, const float (&kb)[4][2],
                                            int n_q, __half* out_env, int ldo, int lane, uint8_t* so, int so_row0, int so_piece0,
                                            float x_lane = 0.f, float kb0 = 0.f, const __half* v0 = nullptr) {
  const int g = lane >> 2, tig = lane & 3;
  const float scale = rsqrtf((float)DH) * 1.4426950408889634f;   // 1/sqrt(dh) * log2(e)
  float s[MT][4][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[mt][nt][e] = 0.f;
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) {
    uint32_t a[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      ldmatrix_x4(a[mt], sq + (mt * 16 + (lane & 15)) * LDQ + (ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint32_t b[4];
      const int row = j * 16 + (lane & 7) + ((lane >> 4) << 3);
      ldmatrix_x4(b, sk + row * LDQ + (ks * 16 + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_f16(s[mt][2 * j], a[mt], b[0], b[1]);
        mma_f16(s[mt][2 * j + 1], a[mt], b[2], b[3]);
      }
    }
  }
  uint32_t pa[MT][2][4];
  float p0[MT][2];                    // BODY: the body key's probability for rows g and g + 8 of each query tile
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    float mx[2] = {-INFINITY, -INFINITY};
    if (BODY) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        p0[mt][r] = fmaf(__shfl_sync(0xffffffffu, x_lane, mt * 16 + g + r * 8), scale, kb0);
        mx[r] = p0[mt][r];
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[mt][nt][e] = fmaf(s[mt][nt][e], scale, kb[nt][e & 1]);   // base-2 logits: scale and key bias carry log2(e)
        mx[e >> 1] = fmaxf(mx[e >> 1], s[mt][nt][e]);
      }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[mt][nt][e] = ex2_approx(s[mt][nt][e] - mx[e >> 1]);
        sum[e >> 1] += s[mt][nt][e];
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
      if (BODY) {
        p0[mt][r] = ex2_approx(p0[mt][r] - mx[r]);
        sum[r] = rcp_approx(sum[r] + p0[mt][r]);
        p0[mt][r] *= sum[r];
      } else {
        sum[r] = rcp_approx(sum[r]);
      }
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      pa[mt][ks][0] = pack_half2(s[mt][2 * ks][0] * sum[0], s[mt][2 * ks][1] * sum[0]);
      pa[mt][ks][1] = pack_half2(s[mt][2 * ks][2] * sum[1], s[mt][2 * ks][3] * sum[1]);
      pa[mt][ks][2] = pack_half2(s[mt][2 * ks + 1][0] * sum[0], s[mt][2 * ks + 1][1] * sum[0]);
      pa[mt][ks][3] = pack_half2(s[mt][2 * ks + 1][2] * sum[1], s[mt][2 * ks + 1][3] * sum[1]);
    }
  }
  float o[MT][DH / 8][4];
#pragma unroll
  for (int nt = 0; nt < DH / 8; ++nt) {
    float2 v = make_float2(0.f, 0.f);
    if (BODY) v = __half22float2(*reinterpret_cast<const __half2*>(v0 + nt * 8 + tig * 2));
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      o[mt][nt][0] = BODY ? p0[mt][0] * v.x : 0.f;
      o[mt][nt][1] = BODY ? p0[mt][0] * v.y : 0.f;
      o[mt][nt][2] = BODY ? p0[mt][1] * v.x : 0.f;
      o[mt][nt][3] = BODY ? p0[mt][1] * v.y : 0.f;
    }
  }
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
    for (int j = 0; j < DH / 16; ++j) {
      uint32_t b[4];
      const int row = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      ldmatrix_x4_trans(b, sv + row * LDQ + (j * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_f16(o[mt][2 * j], pa[mt][ks], b[0], b[1]);
        mma_f16(o[mt][2 * j + 1], pa[mt][ks], b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int qrow = mt * 16 + g + r * 8;
      if (qrow < n_q && so) {
        // staged for the group's TMA store.  128-byte rows: 16-byte piece p of row r at ((p ^ (r & 7)) << 4),
        // the 8 rows of a store instruction hit 32 different banks; 96-byte rows: dense (2-way conflicts)
        const int row = so_row0 + qrow;
        uint8_t* orow = so + row * OB + tig * 4;
#pragma unroll
        for (int nt = 0; nt < DH / 8; ++nt)
          *reinterpret_cast<uint32_t*>(orow + (OB == 128 ? (((so_piece0 + nt) ^ (row & 7)) << 4) : ((so_piece0 + nt) << 4))) =
              pack_half2(o[mt][nt][r * 2], o[mt][nt][r * 2 + 1]);
      } else if (qrow < n_q) {
        __half* orow = out_env + (int64_t)qrow * ldo + tig * 2;
#pragma unroll
        for (int nt = 0; nt < DH / 8; ++nt)
          *reinterpret_cast<uint32_t*>(orow + nt * 8) = pack_half2(o[mt][nt][r * 2], o[mt][nt][r * 2 + 1]);
      }
    }
}

// VRES: the value-residual code of the drain is compiled in (it costs ~14 % of the kernel even when idle)
// BODY: the single-body-token layout (Params::tokens and below); DH = 32, G = 2 only
template <int DH, int G, bool VRES, bool BODY = false>
__global__ void __launch_bounds__(THREADS, 1)
attn_block_kernel(const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_w,
                  const __grid_constant__ CUtensorMap tm_o, Params p) {
  using S = Shape<DH, G>;
  constexpr int STAGES = S::STAGES, GD = S::GD, NG = S::NG, STAGE_BYTES = S::STAGE_BYTES, LDQ = S::LDQ, SQ_BYTES = S::SQ_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  constexpr bool STREAM = S::STREAM;
  const uint32_t sA = base, ring = base + S::A_BYTES, sO = ring + STAGES * STAGE_BYTES, sQ = sO + S::SO_BYTES;
  uint8_t* sO_g = gen + S::A_BYTES + STAGES * STAGE_BYTES;
  uint8_t* sQ_g = sO_g + S::SO_BYTES;
  float* s_bias = reinterpret_cast<float*>(sQ_g + SQ_BYTES);
  uint8_t* sB_g = sQ_g + SQ_BYTES + S::BIAS_BYTES;
  Shared* sh = reinterpret_cast<Shared*>(sB_g + S::SB_BYTES);
  static_assert(!BODY || (DH == 32 && G == 2 && !VRES), "body-token mode: two heads of 32 per group");
  constexpr int NKEYS = BODY ? EROWS : kT;            // live keys of an env inside the tile
  const int T = BODY ? p.tokens : kT;                 // token rows per env in memory
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = p.d, KB = d >> 6, n_groups = d / GD;
  volatile int* abort = &sh->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&sh->w_full[s]), 1);
      mbar_init(smem_u32(&sh->w_empty[s]), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&sh->a_full[i]), 1);
      mbar_init(smem_u32(&sh->a_free[i]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->acc_full[b]), 1);
      mbar_init(smem_u32(&sh->acc_empty[b]), WORKERS);
      mbar_init(smem_u32(&sh->attn_done[b]), WORKERS);
    }
    mbar_init(smem_u32(&sh->mma_done), 1);
    sh->abort = 0;
    for (int e = 0; e < EPT; ++e) sh->quit[e] = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_h);
    tma_prefetch_desc(&tm_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh->tmem_base), 512);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < 3 * d; i += THREADS) s_bias[i] = p.bias[i];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      auto w_stage = [&](int g, int kb, int t) -> bool {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(smem_u32(&sh->w_empty[s]), ph ^ 1, abort)) { give_up(sh, p.status, 1); return false; }
        const uint32_t bar = smem_u32(&sh->w_full[s]);
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(ring + s * STAGE_BYTES, &tm_w, 64 * kb, NG * g, bar);
        if (STREAM) tma_load_3d(ring + s * STAGE_BYTES + S::W_BYTES, &tm_h, 64 * kb, BODY ? p.tok0 : 0, t * EPT, bar);
        ++it;
        return true;
      };
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++tile_i) {
        if (STREAM) {
          for (int g = 0; g < n_groups && ok; ++g)
            for (int kb = 0; kb < KB && ok; ++kb) ok = w_stage(g, kb, t);
          continue;
        }
        for (int kb = 0; kb < KB && ok; ++kb) {
          // chunk kb of the h tile is free once the previous tile's last group has used it
          if (!mbar_wait(smem_u32(&sh->a_free[kb]), (tile_i & 1) ^ 1, abort)) { give_up(sh, p.status, 2); ok = false; break; }
          const uint32_t bar = smem_u32(&sh->a_full[kb]);
          mbar_expect_tx(bar, CHUNK_BYTES);
          tma_load_3d(sA + kb * CHUNK_BYTES, &tm_h, 64 * kb, BODY ? p.tok0 : 0, t * EPT, bar);
          ok = w_stage(0, kb, t);
        }
        for (int g = 1; g < n_groups && ok; ++g)
          for (int kb = 0; kb < KB && ok; ++kb) ok = w_stage(g, kb, t);
      }
      // loads in flight must land before the CTA exits (bounded, ignoring abort)
      for (uint32_t j = it > STAGES ? it - STAGES : 0; j < it; ++j) {
        uint32_t spins = 0;
        while (!mbar_try_wait(smem_u32(&sh->w_full[j % STAGES]), (j / STAGES) & 1) && ++spins < kSpinLimit) {}
        if (spins >= kSpinLimit) give_up(sh, p.status, 3);
      }
      if (!STREAM && tile_i > 0)
        for (int kb = 0; kb < KB; ++kb) {
          uint32_t spins = 0;
          while (!mbar_try_wait(smem_u32(&sh->a_full[kb]), (tile_i - 1) & 1) && ++spins < kSpinLimit) {}
          if (spins >= kSpinLimit) give_up(sh, p.status, 4);
        }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tile_i = 0, gi = 0;
      bool ok = true;
      const uint32_t idesc = idesc_f16(BM, NG);
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++tile_i) {
        for (int g = 0; g < n_groups && ok; ++g, ++gi) {
          const int buf = gi & 1;
          if (!mbar_wait(smem_u32(&sh->acc_empty[buf]), ((gi >> 1) & 1) ^ 1, abort)) { give_up(sh, p.status, 5); ok = false; break; }
          // The workers' attention runs on warp-level MMAs, which queue behind tcgen05 MMAs on the same
          // tensor cores: this group's projection is held back until the attention of two groups ago is
          // over, so that it runs while the workers drain the previous group instead (without the wait the
          // kernel measured 3 % slower).
          if (gi >= 2 && !mbar_wait(smem_u32(&sh->attn_done[buf]), ((gi - 2) >> 1) & 1, abort)) { give_up(sh, p.status, 10); ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * 256;
          for (int kb = 0; kb < KB; ++kb, ++it) {
            if (!STREAM && g == 0 && !mbar_wait(smem_u32(&sh->a_full[kb]), tile_i & 1, abort)) { give_up(sh, p.status, 6); ok = false; break; }
            const int s = it % STAGES;
            if (!mbar_wait(smem_u32(&sh->w_full[s]), (it / STAGES) & 1, abort)) { give_up(sh, p.status, 7); ok = false; break; }
            tc_fence_after();
            const uint64_t ad = smem_desc_sw128(STREAM ? ring + s * STAGE_BYTES + S::W_BYTES : sA + kb * CHUNK_BYTES);
            const uint64_t wd = smem_desc_sw128(ring + s * STAGE_BYTES);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_f16_ss(d_tmem, ad + 2 * k, wd + 2 * k, idesc, (kb | k) != 0);
            tc_commit(smem_u32(&sh->w_empty[s]));
            if (!STREAM && g == n_groups - 1) tc_commit(smem_u32(&sh->a_free[kb]));
          }
          if (ok) tc_commit(smem_u32(&sh->acc_full[buf]));
        }
      }
      tc_commit(smem_u32(&sh->mma_done));
      uint32_t spins = 0;
      while (!mbar_try_wait(smem_u32(&sh->mma_done), 0) && ++spins < kSpinLimit) {}
      if (spins >= kSpinLimit) give_up(sh, p.status, 8);
    }
  } else {
    // ------------------------------------------------------------ workers: drain, then attend
    const int wi = warp - 2;
    const int q = warp & 3, half = wi >> 2;           // TMEM lane quadrant = env of the tile, column half
    const int trow = q * EROWS + lane;                // tile row: token `lane` of env q (29..31: zero rows)
    // drain: the group's NG columns in 16-column units, split between the two halves (6 + 6 or 5 + 4)
    constexpr int UNITS = NG / 16, U0 = (UNITS + 1) / 2;
    const int u_first = half ? U0 : 0, u_count = half ? UNITS - U0 : U0;
    // attention of the env this warp drained: G = 2: one head per warp of the pair, both 16-row query tiles;
    // G = 1: one query tile each
    const int env_l = q, hh = G == 2 ? half : 0, mt_own = G == 2 ? 0 : half;
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory"); };
    uint32_t gi = 0;
    bool ok = true;
    const float vres_a = (VRES && p.vres) ? p.vres[0] : 1.f, vres_b = (VRES && p.vres) ? p.vres[1] : 0.f;
    for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
      const int64_t env = (int64_t)t * EPT + env_l;
      // this lane's key-bias values (keys nt * 8 + tig * 2 + e of the m16n8 accumulator layout, times
      // log2 e; -inf past the 29th key), fetched once per tile and long before the first softmax
      float kb[4][2];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = nt * 8 + (lane & 3) * 2 + e;
          kb[nt][e] = (key < NKEYS && env < p.n_envs) ? p.key_bias[env * T + (BODY ? p.tok0 : 0) + key] * 1.4426950408889634f : -INFINITY;
        }
      // body-token mode: the body key's bias, and this lane's object key's (lane = key in the body row's softmax)
      float kb0 = 0.f, kbl = 0.f;
      if (BODY && env < p.n_envs) {
        kb0 = p.key_bias[env * T] * 1.4426950408889634f;
        kbl = p.key_bias[env * T + 1 + lane] * 1.4426950408889634f;
      }
      // single-query launches (the critic): lane = key in that row's softmax
      const bool one_row = !BODY && p.n_q == 1;
      float kb_row = -INFINITY;
      if (one_row && lane < NKEYS && env < p.n_envs) kb_row = p.key_bias[env * T + lane] * 1.4426950408889634f;
      for (int g = 0; g < n_groups && ok; ++g, ++gi) {
        const int buf = gi & 1;
        // body token's q0 | k0 | v0 of this warp's head: lanes 0..11 fetch one 16-byte piece each, long before use
        uint4 b0v = make_uint4(0, 0, 0, 0);
        if (BODY && lane < 12 && env < p.n_envs)
          b0v = *reinterpret_cast<const uint4*>(p.qkv0 + env * 3 * (int64_t)d + (lane >> 2) * d + (g * G + hh) * DH + (lane & 3) * 8);
        // A failed wait must not leave other workers stuck at the CTA-level barriers below: the
        // warp keeps going (on garbage) and everyone leaves together once one thread has sampled
        // the abort flag ahead of a barrier.
        if (!mbar_wait_warp(smem_u32(&sh->acc_full[buf]), (gi >> 1) & 1, abort) && lane == 0) give_up(sh, p.status, 9);
        tc_fence_after();
        {
          const uint32_t tcol = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256 + u_first * 16;
          const float* bias_u = s_bias + g * NG + u_first * 16;
          uint8_t* dst_u = sQ_g + trow * LDQ + (u_first * 16) * 2;
          // 16 columns -> bias, fp16, two 16-byte pieces of this thread's row
          auto put16 = [&](const uint32_t* v, int u) {
            const float4* b4 = reinterpret_cast<const float4*>(bias_u + u * 16);
            // value residual (python/policy.py:604-615): the group's v columns are written out as
            // this block's own values and / or mixed with block 0's before the attention reads them
            const int vcol = (u_first + u) * 16 - 2 * GD;           // column inside the group's v section
            const bool vres_rows = VRES && vcol >= 0 && lane < kT && env < p.n_envs;
            const int64_t goff = (env * kT + lane) * d + g * GD + vcol;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const float4 b0 = b4[2 * j], b1 = b4[2 * j + 1];
              float f[8] = {__uint_as_float(v[8 * j]) + b0.x,     __uint_as_float(v[8 * j + 1]) + b0.y,
                            __uint_as_float(v[8 * j + 2]) + b0.z, __uint_as_float(v[8 * j + 3]) + b0.w,
                            __uint_as_float(v[8 * j + 4]) + b1.x, __uint_as_float(v[8 * j + 5]) + b1.y,
                            __uint_as_float(v[8 * j + 6]) + b1.z, __uint_as_float(v[8 * j + 7]) + b1.w};
              if (VRES && vres_rows && p.v_out)
                *reinterpret_cast<uint4*>(p.v_out + goff + 8 * j) =
                    make_uint4(pack_half2(f[0], f[1]), pack_half2(f[2], f[3]), pack_half2(f[4], f[5]), pack_half2(f[6], f[7]));
              if (VRES && vres_rows && p.v0) {
                const uint4 o = *reinterpret_cast<const uint4*>(p.v0 + goff + 8 * j);
                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 ov = __half22float2(*reinterpret_cast<const __half2*>(&ow[e]));
                  f[2 * e] = fmaf(vres_a, f[2 * e], vres_b * ov.x);
                  f[2 * e + 1] = fmaf(vres_a, f[2 * e + 1], vres_b * ov.y);
                }
              }
              *reinterpret_cast<uint4*>(dst_u + u * 32 + 16 * j) =
                  make_uint4(pack_half2(f[0], f[1]), pack_half2(f[2], f[3]), pack_half2(f[4], f[5]), pack_half2(f[6], f[7]));
            }
          };
          int u = 0;
          for (; u + 2 <= u_count; u += 2) {
            uint32_t r[32];
            tmem_ld32(tcol + u * 16, r);
            tmem_wait_ld();
            put16(r, u);
            put16(r + 16, u + 1);
          }
          if (u < u_count) {
            uint32_t r[16];
            tmem_ld16(tcol + u * 16, r);
            tmem_wait_ld();
            put16(r, u);
          }
        }
        if (BODY && lane < 12) *reinterpret_cast<uint4*>(sB_g + ((env_l * 2 + hh) * 3 + (lane >> 2)) * 64 + (lane & 3) * 16) = b0v;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[buf]));     // the TMEM buffer may be refilled
        if (half == 0 && lane == 0) {
          sh->quit[q] = *abort;
          if (p.out_tma) bulk_wait_read<0>();           // this env's previous output store has read its sO rows
        }
        pair_sync();                                    // the env's q|k|v rows are complete
        if (*reinterpret_cast<volatile int*>(&sh->quit[q])) {
          ok = false;
          break;
        }
        if (env < p.n_envs) {
          const uint32_t rows = sQ + (env_l * EROWS) * LDQ;
          const uint32_t sq_pair = rows + (p.q_first + mt_own * 16) * LDQ + (hh * DH) * 2,
                         sk_pair = rows + (GD + hh * DH) * 2, sv_pair = rows + (2 * GD + hh * DH) * 2;
          __half* out_pair = p.out + (env * p.n_q + mt_own * 16) * (int64_t)p.ldo + (g * G + hh) * DH;
          const int n_q = p.n_q - mt_own * 16;      // query rows left from this warp's first one
          uint8_t* so_tile = p.out_tma ? sO_g : nullptr;
          if constexpr (BODY) {
            // ---- the body token beside the tile (one warp = one head of the env's group)
            const uint8_t* rows_g = sQ_g + (env_l * EROWS) * LDQ;
            const uint8_t* sb = sB_g + (env_l * 2 + hh) * 192;           // q0 at +0, k0 at +64, v0 at +128
            const float scale = rsqrtf((float)DH) * 1.4426950408889634f;
            float x_lane = 0.f, sc = 0.f, s00 = 0.f;
#pragma unroll
            for (int ch = 0; ch < DH / 8; ++ch) {
              const uint4 q0v = *reinterpret_cast<const uint4*>(sb + ch * 16);
              const uint4 k0v = *reinterpret_cast<const uint4*>(sb + 64 + ch * 16);
              const uint4 qv = *reinterpret_cast<const uint4*>(rows_g + lane * LDQ + (hh * DH) * 2 + ch * 16);
              const uint4 kv = *reinterpret_cast<const uint4*>(rows_g + lane * LDQ + (GD + hh * DH) * 2 + ch * 16);
              const __half2* q0h = reinterpret_cast<const __half2*>(&q0v);
              const __half2* k0h = reinterpret_cast<const __half2*>(&k0v);
              const __half2* qh = reinterpret_cast<const __half2*>(&qv);
              const __half2* kh = reinterpret_cast<const __half2*>(&kv);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 a0 = __half22float2(q0h[e]), b0 = __half22float2(k0h[e]);
                const float2 a = __half22float2(qh[e]), b = __half22float2(kh[e]);
                x_lane = fmaf(a.x, b0.x, fmaf(a.y, b0.y, x_lane));       // object row `lane` against the body key
                sc = fmaf(a0.x, b.x, fmaf(a0.y, b.y, sc));               // body row against object key `lane`
                s00 = fmaf(a0.x, b0.x, fmaf(a0.y, b0.y, s00));           // body row against the body key
              }
            }
            {   // the body token's own output row: softmax over the 32 object keys (one per lane) and the body key
              sc = fmaf(sc, scale, kbl);
              s00 = fmaf(s00, scale, kb0);
              const float mx = fmaxf(warp_max(sc), s00);
              const float pj = ex2_approx(sc - mx), p00 = ex2_approx(s00 - mx);
              const float inv = rcp_approx(warp_sum(pj) + p00);
              const __half* v0h = reinterpret_cast<const __half*>(sb + 128);
              const uint8_t* vcol = rows_g + (2 * GD + hh * DH) * 2 + lane * 2;      // column `lane` of the head's v rows
              float acc = p00 * __half2float(v0h[lane]);
#pragma unroll 8
              for (int j = 0; j < EROWS; ++j)
                acc = fmaf(__shfl_sync(0xffffffffu, pj, j), __half2float(*reinterpret_cast<const __half*>(vcol + j * LDQ)), acc);
              __half* orow = p.out + (env * (p.body_only ? 1 : T)) * (int64_t)p.ldo + (g * G + hh) * DH;
              orow[lane] = __float2half_rn(acc * inv);
            }
            if (!p.body_only)
              attend_pair<2, DH, LDQ, GD * 2, true>(sq_pair, sk_pair, sv_pair, kb, n_q, out_pair, p.ldo, lane, so_tile,
                                                    env_l * EROWS, hh * (DH / 8), x_lane, kb0, reinterpret_cast<const __half*>(sb + 128));
          } else if (one_row) {
            // One query row per env: on the CUDA cores.  A 16-row MMA tile for one row costs the tensor pipe, which
            // the projection of the next head group shares, 16 warp MMAs of 32 cycles per (env, head); this is ~200
            // plain instructions (lane = key for the scores, lane = output column for the weighted sum).
            if (mt_own == 0) {
              const uint8_t* rows_g = sQ_g + (env_l * EROWS) * LDQ;
              const uint8_t* qrow = rows_g + p.q_first * LDQ + (hh * DH) * 2;
              const uint8_t* krow = rows_g + (lane < NKEYS ? lane : 0) * LDQ + (GD + hh * DH) * 2;
              float sc = 0.f;
#pragma unroll
              for (int ch = 0; ch < DH / 8; ++ch) {
                const uint4 qv = *reinterpret_cast<const uint4*>(qrow + ch * 16);
                const uint4 kv = *reinterpret_cast<const uint4*>(krow + ch * 16);
                const __half2* qh = reinterpret_cast<const __half2*>(&qv);
                const __half2* kh = reinterpret_cast<const __half2*>(&kv);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 a = __half22float2(qh[e]), b = __half22float2(kh[e]);
                  sc = fmaf(a.x, b.x, fmaf(a.y, b.y, sc));
                }
              }
              sc = fmaf(sc, rsqrtf((float)DH) * 1.4426950408889634f, kb_row);      // -inf past the last key
              const float mx = warp_max(sc);
              const float pj = ex2_approx(sc - mx);
              const float inv = rcp_approx(warp_sum(pj));
              __half* orow = p.out + env * (int64_t)p.ldo + (g * G + hh) * DH;
#pragma unroll
              for (int dd = 0; dd < DH; dd += 32) {
                const int col = dd + lane;
                const uint8_t* vcol = rows_g + (2 * GD + hh * DH) * 2 + (col < DH ? col : 0) * 2;
                float acc = 0.f;
#pragma unroll 8
                for (int j = 0; j < NKEYS; ++j)
                  acc = fmaf(__shfl_sync(0xffffffffu, pj, j), __half2float(*reinterpret_cast<const __half*>(vcol + j * LDQ)), acc);
                if (col < DH) orow[col] = __float2half_rn(acc * inv);
              }
            }
          } else {
            if (G == 2 && n_q > 16) attend_pair<2, DH, LDQ, GD * 2>(sq_pair, sk_pair, sv_pair, kb, n_q, out_pair, p.ldo, lane, so_tile, env_l * EROWS + mt_own * 16, hh * (DH / 8));
            else if (n_q > 0) attend_pair<1, DH, LDQ, GD * 2>(sq_pair, sk_pair, sv_pair, kb, n_q, out_pair, p.ldo, lane, so_tile, env_l * EROWS + mt_own * 16, hh * (DH / 8));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->attn_done[buf]));
        if (p.out_tma) fence_proxy_async_smem();                         // this thread's sO writes -> the TMA engine
        pair_sync();                                                     // the env's rows may be overwritten
        if (p.out_tma && half == 0 && lane == 0 && env < p.n_envs) {     // token rows 29..31 of the box are clipped
          tma_store_3d(&tm_o, g * GD, BODY ? p.tok0 : 0, (int)env, sO + (uint32_t)(q * EROWS) * (uint32_t)(GD * 2));
          bulk_commit();
        }
      }
    }
    if (p.out_tma && half == 0 && lane == 0) bulk_wait_all();   // the output stores are complete before the CTA exits
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}
}  // namespace

bool attn_block_ok(const AttnBlockArgs& a) {
  if (a.d % 64 != 0 || a.d < 64 || a.n_heads < 1 || a.d % a.n_heads != 0) return false;
  const int dh = a.d / a.n_heads;
  if (!((dh == 32 && a.n_heads % 2 == 0) || dh == 48 || dh == 64)) return false;
  if (a.d > (dh == 64 ? Shape<64, 1>::MAX_D : Shape<32, 2>::MAX_D)) return false;
  if (a.n_envs < 1 || a.n_envs > 0x7fffffffLL / (BM * 2)) return false;
  if (!aligned16(a.h) || !aligned16(a.wg) || !aligned16(a.bg) || !aligned16(a.out) || (a.ldh % 8) || (a.ldo % 8)) return false;
  if (a.body) {      // one body token + 32 object tokens per env; all rows out, or the body row only
    if (dh != 32 || a.tokens != EROWS + 1 || !a.qkv0 || !aligned16(a.qkv0) || a.v_out || a.v0) return false;
    return a.q_first == 0 && (a.n_q == a.tokens || a.n_q == 1);
  }
  if (a.q_first < 0 || a.n_q < 1 || a.q_first + a.n_q > kT) return false;
  return true;
}

int attn_block(const AttnBlockArgs& a, cudaStream_t stream) {
  if (!a.h || !a.wg || !a.bg || !a.key_bias || !a.out) {
    set_error("attn_block: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (!attn_block_ok(a)) {
    set_error("attn_block: shape d=%d heads=%d tokens=%d does not fit the fused kernel (head_dim 32 or 48 with d <= 256, head_dim "
              "64 with d <= 512; body-token layout: head_dim 32, 33 tokens)", a.d, a.n_heads, a.body ? a.tokens : kT);
    return BSRL_ERR_UNSUPPORTED;
  }
  int* status = device_status_ptr();
  if (!status) return BSRL_ERR_CUDA;
  const int dh = a.d / a.n_heads;
  const int T = a.body ? a.tokens : kT;
  CUtensorMap tm_h, tm_w;
  if (!make_tmap_env3d(&tm_h, a.h, a.n_envs, T, a.d, a.ldh, 64, EROWS, EPT)) return BSRL_ERR_CUDA;
  if (!make_tmap_f16(&tm_w, a.wg, 3 * a.d, a.d, a.d, dh == 48 ? Shape<48, 1>::NG : Shape<32, 2>::NG)) return BSRL_ERR_CUDA;
  // all query rows: an env's output for a group is contiguous rows x 128 (two heads of 32) or 96 bytes (one of 48) = one TMA store
  const bool out_tma = a.q_first == 0 && a.n_q == T;
  CUtensorMap tm_o = tm_h;
  if (out_tma && !make_tmap_env3d(&tm_o, a.out, a.n_envs, T, a.d, a.ldo, dh == 48 ? 48 : 64, EROWS, 1)) return BSRL_ERR_CUDA;
  static DeviceOnce once;
  int rc = once.run("attn_block_kernel set-up", [] {
    const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
    cudaError_t e = cudaFuncSetAttribute(attn_block_kernel<32, 2, false>, at, Shape<32, 2>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_block_kernel<32, 2, true>, at, Shape<32, 2>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_block_kernel<32, 2, false, true>, at, Shape<32, 2>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_block_kernel<48, 1, false>, at, Shape<48, 1>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_block_kernel<48, 1, true>, at, Shape<48, 1>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_block_kernel<64, 1, false>, at, Shape<64, 1>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_block_kernel<64, 1, true>, at, Shape<64, 1>::SMEM_BYTES);
    return e;
  });
  if (rc != BSRL_OK) return rc;
  Params p;
  p.d = a.d; p.n_heads = a.n_heads;
  p.q_first = a.body ? 0 : a.q_first;
  p.n_q = a.body ? EROWS : a.n_q;                 // body-token layout: the tile's query rows are the 32 object tokens
  p.n_envs = a.n_envs;
  p.n_tiles = (int)((a.n_envs + EPT - 1) / EPT);
  p.bias = a.bg; p.key_bias = a.key_bias; p.out = a.out; p.ldo = a.ldo;
  p.v_out = a.v_out; p.v0 = a.v0; p.vres = a.vres;
  p.out_tma = out_tma ? 1 : 0;
  p.tokens = T; p.tok0 = a.body ? 1 : 0; p.body_only = (a.body && a.n_q == 1) ? 1 : 0; p.qkv0 = a.qkv0;
  p.status = status;
  const int grid = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
  const bool vres = a.v_out || a.v0;
  if (a.body) attn_block_kernel<32, 2, false, true><<<grid, THREADS, Shape<32, 2>::SMEM_BYTES, stream>>>(tm_h, tm_w, tm_o, p);
  else if (dh == 32 && !vres) attn_block_kernel<32, 2, false><<<grid, THREADS, Shape<32, 2>::SMEM_BYTES, stream>>>(tm_h, tm_w, tm_o, p);
  else if (dh == 32) attn_block_kernel<32, 2, true><<<grid, THREADS, Shape<32, 2>::SMEM_BYTES, stream>>>(tm_h, tm_w, tm_o, p);
  else if (dh == 48 && !vres) attn_block_kernel<48, 1, false><<<grid, THREADS, Shape<48, 1>::SMEM_BYTES, stream>>>(tm_h, tm_w, tm_o, p);
  else if (dh == 48) attn_block_kernel<48, 1, true><<<grid, THREADS, Shape<48, 1>::SMEM_BYTES, stream>>>(tm_h, tm_w, tm_o, p);
  else if (!vres) attn_block_kernel<64, 1, false><<<grid, THREADS, Shape<64, 1>::SMEM_BYTES, stream>>>(tm_h, tm_w, tm_o, p);
  else attn_block_kernel<64, 1, true><<<grid, THREADS, Shape<64, 1>::SMEM_BYTES, stream>>>(tm_h, tm_w, tm_o, p);
  BSRL_LAUNCH_OK("attn_block_kernel");
  return BSRL_OK;
}


}  // namespace bsrl
