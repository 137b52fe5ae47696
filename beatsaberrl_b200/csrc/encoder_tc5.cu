// Fused token encoders on tcgen05 / TMEM: both layers of the four 2-layer MLPs and block 0's LayerNorm
// in one persistent kernel, one 128-row tile of ONE encoder's input rows at a time:
//
//   hid = relu(f W0^T + b0)            f: K-padded fp16 feature rows written by the tokenizer kernel
//   tok = hid W1^T + b1                -> x (fp32 residual stream, scattered into the env's token slots)
//   h   = LayerNorm(tok; g, b)         -> fp16, the first block's attention input (optional)
//
// This is note_mlp / saber_mlp / torso_mlp / leg_mlp, the token concat and blocks[0].ln_attn of the
// reference (python/policy.py:940-952, :1224-1249, :579-585) without the (rows, d) hidden and the
// separate LayerNorm pass going through HBM: per token the kernel reads 128 B of features and writes
// 4d B of x and 2d B of h -- HBM-bound.
//
//   warp 0       TMA producer: the feature tile (128 x 64, 128B swizzle) and the weights through a
//                3-stage ring of (d x 64) tiles: W0, then the d/64 k-blocks of W1 (L2-resident)
//   warp 1       MMA issuer: acc = f W0^T (one k-block, N = d), then -- once the hidden tile is in shared
//                memory -- acc = hid W1^T (d/64 k-blocks) over the same TMEM columns
//   warps 2..5   hidden warps, thread = row: acc -> bias, ReLU, fp16 -> swizzled hid tile
//   warps 6..13  output warps, thread = row, two groups of four warps owning half of the columns each:
//                acc -> bias -> x and the row statistics, then a second pass over acc for the LayerNorm
//                rows.  Rows leave through a per-warp transposition buffer as 16-byte stores covering full
//                128-byte lines of the mapped rows.
// TMEM: tile i of a CTA uses columns [256 (i & 1), 256 (i & 1) + d) for both of its accumulators, so the
// output warps drain tile i while the MMAs and the hidden warps work on tile i + 1: the output phase
// (HBM stores) is the kernel's period, everything else runs in its shadow.  All waits are bounded (tc5.cuh).
#include "kernels.cuh"
#include "tc5.cuh"

namespace bsrl {
namespace {
using namespace tc5;

constexpr int BM = 128;
constexpr int STAGES = 3, STAGE_BYTES = 32768;
constexpr int CHUNK_BYTES = BM * 64 * 2;           // one [128 x 64] fp16 swizzled chunk
constexpr int SA_BYTES = CHUNK_BYTES;              // feature tile
constexpr int SH_BYTES = 4 * CHUNK_BYTES;          // hidden tile, d <= 256
constexpr int HID_WARPS = 4, EPI_WARPS = 8;
constexpr int FIRST_EPI = 2 + HID_WARPS;
constexpr int THREADS = (2 + HID_WARPS + EPI_WARPS) * 32;
constexpr int STG_BYTES = 32 * 128;                // per-warp transposition buffer: 32 rows x 128 bytes
constexpr int PARAM_FLOATS = (2 * 4 + 2) * 256;    // b0[4], b1[4], ln gamma, ln beta
constexpr int PART_BYTES = 2 * BM * 8;
constexpr int SMEM_BYTES = SA_BYTES + SH_BYTES + STAGES * STAGE_BYTES + EPI_WARPS * STG_BYTES + PARAM_FLOATS * 4 +
                           PART_BYTES + 1024 + 256;
constexpr int KERNEL_ID = 4;

struct Shared {
  uint64_t w_full[STAGES], w_empty[STAGES];
  uint64_t a_full, a_free, h_ready, mma_done;
  uint64_t acc1_full[2], acc2_full[2], acc_free[2];     // per TMEM half
  uint32_t tmem_base;
  int abort;
};

struct Maps {
  CUtensorMap a;          // all feature rows, (29 B, 64) fp16
  CUtensorMap w0[4];      // (d, 64) first layers
  CUtensorMap w1[4];      // (d, d) second layers
};

struct EncPart {
  int64_t rows;           // input rows of this encoder
  int64_t row0;           // its first row in the feature matrix
  int64_t tile0;          // its first tile
  int group, first;       // token slots: logical row r -> x row (r / group) * 29 + first + r % group
};

struct EncParams {
  int d;
  EncPart part[4];
  int n_tiles;
  const float* b0[4];
  const float* b1[4];
  const float* ln_g;      // nullptr: no LayerNorm output
  const float* ln_b;
  float eps;
  float* x;               // (n_envs * 29, d) f32
  __half* h;              // (n_envs * 29, d) f16 or nullptr
  int* status;
};

__device__ __forceinline__ void give_up(Shared* sh, int* status, int role) {
  atomicCAS(status, 0, KERNEL_ID * 16 + role);
  sh->abort = 1;
}

// 32 fp32 values of row `row`, columns [col, col + 32) -> fp16 into a swizzled [128 x 64] chunk set
__device__ __forceinline__ void store_h32(uint8_t* chunks, int row, int col, const float (&v)[32]) {
  uint8_t* base = chunks + (col >> 6) * CHUNK_BYTES + (row >> 3) * 1024 + (row & 7) * 128;
  const int p0 = (col & 63) >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w = make_uint4(pack_half2(v[8 * i], v[8 * i + 1]), pack_half2(v[8 * i + 2], v[8 * i + 3]),
                         pack_half2(v[8 * i + 4], v[8 * i + 5]), pack_half2(v[8 * i + 6], v[8 * i + 7]));
    *reinterpret_cast<uint4*>(base + (((p0 + i) ^ (row & 7)) << 4)) = w;
  }
}

__device__ __forceinline__ int part_of_tile(const EncParams& p, int t) {
  int e = 0;
#pragma unroll
  for (int i = 1; i < 4; ++i)
    if (t >= (int)p.part[i].tile0) e = i;
  return e;
}

__global__ void __launch_bounds__(THREADS, 1)
encoder_kernel(const __grid_constant__ Maps m, EncParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sA = base, sH = base + SA_BYTES, ring = sH + SH_BYTES;
  uint8_t* sH_g = gen + SA_BYTES;
  uint8_t* stg_all = gen + SA_BYTES + SH_BYTES + STAGES * STAGE_BYTES;
  float* prm = reinterpret_cast<float*>(stg_all + EPI_WARPS * STG_BYTES);
  float2* part = reinterpret_cast<float2*>(stg_all + EPI_WARPS * STG_BYTES + PARAM_FLOATS * 4);
  Shared* sh = reinterpret_cast<Shared*>(stg_all + EPI_WARPS * STG_BYTES + PARAM_FLOATS * 4 + PART_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = p.d, KB = d >> 6, dh2 = d >> 1;
  volatile int* abort = &sh->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&sh->w_full[s]), 1);
      mbar_init(smem_u32(&sh->w_empty[s]), 1);
    }
    mbar_init(smem_u32(&sh->a_full), 1);
    mbar_init(smem_u32(&sh->a_free), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->acc1_full[b]), 1);
      mbar_init(smem_u32(&sh->acc2_full[b]), 1);
      mbar_init(smem_u32(&sh->acc_free[b]), EPI_WARPS);
    }
    mbar_init(smem_u32(&sh->h_ready), HID_WARPS);
    mbar_init(smem_u32(&sh->mma_done), 1);
    sh->abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&m.a);
    for (int e = 0; e < 4; ++e) {
      tma_prefetch_desc(&m.w0[e]);
      tma_prefetch_desc(&m.w1[e]);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh->tmem_base), 512);
    tmem_relinquish();
  }
  // per-column parameters: b0[e] at e * 256, b1[e] at (4 + e) * 256, gamma at 8 * 256, beta at 9 * 256
  for (int i = threadIdx.x; i < 10 * 256; i += THREADS) {
    const int which = i >> 8, c = i & 255;
    float v = which == 8 ? 1.f : 0.f;
    if (c < d) {
      const float* src = which < 4 ? p.b0[which] : which < 8 ? p.b1[which - 4] : which == 8 ? p.ln_g : p.ln_b;
      if (src) v = src[c];
    }
    prm[i] = v;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const uint32_t stage_bytes = (uint32_t)d * 128u;      // a (d x 64) fp16 weight tile

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      auto stage = [&](const CUtensorMap* map, int x0) -> bool {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(smem_u32(&sh->w_empty[s]), ph ^ 1, abort)) { give_up(sh, p.status, 1); return false; }
        const uint32_t bar = smem_u32(&sh->w_full[s]);
        mbar_expect_tx(bar, stage_bytes);
        tma_load_2d(ring + s * STAGE_BYTES, map, x0, 0, bar);
        ++it;
        return true;
      };
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++tile_i) {
        const int e = part_of_tile(p, t);
        const int64_t row0 = p.part[e].row0 + (int64_t)(t - (int)p.part[e].tile0) * BM;
        if (!mbar_wait(smem_u32(&sh->a_free), (tile_i & 1) ^ 1, abort)) { give_up(sh, p.status, 2); break; }
        const uint32_t bar = smem_u32(&sh->a_full);
        mbar_expect_tx(bar, SA_BYTES);
        tma_load_2d(sA, &m.a, 0, (int)row0, bar);
        ok = stage(&m.w0[e], 0);
        for (int kb = 0; kb < KB && ok; ++kb) ok = stage(&m.w1[e], 64 * kb);
      }
      // loads in flight must land before the CTA exits (bounded, ignoring abort)
      for (uint32_t j = it > STAGES ? it - STAGES : 0; j < it; ++j) {
        uint32_t spins = 0;
        while (!mbar_try_wait(smem_u32(&sh->w_full[j % STAGES]), (j / STAGES) & 1) && ++spins < kSpinLimit) {}
        if (spins >= kSpinLimit) give_up(sh, p.status, 3);
      }
      if (tile_i > 0) {
        uint32_t spins = 0;
        while (!mbar_try_wait(smem_u32(&sh->a_full), (tile_i - 1) & 1) && ++spins < kSpinLimit) {}
        if (spins >= kSpinLimit) give_up(sh, p.status, 4);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      const uint32_t idesc = idesc_f16(BM, d);
      // one ring stage: four K = 16 MMAs of A chunk x the staged (d x 64) weight tile
      auto kblock = [&](uint32_t a_addr, uint32_t d_tmem, bool acc_first) -> bool {
        const int s = it % STAGES;
        if (!mbar_wait(smem_u32(&sh->w_full[s]), (it / STAGES) & 1, abort)) { give_up(sh, p.status, 5); return false; }
        tc_fence_after();
        const uint64_t ad = smem_desc_sw128(a_addr), bd = smem_desc_sw128(ring + s * STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_f16_ss(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (acc_first || k) ? 1u : 0u);
        tc_commit(smem_u32(&sh->w_empty[s]));
        ++it;
        return true;
      };
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++tile_i) {
        const uint32_t par = tile_i & 1, b = tile_i & 1, use = (tile_i >> 1) & 1;
        const uint32_t acc = tmem_base + 256u * b;
        if (!mbar_wait(smem_u32(&sh->a_full), par, abort)) { give_up(sh, p.status, 6); break; }
        // this half of TMEM is free once the output warps have drained the tile before last
        if (!mbar_wait(smem_u32(&sh->acc_free[b]), use ^ 1, abort)) { give_up(sh, p.status, 7); break; }
        tc_fence_after();
        if (!kblock(sA, acc, false)) break;
        tc_commit(smem_u32(&sh->a_free));
        tc_commit(smem_u32(&sh->acc1_full[b]));
        // the second GEMM overwrites the first one's accumulator: the hidden warps must have read all of it
        if (!mbar_wait(smem_u32(&sh->h_ready), par, abort)) { give_up(sh, p.status, 9); break; }
        tc_fence_after();
        for (int kb = 0; kb < KB && ok; ++kb) ok = kblock(sH + kb * CHUNK_BYTES, acc, kb != 0);
        if (ok) tc_commit(smem_u32(&sh->acc2_full[b]));
      }
      tc_commit(smem_u32(&sh->mma_done));
      uint32_t spins = 0;
      while (!mbar_try_wait(smem_u32(&sh->mma_done), 0) && ++spins < kSpinLimit) {}
      if (spins >= kSpinLimit) give_up(sh, p.status, 10);
    }
  } else if (warp < FIRST_EPI) {
    // ------------------------------------------------------------ hidden warps, thread = row
    // layer 0: relu(acc + b0) -> the fp16 hidden tile, all d columns of this warp's 32 rows
    const int q = warp & 3;
    const int trow = q * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    const float4* prm4 = reinterpret_cast<const float4*>(prm);
    uint32_t tile_i = 0;
    for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, ++tile_i) {
      const uint32_t b = tile_i & 1, use = (tile_i >> 1) & 1;
      const float4* P_b0 = prm4 + part_of_tile(p, t) * 64;
      // the first GEMM of this tile was issued after the second GEMM of the tile before: its completion also
      // means that nothing reads the hidden tile any more
      if (!mbar_wait_warp(smem_u32(&sh->acc1_full[b]), use, abort)) {
        if (lane == 0) give_up(sh, p.status, 11);
        break;
      }
      tc_fence_after();
      for (int c = 0; c < d; c += 32) {
        uint32_t r[32];
        float v[32];
        tmem_ld32(lane_base + 256u * b + c, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 b0 = P_b0[(c >> 2) + j];
          v[4 * j] = fmaxf(__uint_as_float(r[4 * j]) + b0.x, 0.f);
          v[4 * j + 1] = fmaxf(__uint_as_float(r[4 * j + 1]) + b0.y, 0.f);
          v[4 * j + 2] = fmaxf(__uint_as_float(r[4 * j + 2]) + b0.z, 0.f);
          v[4 * j + 3] = fmaxf(__uint_as_float(r[4 * j + 3]) + b0.w, 0.f);
        }
        store_h32(sH_g, trow, c, v);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->h_ready));
    }
  } else {
    // ------------------------------------------------------------ output warps, thread = row
    const int ew = warp - FIRST_EPI;
    const int grp = ew >> 2;
    const int q = warp & 3;
    const int trow = q * 32 + lane;
    const uint32_t lane_q = tmem_base + ((uint32_t)(q * 32) << 16);
    uint8_t* stg = stg_all + ew * STG_BYTES;
    const int sub = lane >> 3, piece = lane & 7;            // transposed phase: row sub + 4 i, 16-byte piece
    const int c_lo = grp * dh2, c_hi = c_lo + dh2;
    const float4* prm4 = reinterpret_cast<const float4*>(prm);
    const float4 *P_g = prm4 + 8 * 64, *P_b = prm4 + 9 * 64;
    const float inv_d = 1.0f / (float)d;
    uint32_t tile_i = 0;
    for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, ++tile_i) {
      const uint32_t b = tile_i & 1, use = (tile_i >> 1) & 1;
      const uint32_t lane_base = lane_q + 256u * b;
      const int e = part_of_tile(p, t);
      const EncPart pe = p.part[e];
      const float4* P_b1 = prm4 + (4 + e) * 64;
      // x / h row offsets (elements) of the 8 rows this lane writes in the transposed phase; -1 past the end
      // (one division per tile, then steps of four rows that jump over the other encoders' slots at an env
      // boundary: eight 64-bit divisions here cost the epilogue ~2 K cycles per tile)
      int64_t orow[8];
      const int64_t r_tile = (int64_t)(t - (int)pe.tile0) * BM;
      {
        int slot;
        const int64_t env = div_index(r_tile + q * 32 + sub, pe.group, &slot);      // rows < 2^31 (checked on the host)
        int64_t off = (env * kT + pe.first + slot) * (int64_t)d;
        const int64_t rows_left = pe.rows - (r_tile + q * 32 + sub);
        const int step4 = 4 * d, jump = (kT - pe.group) * d;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          orow[i] = 4 * i < rows_left ? off : -1;
          slot += 4;
          off += step4;
          while (slot >= pe.group) {
            slot -= pe.group;
            off += jump;
          }
        }
      }
      // ---- layer 1: tok = acc + b1 -> x (fp32), row statistics
      if (!mbar_wait_warp(smem_u32(&sh->acc2_full[b]), use, abort)) {
        if (lane == 0) give_up(sh, p.status, 12);
        break;
      }
      tc_fence_after();
      float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f), q4 = s4;      // per-component partial sums: four short chains
      // 32 accumulator columns -> bias, statistics, fp32 staging block -> 16-byte stores covering full lines
      auto x_block = [&](const uint32_t (&r)[32], int c) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 b1 = P_b1[(c >> 2) + j];
          const float4 v = make_float4(__uint_as_float(r[4 * j]) + b1.x, __uint_as_float(r[4 * j + 1]) + b1.y,
                                       __uint_as_float(r[4 * j + 2]) + b1.z, __uint_as_float(r[4 * j + 3]) + b1.w);
          s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
          q4.x = fmaf(v.x, v.x, q4.x); q4.y = fmaf(v.y, v.y, q4.y); q4.z = fmaf(v.z, v.z, q4.z); q4.w = fmaf(v.w, v.w, q4.w);
          *reinterpret_cast<float4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (orow[i] < 0) continue;
          const int rr = i * 4 + sub;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((piece ^ (rr & 7)) << 4));
          *reinterpret_cast<uint4*>(p.x + orow[i] + c + piece * 4) = v;
        }
        __syncwarp();
      };
      for (int c = c_lo; c < c_hi; c += 32) {
        uint32_t r0[32];
        tmem_ld32(lane_base + c, r0);
        tmem_wait_ld();
        x_block(r0, c);
      }
      const float sum = (s4.x + s4.y) + (s4.z + s4.w), sq = (q4.x + q4.y) + (q4.z + q4.w);
      // ---- block 0's LayerNorm rows (fp16), second pass over the accumulator
      if (p.h) {
        part[grp * BM + trow] = make_float2(sum, sq);
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        const float2 o = part[(grp ^ 1) * BM + trow];
        const float mean = (sum + o.x) * inv_d;
        const float rstd = rsqrtf(fmaxf((sq + o.y) * inv_d - mean * mean, 0.f) + p.eps);
        const float shift = -mean * rstd;
        for (int c = c_lo; c < c_hi; c += 64) {             // 64 columns = 128 bytes of fp16 per row
          const int nc = c_hi - c < 64 ? c_hi - c : 64;     // 32 when the half is an odd number of 32s
#pragma unroll
          for (int s32 = 0; s32 < 64; s32 += 32) {
            if (s32 >= nc) break;
            uint32_t r[32];
            tmem_ld32(lane_base + c + s32, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 4; ++j) {                   // 8 columns -> one 16-byte piece
              float y[8];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int f4 = ((c + s32) >> 2) + 2 * j + u;
                const float4 b1 = P_b1[f4], g = P_g[f4], bb = P_b[f4];
                y[4 * u] = fmaf(fmaf(__uint_as_float(r[8 * j + 4 * u]) + b1.x, rstd, shift), g.x, bb.x);
                y[4 * u + 1] = fmaf(fmaf(__uint_as_float(r[8 * j + 4 * u + 1]) + b1.y, rstd, shift), g.y, bb.y);
                y[4 * u + 2] = fmaf(fmaf(__uint_as_float(r[8 * j + 4 * u + 2]) + b1.z, rstd, shift), g.z, bb.z);
                y[4 * u + 3] = fmaf(fmaf(__uint_as_float(r[8 * j + 4 * u + 3]) + b1.w, rstd, shift), g.w, bb.w);
              }
              *reinterpret_cast<uint4*>(stg + lane * 128 + ((((s32 >> 3) + j) ^ (lane & 7)) << 4)) =
                  make_uint4(pack_half2(y[0], y[1]), pack_half2(y[2], y[3]), pack_half2(y[4], y[5]), pack_half2(y[6], y[7]));
            }
          }
          __syncwarp();
          if (piece * 8 < nc) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (orow[i] < 0) continue;
              const int rr = i * 4 + sub;
              const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((piece ^ (rr & 7)) << 4));
              *reinterpret_cast<uint4*>(p.h + orow[i] + c + piece * 8) = v;
            }
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->acc_free[b]));
    }
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

bool encoder_fused_ok(const EncoderArgs& a) {
  if (a.d % 64 != 0 || a.d < 64 || a.d > 256) return false;
  if (a.n_envs < 1 || a.n_envs > 0x7fffff00LL / kT) return false;
  if (!aligned16(a.feat) || !aligned16(a.x) || (a.h && !aligned16(a.h))) return false;
  for (int e = 0; e < 4; ++e)
    if (!aligned16(a.w0[e]) || !aligned16(a.w1[e]) || a.k0[e] != 64) return false;
  return true;
}

int encoder_fused(const EncoderArgs& a, cudaStream_t stream) {
  if (!a.feat || !a.x) {
    set_error("encoder: NULL operand");
    return BSRL_ERR_NULL;
  }
  for (int e = 0; e < 4; ++e)
    if (!a.w0[e] || !a.w1[e] || !a.b0[e] || !a.b1[e]) {
      set_error("encoder: NULL weights of encoder %d", e);
      return BSRL_ERR_NULL;
    }
  if (!encoder_fused_ok(a)) {
    set_error("encoder: shape d=%d does not fit the fused kernel (d in {64, 128, 192, 256}, 64-wide padded inputs)", a.d);
    return BSRL_ERR_UNSUPPORTED;
  }
  int* status = device_status_ptr();
  if (!status) return BSRL_ERR_CUDA;
  const int64_t B = a.n_envs;
  Maps m;
  if (!make_tmap_f16(&m.a, a.feat, B * kT, 64, 64, BM)) return BSRL_ERR_CUDA;
  for (int e = 0; e < 4; ++e) {
    if (!make_tmap_f16(&m.w0[e], a.w0[e], a.d, 64, 64, a.d)) return BSRL_ERR_CUDA;
    if (!make_tmap_f16(&m.w1[e], a.w1[e], a.d, a.d, a.d, a.d)) return BSRL_ERR_CUDA;
  }
  static DeviceOnce once;
  int rc = once.run("encoder_kernel set-up", [] {
    return cudaFuncSetAttribute(encoder_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  if (rc != BSRL_OK) return rc;
  EncParams p;
  p.d = a.d;
  // encoders in the order of the feature matrix and of EncoderArgs: saber (2 rows per env, slots 0-1),
  // torso (1, slot 2), leg (2, slots 3-4), note (24, slots 5-28); tiles: the note tiles first
  const int64_t rows[4] = {2 * B, B, 2 * B, (int64_t)kSlots * B};
  const int group[4] = {2, 1, 2, kSlots}, first[4] = {0, 2, 3, kLead};
  int64_t row0 = 0;
  for (int e = 0; e < 4; ++e) {
    p.part[e].rows = rows[e];
    p.part[e].row0 = row0;
    p.part[e].group = group[e];
    p.part[e].first = first[e];
    row0 += rows[e];
    p.b0[e] = a.b0[e];
    p.b1[e] = a.b1[e];
  }
  // tile numbering must be monotone in the part index for part_of_tile: parts are numbered 0..3 in tile order
  // note, saber, torso, leg -> remap so that part[0] is the note encoder
  EncPart ordered[4] = {p.part[3], p.part[0], p.part[1], p.part[2]};
  const float* b0o[4] = {a.b0[3], a.b0[0], a.b0[1], a.b0[2]};
  const float* b1o[4] = {a.b1[3], a.b1[0], a.b1[1], a.b1[2]};
  Maps mo = m;
  const int src[4] = {3, 0, 1, 2};
  int64_t tile0 = 0;
  for (int i = 0; i < 4; ++i) {
    p.part[i] = ordered[i];
    p.part[i].tile0 = tile0;
    tile0 += (ordered[i].rows + BM - 1) / BM;
    p.b0[i] = b0o[i];
    p.b1[i] = b1o[i];
    mo.w0[i] = m.w0[src[i]];
    mo.w1[i] = m.w1[src[i]];
  }
  if (tile0 > 0x7fffffff) {
    set_error("encoder: too many tiles");
    return BSRL_ERR_SHAPE;
  }
  p.n_tiles = (int)tile0;
  p.ln_g = a.h ? a.ln_g : nullptr;
  p.ln_b = a.h ? a.ln_b : nullptr;
  p.eps = a.eps;
  p.x = a.x;
  p.h = a.h;
  p.status = status;
  const int grid = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
  encoder_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(mo, p);
  BSRL_LAUNCH_OK("encoder_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
