// Projection + residual + LayerNorm in one tcgen05 kernel, for rows too wide for the fused block tail
// (d = 512: the wide policy):
//
//   x_out = R + A W^T + b        (fp32 residual stream, N = d columns)
//   h     = LayerNorm(x_out)     (fp16 rows: the operand of the GEMM that follows)
//
// A 128-row tile of a 512-wide fp32 row fills all 512 TMEM columns, so there is no second accumulator
// buffer: the MMAs of a tile and its epilogue run one after the other, and the epilogue is what the kernel
// is made of -- it moves 5 KB per row (residual in, stream out, LayerNorm row out) against 2 N K FLOP, i.e.
// the kernel is HBM-bound for K = d and only worth having there.  What it saves is the separate LayerNorm
// pass (2 KB read + 1 KB written per row again) and the slower residual epilogue of the plain GEMM.
//
//   warp 0      TMA producer: stages of a (128 x 64) A chunk + the (N x 64) weight chunk, 2 stages
//   warp 1      MMA issuer: per 16-wide K step two tcgen05.mma (M = 128, N = 256) into the two column halves
//   warps 2..9  epilogue; warp w reads TMEM lane quadrant w & 3 and owns column half (w - 2) / 4:
//     pass 1    32 columns at a time: accumulator + bias, transposed through a 4 KB staging block so that the
//               residual is read and the stream written with 8 lanes per 128-byte line; row sums of x and
//               x^2 on the way; x goes back into TMEM for pass 2
//     exchange  the two warps that share a quadrant swap their half-row sums (a 64-thread named barrier)
//     pass 2    64 columns at a time: TMEM -> (x - mean) rstd gamma + beta -> fp16 -> staging -> one TMA store
//
// Statistics are fp32 sums of x and x^2 over pieces of 32 values, combined pairwise (lanes, then halves).
// Stands in for out_proj + ln_ffn.forward_add (python/policy.py:655-668; ln_fwd_add,
// python/beat_arena_env/csrc/layer_norm.cu) where the fused block tail does not reach.  All waits are bounded.
#include "kernels.cuh"
#include "tc5.cuh"

namespace bsrl {
namespace {
using namespace tc5;

constexpr int BM = 128, BK = 64, STAGES = 2;
constexpr int MAX_N = 512;
constexpr int A_BYTES = BM * BK * 2;             // 16 KB
constexpr int W_BYTES = MAX_N * BK * 2;          // 64 KB
constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = (2 + EPI_WARPS) * 32;
constexpr int STG_BYTES = 32 * 128;
constexpr int PRM_BYTES = 3 * MAX_N * 4;         // bias | gamma | beta
constexpr int PART_BYTES = 2 * BM * 8;           // per half and row: (sum, sum of squares)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * STG_BYTES + PRM_BYTES + PART_BYTES + 1024 + 256;
constexpr int KERNEL_ID = 6;

struct Shared {
  uint64_t full[STAGES], empty[STAGES], acc_full, acc_empty, mma_done;
  uint32_t tmem_base;
  int abort;
  int quit[4][2];   // abort as sampled by one thread of a quadrant's warp pair ahead of their barrier (per tile parity),
                    // so that both warps leave the tile loop at the same tile
};

struct Params {
  int N, K;
  int64_t M;
  const float* bias;
  const float* gamma;
  const float* beta;
  float eps;
  const float* R;     // (M, ldr) f32 residual
  int64_t ldr;
  float* x_out;       // (M, ldx) f32
  int64_t ldx;
  int n_tiles;
  int* status;
};

__device__ __forceinline__ void give_up(Shared* sh, int* status, int role) {
  atomicCAS(status, 0, KERNEL_ID * 16 + role);
  sh->abort = 1;
}

// 16-byte global load that stays where it is written (the compiler may not sink it to its first use)
__device__ __forceinline__ float4 ld_f4_here(const float* p) {
  float4 v;
  asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(THREADS, 1)
linear_ln_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                 const __grid_constant__ CUtensorMap tm_h, Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  uint8_t* staging = smem_raw + (ring - raw) + STAGES * STAGE_BYTES;
  float* prm = reinterpret_cast<float*>(staging + EPI_WARPS * STG_BYTES);
  float2* part = reinterpret_cast<float2*>(staging + EPI_WARPS * STG_BYTES + PRM_BYTES);
  Shared* sh = reinterpret_cast<Shared*>(staging + EPI_WARPS * STG_BYTES + PRM_BYTES + PART_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int N = p.N, k_blocks = p.K / BK, n_halves = N > 256 ? 2 : 1, NH = N / n_halves;   // NH: columns per half
  volatile int* abort = &sh->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    mbar_init(smem_u32(&sh->acc_full), 1);
    mbar_init(smem_u32(&sh->acc_empty), EPI_WARPS);
    mbar_init(smem_u32(&sh->mma_done), 1);
    sh->abort = 0;
    for (int i = 0; i < 8; ++i) (&sh->quit[0][0])[i] = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_h);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh->tmem_base), 512);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < N; i += THREADS) {
    prm[i] = p.bias ? p.bias[i] : 0.f;
    prm[MAX_N + i] = p.gamma[i];
    prm[2 * MAX_N + i] = p.beta[i];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const uint32_t stage_tx = (uint32_t)(A_BYTES + N * BK * 2);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(smem_u32(&sh->empty[s]), ((it / STAGES) & 1) ^ 1, abort)) { give_up(sh, p.status, 1); ok = false; break; }
          const uint32_t bar = smem_u32(&sh->full[s]);
          mbar_expect_tx(bar, stage_tx);
          const uint32_t dst = ring + s * STAGE_BYTES;
          tma_load_2d(dst, &tm_a, kb * BK, t * BM, bar);
          for (int hf = 0; hf < n_halves; ++hf) tma_load_2d(dst + A_BYTES + hf * NH * BK * 2, &tm_w, kb * BK, hf * NH, bar);
        }
      }
      for (uint32_t j = it > STAGES ? it - STAGES : 0; j < it; ++j) {   // loads in flight land before the CTA exits
        uint32_t spins = 0;
        while (!mbar_try_wait(smem_u32(&sh->full[j % STAGES]), (j / STAGES) & 1) && ++spins < kSpinLimit) {}
        if (spins >= kSpinLimit) give_up(sh, p.status, 2);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      const uint32_t idesc = idesc_f16(BM, NH);
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++tile_i) {
        if (!mbar_wait(smem_u32(&sh->acc_empty), (tile_i & 1) ^ 1, abort)) { give_up(sh, p.status, 3); ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(smem_u32(&sh->full[s]), (it / STAGES) & 1, abort)) { give_up(sh, p.status, 4); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = ring + s * STAGE_BYTES;
          const uint64_t ad = smem_desc_sw128(a_addr);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            for (int hf = 0; hf < n_halves; ++hf)
              mma_f16_ss(tmem_base + hf * 256, ad + 2 * k, smem_desc_sw128(a_addr + A_BYTES + hf * NH * BK * 2) + 2 * k, idesc,
                         (kb | k) ? 1u : 0u);
          tc_commit(smem_u32(&sh->empty[s]));
        }
        if (ok) tc_commit(smem_u32(&sh->acc_full));
      }
      tc_commit(smem_u32(&sh->mma_done));
      uint32_t spins = 0;
      while (!mbar_try_wait(smem_u32(&sh->mma_done), 0) && ++spins < kSpinLimit) {}
      if (spins >= kSpinLimit) give_up(sh, p.status, 6);
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int q = warp & 3, half = (warp - 2) >> 2;
    const bool active = half < n_halves;                 // N <= 256: the second group of warps only keeps the barriers company
    uint8_t* stg = staging + (warp - 2) * STG_BYTES;
    const int sub = lane >> 3, piece = lane & 7;
    const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + half * 256;
    const int col0 = half * NH;
    const float inv_n = 1.f / (float)N;
    uint32_t tile_i = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++tile_i) {
      const int64_t m0 = (int64_t)t * BM;
      int64_t rrow[8];                                   // rows this lane touches in the transposed phase, or -1
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t row = m0 + q * 32 + i * 4 + sub;
        rrow[i] = row < p.M ? row : -1;
      }
      // a failed wait does not leave the loop here: the warp goes on (on garbage) to the pair barrier, where both
      // warps of the quadrant take the same decision
      if (!mbar_wait_warp(smem_u32(&sh->acc_full), tile_i & 1, abort) && lane == 0) give_up(sh, p.status, 5);
      tc_fence_after();
      float s1[8], s2[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) s1[i] = s2[i] = 0.f;
      // ---- pass 1: x = acc + bias + R, written out and kept in TMEM; row sums
      if (active) {
        // the residual pieces of a block are asked for one block ahead: read on demand they arrive at DRAM
        // latency with one block's worth of loads in flight, and this loop is most of the kernel
        float4 rv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          rv[i] = rrow[i] >= 0 ? ld_f4_here(p.R + rrow[i] * p.ldr + col0 + piece * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int c = 0; c < NH; c += 32) {
          const int col = col0 + c, pc = col + piece * 4;
          float4 rn[8];
          if (c + 32 < NH) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              rn[i] = rrow[i] >= 0 ? ld_f4_here(p.R + rrow[i] * p.ldr + pc + 32) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
          uint32_t r[32];
          tmem_ld32(tbase + c, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 bv = *reinterpret_cast<const float4*>(prm + col + 4 * j);
            *reinterpret_cast<float4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_float4(__uint_as_float(r[4 * j]) + bv.x, __uint_as_float(r[4 * j + 1]) + bv.y,
                            __uint_as_float(r[4 * j + 2]) + bv.z, __uint_as_float(r[4 * j + 3]) + bv.w);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + sub;
            float4* sp = reinterpret_cast<float4*>(stg + rr * 128 + ((piece ^ (rr & 7)) << 4));
            float4 f = *sp;
            f.x += rv[i].x; f.y += rv[i].y; f.z += rv[i].z; f.w += rv[i].w;
            *sp = f;
            s1[i] += (f.x + f.y) + (f.z + f.w);
            s2[i] += (f.x * f.x + f.y * f.y) + (f.z * f.z + f.w * f.w);
            if (rrow[i] >= 0) *reinterpret_cast<float4*>(p.x_out + rrow[i] * p.ldx + pc) = f;
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 f = *reinterpret_cast<const float4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4));
            r[4 * j] = __float_as_uint(f.x); r[4 * j + 1] = __float_as_uint(f.y);
            r[4 * j + 2] = __float_as_uint(f.z); r[4 * j + 3] = __float_as_uint(f.w);
          }
          tmem_st32(tbase + c, r);
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) rv[i] = rn[i];
        }
        tmem_wait_st();
        // the 8 lanes of a row add up their pieces; lane piece 0 publishes the half-row sums
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
          for (int o = 1; o < 8; o <<= 1) {
            s1[i] += __shfl_xor_sync(0xffffffffu, s1[i], o);
            s2[i] += __shfl_xor_sync(0xffffffffu, s2[i], o);
          }
          if (piece == 0) part[half * BM + q * 32 + i * 4 + sub] = make_float2(s1[i], s2[i]);
        }
      }
      if (half == 0 && lane == 0) sh->quit[q][tile_i & 1] = *abort;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");        // the quadrant's two warps: half-row sums are in
      const bool quit = *reinterpret_cast<volatile int*>(&sh->quit[q][tile_i & 1]) != 0;
      // ---- pass 2: thread = row again: normalise, fp16, 64 columns per TMA store
      if (active && !quit) {
        const int trow = q * 32 + lane;
        float2 a = part[trow];
        if (n_halves == 2) {
          const float2 b = part[BM + trow];
          a.x += b.x; a.y += b.y;
        }
        const float mean = a.x * inv_n;
        const float rstd = rsqrtf(fmaxf(a.y * inv_n - mean * mean, 0.f) + p.eps);
#pragma unroll 1
        for (int c = 0; c < NH; c += 64) {
          const int col = col0 + c;
          uint32_t r[32];
          if (c > 0) {                      // the previous block's TMA store has read the staging buffer
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
          }
#pragma unroll
          for (int s32 = 0; s32 < 64; s32 += 32) {
            tmem_ld32(tbase + c + s32, r);
            tmem_wait_ld();
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 g = *reinterpret_cast<const float4*>(prm + MAX_N + col + s32 + j);
              const float4 b = *reinterpret_cast<const float4*>(prm + 2 * MAX_N + col + s32 + j);
              v[j] = (__uint_as_float(r[j]) - mean) * rstd * g.x + b.x;
              v[j + 1] = (__uint_as_float(r[j + 1]) - mean) * rstd * g.y + b.y;
              v[j + 2] = (__uint_as_float(r[j + 2]) - mean) * rstd * g.z + b.z;
              v[j + 3] = (__uint_as_float(r[j + 3]) - mean) * rstd * g.w + b.w;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(stg + lane * 128 + ((((s32 >> 3) + j) ^ (lane & 7)) << 4)) =
                  make_uint4(pack_half2(v[8 * j], v[8 * j + 1]), pack_half2(v[8 * j + 2], v[8 * j + 3]),
                             pack_half2(v[8 * j + 4], v[8 * j + 5]), pack_half2(v[8 * j + 6], v[8 * j + 7]));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && m0 + q * 32 < p.M) {
            tma_store_2d(&tm_h, col, (int)(m0 + q * 32), smem_u32(stg));
            bulk_commit();
          }
        }
        if (lane == 0) bulk_wait_read<0>();    // pass 1 of the next tile writes the staging buffer with plain stores
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty));
      if (quit) ok = false;
    }
    if (lane == 0) bulk_wait_all();
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

bool linear_ln_ok(const LinearLnArgs& a) {
  if (!a.A || !a.W || !a.R || !a.x_out || !a.h || !a.gamma || !a.beta || a.M < 1) return false;
  if (a.N % 64 != 0 || a.N < 64 || a.N > MAX_N || (a.N > 256 && a.N % 128 != 0) || a.K % BK != 0 || a.K < BK) return false;
  if (!aligned16(a.A) || !aligned16(a.W) || !aligned16(a.R) || !aligned16(a.x_out) || !aligned16(a.h)) return false;
  if ((a.lda % 8) || (a.ldw % 8) || (a.ldr % 4) || (a.ldx % 4) || (a.ldh % 8)) return false;
  if ((a.bias && !aligned16(a.bias)) || a.M > 0x7fffff00) return false;
  return true;
}

int linear_ln(const LinearLnArgs& a, cudaStream_t stream) {
  if (!linear_ln_ok(a)) {
    set_error("linear_ln: shape m=%lld n=%d k=%d does not fit (n a multiple of 64 up to 512, k a multiple of 64, aligned rows)",
              (long long)a.M, a.N, a.K);
    return BSRL_ERR_UNSUPPORTED;
  }
  int* status = device_status_ptr();
  if (!status) return BSRL_ERR_CUDA;
  const int NH = a.N > 256 ? a.N / 2 : a.N;
  CUtensorMap tm_a, tm_w, tm_h;
  if (!make_tmap_f16(&tm_a, a.A, a.M, a.K, a.lda, BM)) return BSRL_ERR_CUDA;
  if (!make_tmap_f16(&tm_w, a.W, a.N, a.K, a.ldw, NH)) return BSRL_ERR_CUDA;
  if (!make_tmap_rows(&tm_h, a.h, 2, a.M, a.N, a.ldh, 32, 128)) return BSRL_ERR_CUDA;
  static DeviceOnce once;
  int rc = once.run("linear_ln_kernel set-up", [] {
    return cudaFuncSetAttribute(linear_ln_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  if (rc != BSRL_OK) return rc;
  Params p;
  p.N = a.N; p.K = a.K; p.M = a.M;
  p.bias = a.bias; p.gamma = a.gamma; p.beta = a.beta; p.eps = a.eps;
  p.R = a.R; p.ldr = a.ldr; p.x_out = a.x_out; p.ldx = a.ldx;
  p.n_tiles = (int)((a.M + BM - 1) / BM);
  p.status = status;
  const int grid = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
  linear_ln_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tm_a, tm_w, tm_h, p);
  BSRL_LAUNCH_OK("linear_ln_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
