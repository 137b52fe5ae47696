// Fused tail of one transformer block on tcgen05 / TMEM, one 128-row token tile at a time:
//
//   x1   = x + att Wo^T + bo                      (attention out-projection + residual)
//   h2   = LN_ffn(x1)                             (fp32 statistics, fp16 operand)
//   xo   = x1 + relu(h2 W0^T + b0) W2^T + b2      (FFN; the 4d-wide hidden never leaves the SM)
//   out  : xo (fp32, optional), and up to two fp16 rows  LN_a(xo), LN_b(xo)  or plain fp16(xo)
//
// This is the reference's out_proj + ln_ffn.forward_add + fused_ffn(+ next LayerNorm) chain
// (python/policy.py:655-715; ffn_fused_kernel, python/beat_arena_env/csrc/fused_ffn.cu:242-485)
// as ONE kernel.  HBM traffic per token: read att (2d B) + x (4d B), write xo (4d B) + LN rows
// (2d B each) -- against 18 d^2 FLOP, i.e. tensor-bound.
//
// Layout of one CTA (persistent, one per SM, 352 threads):
//   warp 0       TMA producer of the weight tiles: a 3-stage ring of 32 KB stages, in the MMA's
//                consumption order
//   warp 10      TMA producer of the attention tiles (att tile -> sA, d/64 chunks of [128 x 64], 128B
//                swizzle; sA is freed before the tile ends); pulls the next tile's residual rows into L2
//   warp 1       MMA issuer (one thread): tcgen05.mma, M = 128, K = 16
//   warps 2..9   epilogue (two groups of four warps, each group owns half of the columns), thread = row:
//                LayerNorm on TMEM rows -> h2 into sA; bias + ReLU of each 128-wide hidden chunk -> sH;
//                final drain and LayerNorm outputs.  Global traffic moves as per-warp TMA boxes (32 rows
//                x 64 bytes) through three 2 KB swizzled buffers per warp -- residual rows in, fp32 and
//                fp16 rows out; rows gathered through a row map fall back to coalesced loads through
//                the staging buffer.  The per-column parameters live in shared memory.
// TMEM (512 columns): region X (d columns) accumulates x1 and then xo in place -- x is
// pre-stored there by the epilogue warps, so the out-projection and the FFN-down MMAs simply
// accumulate onto it; the other 256 columns are two 128-column buffers for hidden chunks.  The
// two regions swap roles every tile, so the next tile's x can be pre-stored and its
// out-projection issued while this tile drains.
//
// Every wait is bounded (see tc5.cuh); on expiry the status word is set and all roles fall
// through to the teardown.
#include <type_traits>

#include "kernels.cuh"
#include "tc5.cuh"

namespace bsrl {
namespace {
using namespace tc5;

constexpr int BM = 128;          // rows per tile
constexpr int HC = 128;          // hidden chunk width
constexpr int STAGES = 3, STAGE_BYTES = 32768;   // weight ring
constexpr int RING_BYTES = STAGES * STAGE_BYTES;
constexpr int CHUNK_BYTES = BM * 64 * 2;   // one [128 x 64] fp16 swizzled chunk
constexpr int SA_BYTES = 4 * CHUNK_BYTES;  // d <= 256
constexpr int SH_BYTES = 2 * CHUNK_BYTES;  // one 128 x 128 hidden chunk
constexpr int EPI_WARPS = 8;                     // two groups of four: each group owns half of the columns
constexpr int PROD_WARP = 2 + EPI_WARPS;         // attention-tile producer / L2 prefetcher
constexpr int THREADS = (3 + EPI_WARPS) * 32;
constexpr int STG_BYTES = 32 * 64;               // per-warp transposition buffer (32 rows x 64 B)
constexpr int PARAM_FLOATS = 8 * 256 + 1024;     // bo, ln_g, ln_b, b2, g16[2], b16[2] (d each) + b0 (F)
constexpr int PART_BYTES = 2 * 2 * BM * 8;       // LayerNorm partial sums exchanged between the two groups
constexpr int SMEM_BYTES = SA_BYTES + SH_BYTES + RING_BYTES + EPI_WARPS * STG_BYTES + PARAM_FLOATS * 4 +
                           PART_BYTES + 1024 + 256;
constexpr int KERNEL_ID = 2;

struct Shared {
  uint64_t w_full[STAGES], w_empty[STAGES];
  uint64_t a_full, a_free, x_ready, o_done, h2_ready, x_done, mma_done;
  uint64_t acc1_full[2], hid_ready[2], hid_free[2];   // hid_*: per 64-column half of the hidden chunk
  uint64_t io_full[EPI_WARPS][3];                     // per epilogue warp: residual blocks landed in its buffers
  uint32_t tmem_base;
  int abort;
};

struct TailParams {
  int d, F;                 // embed, FFN hidden
  int64_t M;                // rows
  const float* x;           // residual in (fp32), rows mapped by xmap
  int64_t ldx;
  RowMap xmap;
  const float* bo;          // (d)
  const float* ln_g;        // ln_ffn gamma / beta (d)
  const float* ln_b;
  const float* b0;          // (F)
  const float* b2;          // (d)
  float eps;
  float* x_out;             // (M, d) fp32 or nullptr
  // up to two fp16 outputs: LayerNorm(xo) with (g, b), or plain fp16(xo) when g == nullptr
  __half* out16[2];
  int64_t ld16[2];
  const float* g16[2];
  const float* b16[2];
  int n_tiles;
  int x_tma;                // residual rows are read with TMA (identity row map)
  int* status;
};

__device__ __forceinline__ void give_up(Shared* sh, int* status, int role) {
  atomicCAS(status, 0, KERNEL_ID * 16 + role);
  sh->abort = 1;
}

#define TAIL_WAIT_WARP(bar, parity, role)                          \
  if (!mbar_wait_warp(smem_u32(bar), (parity), abort)) {           \
    if ((threadIdx.x & 31) == 0) give_up(sh, p.status, role);      \
    ok = false;                                                    \
    break;                                                         \
  }

#define TAIL_WAIT(bar, parity, role)                               \
  if (!mbar_wait(smem_u32(bar), (parity), abort)) {                \
    give_up(sh, p.status, role);                                   \
    ok = false;                                                    \
    break;                                                         \
  }

// four MMAs (K = 64) of one k-block: A chunk and B tile both [rows x 64] swizzled
__device__ __forceinline__ void mma_kblock(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc,
                                           bool acc_first) {
  const uint64_t ad = smem_desc_sw128(a_addr), bd = smem_desc_sw128(b_addr);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    mma_f16_ss(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (acc_first || k) ? 1u : 0u);
  }
}

// the same four MMAs from ready-made descriptors; `fresh`: the first one overwrites the accumulator
__device__ __forceinline__ void mma_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void mma_kblock_desc(uint32_t d_tmem, uint64_t ad, uint64_t bd, uint32_t idesc, bool fresh) {
  if (fresh) mma_f16_ss(d_tmem, ad, bd, idesc, 0u);
  else mma_acc(d_tmem, ad, bd, idesc);
  mma_acc(d_tmem, ad + 2, bd + 2, idesc);
  mma_acc(d_tmem, ad + 4, bd + 4, idesc);
  mma_acc(d_tmem, ad + 6, bd + 6, idesc);
}
template <int N>
using StageNo = std::integral_constant<int, N>;

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

// GELU: the FFN activation is the exact GELU instead of ReLU (a compile-time variant: the hidden-chunk
// epilogue sits on the chunk loop's critical path)
template <bool GELU>
__global__ void __launch_bounds__(THREADS, 1)
block_tail_kernel(const __grid_constant__ CUtensorMap tm_att, const __grid_constant__ CUtensorMap tm_wo,
                  const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w2,
                  const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_xo,
                  const __grid_constant__ CUtensorMap tm_o0, const __grid_constant__ CUtensorMap tm_o1,
                  TailParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  // tiles of this CTA: tile0, tile0 + tstep, ... < t_end
  // (kept as expressions of the unsigned special registers rather than int variables: the
  // kernel measured 11 % slower with them held in signed locals)
#define tile0 ((int)blockIdx.x)
#define tstep (gridDim.x)
#define t_end (p.n_tiles)
  const uint32_t sA = base, sH = base + SA_BYTES, ring = sH + SH_BYTES;
  uint8_t* sA_g = gen;
  uint8_t* sH_g = gen + SA_BYTES;
  uint8_t* stg_all = gen + SA_BYTES + SH_BYTES + RING_BYTES;
  float* prm = reinterpret_cast<float*>(stg_all + EPI_WARPS * STG_BYTES);
  float2* part = reinterpret_cast<float2*>(stg_all + EPI_WARPS * STG_BYTES + PARAM_FLOATS * 4);
  Shared* sh = reinterpret_cast<Shared*>(stg_all + EPI_WARPS * STG_BYTES + PARAM_FLOATS * 4 + PART_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = p.d, KB = d >> 6, NC = p.F / HC, S1 = (KB + 1) >> 1;
  volatile int* abort = &sh->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&sh->w_full[s]), 1);
      mbar_init(smem_u32(&sh->w_empty[s]), 1);
    }
    mbar_init(smem_u32(&sh->a_full), 1);
    mbar_init(smem_u32(&sh->a_free), 1);
    mbar_init(smem_u32(&sh->x_ready), EPI_WARPS);
    mbar_init(smem_u32(&sh->o_done), 1);
    mbar_init(smem_u32(&sh->h2_ready), EPI_WARPS);
    mbar_init(smem_u32(&sh->x_done), 1);
    mbar_init(smem_u32(&sh->mma_done), 1);
    for (int b = 0; b < 2; ++b) mbar_init(smem_u32(&sh->acc1_full[b]), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->hid_ready[b]), 4);
      mbar_init(smem_u32(&sh->hid_free[b]), 1);
    }
    for (int w = 0; w < EPI_WARPS; ++w)
      for (int b = 0; b < 3; ++b) mbar_init(smem_u32(&sh->io_full[w][b]), 1);
    sh->abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_att);
    tma_prefetch_desc(&tm_wo);
    tma_prefetch_desc(&tm_w0);
    tma_prefetch_desc(&tm_w2);
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_xo);
    tma_prefetch_desc(&tm_o0);
    tma_prefetch_desc(&tm_o1);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh->tmem_base), 512);
    tmem_relinquish();
  }
  // per-column parameters into shared memory: [bo | ln_g | ln_b | b2 | g16_0 | b16_0 | g16_1 | b16_1] (256
  // floats each) then b0 (F floats); absent vectors read as gamma = 1, beta = 0
  for (int i = threadIdx.x; i < 8 * 256; i += THREADS) {
    const int which = i >> 8, c = i & 255;
    float v = (which == 4 || which == 6) ? 1.f : 0.f;
    if (c < d) {
      const float* src = which == 0 ? p.bo : which == 1 ? p.ln_g : which == 2 ? p.ln_b : which == 3 ? p.b2
                       : which == 4 ? p.g16[0] : which == 5 ? p.b16[0] : which == 6 ? p.g16[1] : p.b16[1];
      if (src) v = src[c];
    }
    prm[i] = v;
  }
  for (int i = threadIdx.x; i < p.F; i += THREADS) prm[8 * 256 + i] = p.b0[i];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const int rows_d = d;          // weight rows of an N = d tile
  const int rows_h = HC;         // ... of an N = 128 tile

  if (warp == 0) {
    // ------------------------------------------------------------ weight producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      // one ring stage: wait for it to be free, arm the barrier, issue the loads
      auto stage = [&](const CUtensorMap* map, int x0, int y0, int n_loads, uint32_t bytes_each) -> bool {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(smem_u32(&sh->w_empty[s]), ph ^ 1, abort)) { give_up(sh, p.status, 1); return false; }
        const uint32_t bar = smem_u32(&sh->w_full[s]);
        mbar_expect_tx(bar, bytes_each * n_loads);
        for (int i = 0; i < n_loads; ++i)
          tma_load_2d(ring + s * STAGE_BYTES + i * bytes_each, map, x0 + i * 64, y0, bar);
        ++it;
        return true;
      };
      auto g1 = [&](int j) -> bool {   // W0 rows [128 j, +128), two k-blocks per stage
        for (int i = 0; i < S1; ++i) {
          const int n = (2 * i + 1 < KB) ? 2 : 1;
          if (!stage(&tm_w0, 128 * i, HC * j, n, rows_h * 128)) return false;
        }
        return true;
      };
      for (int t = tile0; t < t_end && ok; t += tstep) {
        for (int kb = 0; kb < KB && ok; ++kb) ok = stage(&tm_wo, 64 * kb, 0, 1, rows_d * 128);
        ok = ok && g1(0) && g1(1);
        for (int j = 0; j < NC && ok; ++j) {
          for (int kc = 0; kc < 2 && ok; ++kc) ok = stage(&tm_w2, HC * j + 64 * kc, 0, 1, rows_d * 128);
          if (ok && j + 2 < NC) ok = g1(j + 2);
        }
      }
      // loads in flight must land before the CTA exits (bounded, ignoring abort)
      for (uint32_t j = it > STAGES ? it - STAGES : 0; j < it; ++j) {
        uint32_t spins = 0;
        while (!mbar_try_wait(smem_u32(&sh->w_full[j % STAGES]), (j / STAGES) & 1) && ++spins < kSpinLimit) {}
        if (spins >= kSpinLimit) give_up(sh, p.status, 2);
      }
    }
  } else if (warp == PROD_WARP) {
    // ------------------------------------------------------------ attention-tile producer
    // lane 0 loads the attention tile into sA as soon as the previous tile's last reader is done;
    // the whole warp then pulls the NEXT tile's residual rows into L2, so that the epilogue's
    // pre-store of x finds them there.
    uint32_t tile_i = 0;
    bool ok = true;
    for (int t = tile0; t < t_end && ok; t += tstep, ++tile_i) {
      if (!mbar_wait_warp(smem_u32(&sh->a_free), (tile_i & 1) ^ 1, abort)) {
        if (lane == 0) give_up(sh, p.status, 3);
        ok = false;
        break;
      }
      if (lane == 0) {
        const uint32_t bar = smem_u32(&sh->a_full);
        mbar_expect_tx(bar, KB * CHUNK_BYTES);
        for (int c = 0; c < KB; ++c) tma_load_2d(sA + c * CHUNK_BYTES, &tm_att, 64 * c, t * BM, bar);
      }
      const int tn = t + tstep;
      if (tn < t_end) {
        for (int r = lane; r < BM; r += 32) {
          const int64_t row = (int64_t)tn * BM + r;
          if (row < p.M) {
            const float* xr = p.x + p.xmap.plain(row) * p.ldx;
            for (int c = 0; c < d; c += 32) prefetch_l2(xr + c);
          }
        }
      }
    }
    if (lane == 0 && tile_i > 0) {
      uint32_t spins = 0;
      while (!mbar_try_wait(smem_u32(&sh->a_full), (tile_i - 1) & 1) && ++spins < kSpinLimit) {}
      if (spins >= kSpinLimit) give_up(sh, p.status, 4);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tile_i = 0, n_hid = 0;
      bool ok = true;
      const uint32_t idesc_d = idesc_f16(BM, d), idesc_h = idesc_f16(BM, HC);
      // completion of the MMAs issued so far -> the barrier
      auto commit = [&](uint64_t* bar) { tc_commit(smem_u32(bar)); };
      // consume one ring stage: wait, run `body(stage address)`, release the stage
      auto with_stage = [&](auto&& body) -> bool {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(smem_u32(&sh->w_full[s]), ph, abort)) { give_up(sh, p.status, 5); return false; }
        tc_fence_after();
        body(ring + s * STAGE_BYTES);
        commit(&sh->w_empty[s]);
        ++it;
        return true;
      };
      // ---- the widest shape (d = 256, F = 1024: 36 ring stages per tile = 12 whole turns of the ring): every stage's
      // ring slot and barrier phase are compile-time constants and the operand descriptors are built once.  The
      // issuing thread is the bottleneck of the chunk loop -- an MMA costs it ~50 cycles, a wait 16, a commit 44 --
      // and the general loop below spends as much again on index arithmetic and descriptor set-up (chunk loop
      // replayed without dependencies: 2,960 cycles per chunk with the general loop, 2,280 with this one).
      if (KB == 4 && NC == 8) {
        const uint64_t rd0 = smem_desc_sw128(ring), ad0 = smem_desc_sw128(sA), hd0 = smem_desc_sw128(sH);
        const uint32_t wf0 = smem_u32(&sh->w_full[0]), we0 = smem_u32(&sh->w_empty[0]);
        constexpr uint64_t kSlot = STAGE_BYTES >> 4, kChunk = CHUNK_BYTES >> 4;   // descriptor address units
        // wait for ring stage n (tile-relative): slot n % 3, phase (n / 3) & 1
        auto wait_stage = [&](auto n_) -> bool {
          constexpr int n = decltype(n_)::value;
          if (!mbar_wait(wf0 + 8u * (n % 3), (uint32_t)((n / 3) & 1), abort)) { give_up(sh, p.status, 5); return false; }
          tc_fence_after();
          return true;
        };
        auto release_stage = [&](auto n_) { tc_commit(we0 + 8u * (decltype(n_)::value % 3)); };
        // FFN-up of one hidden chunk: two stages of two k-blocks each, N = 128
        auto up = [&](auto n_, uint32_t dst, uint64_t* acc1_bar) -> bool {
          constexpr int n = decltype(n_)::value;
          if (!wait_stage(StageNo<n>{})) return false;
          mma_kblock_desc(dst, ad0, rd0 + kSlot * (n % 3), idesc_h, true);
          mma_kblock_desc(dst, ad0 + kChunk, rd0 + kSlot * (n % 3) + kChunk, idesc_h, false);
          release_stage(StageNo<n>{});
          if (!wait_stage(StageNo<n + 1>{})) return false;
          mma_kblock_desc(dst, ad0 + 2 * kChunk, rd0 + kSlot * ((n + 1) % 3), idesc_h, false);
          mma_kblock_desc(dst, ad0 + 3 * kChunk, rd0 + kSlot * ((n + 1) % 3) + kChunk, idesc_h, false);
          release_stage(StageNo<n + 1>{});
          tc_commit(smem_u32(acc1_bar));
          return true;
        };
        // FFN-down of one hidden chunk: its two 64-column halves as the epilogue publishes them, N = 256
        auto down = [&](auto n_, uint32_t xcol, uint32_t hid_par) -> bool {
          constexpr int n = decltype(n_)::value;
          if (!mbar_wait(smem_u32(&sh->hid_ready[0]), hid_par, abort)) { give_up(sh, p.status, 9); return false; }
          if (!wait_stage(StageNo<n>{})) return false;
          mma_kblock_desc(xcol, hd0, rd0 + kSlot * (n % 3), idesc_d, false);
          release_stage(StageNo<n>{});
          tc_commit(smem_u32(&sh->hid_free[0]));
          if (!mbar_wait(smem_u32(&sh->hid_ready[1]), hid_par, abort)) { give_up(sh, p.status, 9); return false; }
          if (!wait_stage(StageNo<n + 1>{})) return false;
          mma_kblock_desc(xcol, hd0 + kChunk, rd0 + kSlot * ((n + 1) % 3), idesc_d, false);
          release_stage(StageNo<n + 1>{});
          tc_commit(smem_u32(&sh->hid_free[1]));
          return true;
        };
        for (int t = tile0; t < t_end && ok; t += tstep, ++tile_i) {
          const uint32_t par = tile_i & 1;
          const uint32_t xcol = tmem_base + (par ? 256u : 0u);     // region X of this tile
          const uint32_t acol = tmem_base + (par ? 0u : 256u);     // two hidden-chunk buffers
          TAIL_WAIT(&sh->a_full, par, 6);
          TAIL_WAIT(&sh->x_ready, par, 7);
          tc_fence_after();
          // x1 = x (pre-stored) + att Wo^T: stages 0..3
          ok = wait_stage(StageNo<0>{});
          if (!ok) break;
          mma_kblock_desc(xcol, ad0, rd0, idesc_d, false);
          release_stage(StageNo<0>{});
          ok = wait_stage(StageNo<1>{});
          if (!ok) break;
          mma_kblock_desc(xcol, ad0 + kChunk, rd0 + kSlot, idesc_d, false);
          release_stage(StageNo<1>{});
          ok = wait_stage(StageNo<2>{});
          if (!ok) break;
          mma_kblock_desc(xcol, ad0 + 2 * kChunk, rd0 + 2 * kSlot, idesc_d, false);
          release_stage(StageNo<2>{});
          ok = wait_stage(StageNo<3>{});
          if (!ok) break;
          mma_kblock_desc(xcol, ad0 + 3 * kChunk, rd0, idesc_d, false);
          release_stage(StageNo<3>{});
          commit(&sh->o_done);
          TAIL_WAIT(&sh->h2_ready, par, 8);
          tc_fence_after();
          // hidden chunks 0 and 1: stages 4..7
          ok = up(StageNo<4>{}, acol, &sh->acc1_full[0]) && up(StageNo<6>{}, acol + HC, &sh->acc1_full[1]);
          // chunks j = 3 g + {0, 1, 2}: FFN-down of chunk j, then FFN-up of chunk j + 2 (12 stages = 4 turns of the ring
          // per g: slots and phases repeat); the hidden-chunk barriers complete once per chunk: parity j & 1
          for (uint32_t g = 0; g < 2 && ok; ++g) {
            ok = down(StageNo<8>{}, xcol, g & 1) && up(StageNo<10>{}, acol + ((g & 1) ? HC : 0), &sh->acc1_full[g & 1]) &&
                 down(StageNo<12>{}, xcol, (g & 1) ^ 1) && up(StageNo<14>{}, acol + ((g & 1) ? 0 : HC), &sh->acc1_full[(g & 1) ^ 1]) &&
                 down(StageNo<16>{}, xcol, g & 1) && up(StageNo<18>{}, acol + ((g & 1) ? HC : 0), &sh->acc1_full[g & 1]);
          }
          if (!ok) break;
          commit(&sh->a_free);                                     // the last reader of h2 (chunk 7's FFN-up) is issued
          // chunks 6 and 7: FFN-down only, stages 32..35
          ok = down(StageNo<32>{}, xcol, 0u) && down(StageNo<34>{}, xcol, 1u);
          if (ok) commit(&sh->x_done);
          it += 36;
          n_hid += 8;
        }
      } else if (KB == 3 && NC == 6) {
        // ---- d = 192, F = 768 (the reference's production width): 27 ring stages per tile = 9 whole turns of the
        // ring, an odd number: the slots repeat from tile to tile, the phases alternate with the tile's parity
        const uint64_t rd0 = smem_desc_sw128(ring), ad0 = smem_desc_sw128(sA), hd0 = smem_desc_sw128(sH);
        const uint32_t wf0 = smem_u32(&sh->w_full[0]), we0 = smem_u32(&sh->w_empty[0]);
        constexpr uint64_t kSlot = STAGE_BYTES >> 4, kChunk = CHUNK_BYTES >> 4;   // descriptor address units
        uint32_t flip = 0;                                          // tile parity: phase of stage n is ((n / 3) & 1) ^ flip
        auto wait_stage = [&](auto n_) -> bool {
          constexpr int n = decltype(n_)::value;
          if (!mbar_wait(wf0 + 8u * (n % 3), (uint32_t)((n / 3) & 1) ^ flip, abort)) { give_up(sh, p.status, 5); return false; }
          tc_fence_after();
          return true;
        };
        auto release_stage = [&](auto n_) { tc_commit(we0 + 8u * (decltype(n_)::value % 3)); };
        // FFN-up of one hidden chunk: k-blocks 0 and 1 from one stage, k-block 2 from the next, N = 128
        auto up = [&](auto n_, uint32_t dst, uint64_t* acc1_bar) -> bool {
          constexpr int n = decltype(n_)::value;
          if (!wait_stage(StageNo<n>{})) return false;
          mma_kblock_desc(dst, ad0, rd0 + kSlot * (n % 3), idesc_h, true);
          mma_kblock_desc(dst, ad0 + kChunk, rd0 + kSlot * (n % 3) + kChunk, idesc_h, false);
          release_stage(StageNo<n>{});
          if (!wait_stage(StageNo<n + 1>{})) return false;
          mma_kblock_desc(dst, ad0 + 2 * kChunk, rd0 + kSlot * ((n + 1) % 3), idesc_h, false);
          release_stage(StageNo<n + 1>{});
          tc_commit(smem_u32(acc1_bar));
          return true;
        };
        auto down = [&](auto n_, uint32_t xcol, uint32_t hid_par) -> bool {
          constexpr int n = decltype(n_)::value;
          if (!mbar_wait(smem_u32(&sh->hid_ready[0]), hid_par, abort)) { give_up(sh, p.status, 9); return false; }
          if (!wait_stage(StageNo<n>{})) return false;
          mma_kblock_desc(xcol, hd0, rd0 + kSlot * (n % 3), idesc_d, false);
          release_stage(StageNo<n>{});
          tc_commit(smem_u32(&sh->hid_free[0]));
          if (!mbar_wait(smem_u32(&sh->hid_ready[1]), hid_par, abort)) { give_up(sh, p.status, 9); return false; }
          if (!wait_stage(StageNo<n + 1>{})) return false;
          mma_kblock_desc(xcol, hd0 + kChunk, rd0 + kSlot * ((n + 1) % 3), idesc_d, false);
          release_stage(StageNo<n + 1>{});
          tc_commit(smem_u32(&sh->hid_free[1]));
          return true;
        };
        for (int t = tile0; t < t_end && ok; t += tstep, ++tile_i) {
          const uint32_t par = tile_i & 1;
          const uint32_t xcol = tmem_base + (par ? 256u : 0u);     // region X of this tile
          const uint32_t acol = tmem_base + (par ? 0u : 256u);     // two hidden-chunk buffers
          flip = par;
          TAIL_WAIT(&sh->a_full, par, 6);
          TAIL_WAIT(&sh->x_ready, par, 7);
          tc_fence_after();
          // x1 = x (pre-stored) + att Wo^T: stages 0..2
          ok = wait_stage(StageNo<0>{});
          if (!ok) break;
          mma_kblock_desc(xcol, ad0, rd0, idesc_d, false);
          release_stage(StageNo<0>{});
          ok = wait_stage(StageNo<1>{});
          if (!ok) break;
          mma_kblock_desc(xcol, ad0 + kChunk, rd0 + kSlot, idesc_d, false);
          release_stage(StageNo<1>{});
          ok = wait_stage(StageNo<2>{});
          if (!ok) break;
          mma_kblock_desc(xcol, ad0 + 2 * kChunk, rd0 + 2 * kSlot, idesc_d, false);
          release_stage(StageNo<2>{});
          commit(&sh->o_done);
          TAIL_WAIT(&sh->h2_ready, par, 8);
          tc_fence_after();
          // hidden chunks 0 and 1 (stages 3..6), then chunk j's FFN-down and chunk j + 2's FFN-up for j = 0..3
          // (stages 7..22), then the FFN-down of chunks 4 and 5 (stages 23..26); the hidden-chunk barriers complete
          // once per chunk, six times per tile: parity j & 1
          ok = up(StageNo<3>{}, acol, &sh->acc1_full[0]) && up(StageNo<5>{}, acol + HC, &sh->acc1_full[1]) &&
               down(StageNo<7>{}, xcol, 0u) && up(StageNo<9>{}, acol, &sh->acc1_full[0]) &&
               down(StageNo<11>{}, xcol, 1u) && up(StageNo<13>{}, acol + HC, &sh->acc1_full[1]) &&
               down(StageNo<15>{}, xcol, 0u) && up(StageNo<17>{}, acol, &sh->acc1_full[0]) &&
               down(StageNo<19>{}, xcol, 1u) && up(StageNo<21>{}, acol + HC, &sh->acc1_full[1]);
          if (!ok) break;
          commit(&sh->a_free);                                     // the last reader of h2 (chunk 5's FFN-up) is issued
          ok = down(StageNo<23>{}, xcol, 0u) && down(StageNo<25>{}, xcol, 1u);
          if (ok) commit(&sh->x_done);
        }
      } else
      for (int t = tile0; t < t_end && ok; t += tstep, ++tile_i) {
        const uint32_t par = tile_i & 1;
        const uint32_t xcol = tmem_base + (par ? 256u : 0u);     // region X of this tile
        const uint32_t acol = tmem_base + (par ? 0u : 256u);     // two hidden-chunk buffers
        auto g1 = [&](int j) -> bool {                           // hidden chunk j = h2 W0[j]^T
          const uint32_t dst = acol + (j & 1) * HC;
          for (int i = 0; i < S1; ++i) {
            if (!with_stage([&](uint32_t st) {
                  mma_kblock(dst, sA + (2 * i) * CHUNK_BYTES, st, idesc_h, i != 0);
                  if (2 * i + 1 < KB) mma_kblock(dst, sA + (2 * i + 1) * CHUNK_BYTES, st + rows_h * 128, idesc_h, true);
                }))
              return false;
          }
          commit(&sh->acc1_full[j & 1]);
          return true;
        };
        TAIL_WAIT(&sh->a_full, par, 6);
        TAIL_WAIT(&sh->x_ready, par, 7);
        tc_fence_after();
        for (int kb = 0; kb < KB && ok; ++kb)       // x1 = x (pre-stored) + att Wo^T
          ok = with_stage([&](uint32_t st) { mma_kblock(xcol, sA + kb * CHUNK_BYTES, st, idesc_d, true); });
        if (!ok) break;
        commit(&sh->o_done);
        TAIL_WAIT(&sh->h2_ready, par, 8);
        tc_fence_after();
        ok = g1(0) && g1(1);
        if (NC == 2 && ok) commit(&sh->a_free);
        for (int j = 0; j < NC && ok; ++j) {
          for (int kc = 0; kc < 2 && ok; ++kc) {    // xo += hidden chunk j * W2[:, chunk j]^T, one 64-column half at a time
            if (!mbar_wait(smem_u32(&sh->hid_ready[kc]), n_hid & 1, abort)) { give_up(sh, p.status, 9); ok = false; break; }
            tc_fence_after();
            ok = with_stage([&](uint32_t st) { mma_kblock(xcol, sH + kc * CHUNK_BYTES, st, idesc_d, true); });
            if (ok) commit(&sh->hid_free[kc]);   // this half of sH may be overwritten once retired
          }
          ++n_hid;
          if (ok && j + 2 < NC) {
            ok = g1(j + 2);
            if (ok && j + 3 == NC) commit(&sh->a_free);   // last reader of h2 issued
          }
        }
        if (ok) commit(&sh->x_done);
      }
      commit(&sh->mma_done);
      uint32_t spins = 0;
      while (!mbar_try_wait(smem_u32(&sh->mma_done), 0) && ++spins < kSpinLimit) {}
      if (spins >= kSpinLimit) give_up(sh, p.status, 10);
    }
  } else if (warp >= 2 && warp < PROD_WARP) {
    // ------------------------------------------------------------ epilogue warps, thread = row
    // Two groups of four warps; both cover all 128 rows (warp & 3 = TMEM lane quadrant), group 0
    // owns the low half of the columns, group 1 the high half.  Global memory is touched only in
    // "transposed" form: a 32-row x 64-byte block goes through the warp's staging buffer so that
    // 4 lanes cover 64 contiguous bytes of one row (lane = (row sub8 + 8 i, 16-byte piece)).
    const int grp = (warp - 2) >> 2;
    const int q = warp & 3;
    const int trow = q * 32 + lane;                         // row inside the tile
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint8_t* stg = stg_all + (warp - 2) * STG_BYTES;
    const int sub8 = lane >> 2, piece = lane & 3;
    const int dh2 = d >> 1, c_lo = grp * dh2;               // this group's columns of the d-wide row
    const float4* prm4 = reinterpret_cast<const float4*>(prm);
    const float4 *P_bo = prm4, *P_g = prm4 + 64, *P_b = prm4 + 128, *P_b2 = prm4 + 192, *P_b0 = prm4 + 512;
    uint32_t tile_i = 0, n_acc[2] = {0, 0}, n_free = 0;
    bool ok = true;
    const float inv_d = 1.0f / (float)d;

    // Three 2 KB transposition buffers per warp (32 rows x 64 B, 64-byte swizzle -- the layout of the
    // 64-byte-wide TMA boxes): its slice of the staging area and, while no hidden chunk is live (from
    // the tile's last FFN-down MMA to the next tile's first hidden chunk), 4 KB of sH.
    auto io_buf = [&](int b) -> uint8_t* { return b == 0 ? stg : sH_g + (warp - 2) * 4096 + (b - 1) * 2048; };
    auto buf_write = [&](uint8_t* buf, int row, int pc, uint4 v) {   // 16-byte piece pc (0..3) of row
      *reinterpret_cast<uint4*>(buf + row * 64 + ((pc ^ ((row >> 1) & 3)) << 4)) = v;
    };
    auto buf_read = [&](const uint8_t* buf, int row, int pc) -> uint4 {
      return *reinterpret_cast<const uint4*>(buf + row * 64 + ((pc ^ ((row >> 1) & 3)) << 4));
    };
    auto stg_write = [&](int row, int pc, uint4 v) { buf_write(stg, row, pc, v); };
    auto stg_read = [&](int row, int pc) -> uint4 { return buf_read(stg, row, pc); };
    uint32_t n_io = 0;                                      // residual blocks this warp has consumed so far
    auto group_sync = [&]() { asm volatile("bar.sync 2, %0;" ::"n"(EPI_WARPS * 32) : "memory"); };
    auto signal = [&](uint64_t* bar) {   // one arrival per warp, after everyone's writes
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar));
    };
    // shared-memory writes of this thread -> visible to the tensor core (the all-state-space form of
    // the fence measured ~2,000 cycles per use and is not needed for this CTA's own shared memory)
    auto publish_smem = [&]() { fence_proxy_async_smem(); };
    // row statistics of the whole row from this group's partial sums and the other group's
    auto row_stats = [&](int phase, float sum, float sq, float& mean, float& rstd) {
      part[(phase * 2 + grp) * BM + trow] = make_float2(sum, sq);
      group_sync();
      const float2 o = part[(phase * 2 + (grp ^ 1)) * BM + trow];
      mean = (sum + o.x) * inv_d;
      rstd = rsqrtf(fmaxf((sq + o.y) * inv_d - mean * mean, 0.f) + p.eps);
    };
    // pre-store (x + bo) of tile t, this group's columns, into TMEM columns col0 + ...
    // (a) rows gathered through the row map: coalesced loads, transposed through the staging buffer
    auto prestore_ldg = [&](int t, uint32_t col0) {
      const float* src[4];                                  // this lane's 4 rows in the transposed phase
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t row = (int64_t)t * BM + q * 32 + i * 8 + sub8;
        src[i] = row < p.M ? p.x + p.xmap.plain(row) * p.ldx + piece * 4 : nullptr;
      }
      uint4 nxt[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        nxt[i] = src[i] ? *reinterpret_cast<const uint4*>(src[i] + c_lo) : make_uint4(0, 0, 0, 0);
      for (int c = c_lo; c < c_lo + dh2; c += 32) {
        uint32_t r[32];
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {                    // two 16-column blocks per 32 TMEM columns
          const int cc = c + 16 * hb;
#pragma unroll
          for (int i = 0; i < 4; ++i) stg_write(i * 8 + sub8, piece, nxt[i]);
          if (cc + 16 < c_lo + dh2) {                       // next block's loads fly during this one
#pragma unroll
            for (int i = 0; i < 4; ++i)
              nxt[i] = src[i] ? *reinterpret_cast<const uint4*>(src[i] + cc + 16) : make_uint4(0, 0, 0, 0);
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v = stg_read(lane, j);
            const float4 bo = P_bo[(cc >> 2) + j];
            r[16 * hb + 4 * j] = __float_as_uint(__uint_as_float(v.x) + bo.x);
            r[16 * hb + 4 * j + 1] = __float_as_uint(__uint_as_float(v.y) + bo.y);
            r[16 * hb + 4 * j + 2] = __float_as_uint(__uint_as_float(v.z) + bo.z);
            r[16 * hb + 4 * j + 3] = __float_as_uint(__uint_as_float(v.w) + bo.w);
          }
          __syncwarp();
        }
        tmem_st32(lane_base + col0 + c, r);
      }
      tmem_wait_st();
    };
    // (b) dense rows: 16-column blocks of this warp's 32 rows arrive by TMA in the three buffers, up to
    // three in flight; block n (counted over the whole kernel) uses buffer n % 3, phase (n / 3) & 1
    auto prestore_tma = [&](int t, uint32_t col0) -> bool {
      const int row0 = t * BM + q * 32;
      const int nb = dh2 >> 4;
      auto issue = [&](int k) {                             // k-th block of this call
        if (lane == 0) {
          const uint32_t n = n_io + k;
          const uint32_t bar = smem_u32(&sh->io_full[warp - 2][n % 3]);
          mbar_expect_tx(bar, STG_BYTES);
          tma_load_2d(smem_u32(io_buf(n % 3)), &tm_x, c_lo + 16 * k, row0, bar);
        }
      };
      for (int k = 0; k < 3 && k < nb; ++k) issue(k);
      int k = 0;
      for (int c = c_lo; c < c_lo + dh2; c += 32) {
        uint32_t r[32];
#pragma unroll
        for (int hb = 0; hb < 2; ++hb, ++k) {
          const uint32_t n = n_io + k;
          if (!mbar_wait_warp(smem_u32(&sh->io_full[warp - 2][n % 3]), (n / 3) & 1, abort)) {
            if (lane == 0) give_up(sh, p.status, 15);
            return false;
          }
          const uint8_t* buf = io_buf(n % 3);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v = buf_read(buf, lane, j);
            const float4 bo = P_bo[((c + 16 * hb) >> 2) + j];
            r[16 * hb + 4 * j] = __float_as_uint(__uint_as_float(v.x) + bo.x);
            r[16 * hb + 4 * j + 1] = __float_as_uint(__uint_as_float(v.y) + bo.y);
            r[16 * hb + 4 * j + 2] = __float_as_uint(__uint_as_float(v.z) + bo.z);
            r[16 * hb + 4 * j + 3] = __float_as_uint(__uint_as_float(v.w) + bo.w);
          }
          __syncwarp();                                     // everyone has read the buffer: refill it
          if (k + 3 < nb) issue(k + 3);
        }
        tmem_st32(lane_base + col0 + c, r);
      }
      n_io += nb;
      tmem_wait_st();
      return true;
    };
    auto prestore = [&](int t, uint32_t col0) -> bool {
      if (p.x_tma) return prestore_tma(t, col0);
      prestore_ldg(t, col0);
      return true;
    };

    if (tile0 < t_end) {
      ok = prestore(tile0, 0u);
      signal(&sh->x_ready);
    }
    for (int t = tile0; t < t_end && ok; t += tstep, ++tile_i) {
      const uint32_t par = tile_i & 1;
      const uint32_t xcol = par ? 256u : 0u, acol = par ? 0u : 256u;
      const int t_next = t + tstep;
      // ---- E1: h2 = LN_ffn(x1) -> sA   (X already holds x + bo + att Wo^T)
      TAIL_WAIT_WARP(&sh->o_done, par, 11);
      tc_fence_after();
      {
        float sum = 0.f, sq = 0.f;
        for (int c = c_lo; c < c_lo + dh2; c += 32) {
          uint32_t r[32];
          tmem_ld32(lane_base + xcol + c, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = __uint_as_float(r[j]);
            sum += v;
            sq = fmaf(v, v, sq);
          }
        }
        float mean, rstd;
        row_stats(0, sum, sq, mean, rstd);
        const float shift = -mean * rstd;
        for (int c = c_lo; c < c_lo + dh2; c += 32) {
          uint32_t r[32];
          float v[32];
          tmem_ld32(lane_base + xcol + c, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 g = P_g[(c >> 2) + j], bb = P_b[(c >> 2) + j];
            v[4 * j] = fmaf(fmaf(__uint_as_float(r[4 * j]), rstd, shift), g.x, bb.x);
            v[4 * j + 1] = fmaf(fmaf(__uint_as_float(r[4 * j + 1]), rstd, shift), g.y, bb.y);
            v[4 * j + 2] = fmaf(fmaf(__uint_as_float(r[4 * j + 2]), rstd, shift), g.z, bb.z);
            v[4 * j + 3] = fmaf(fmaf(__uint_as_float(r[4 * j + 3]), rstd, shift), g.w, bb.w);
          }
          store_h32(sA_g, trow, c, v);
        }
      }
      publish_smem();
      signal(&sh->h2_ready);
      // ---- hidden chunks: relu(acc + b0) -> sH; this group handles 64 of the chunk's 128 columns
      for (int j = 0; j < NC && ok; ++j) {
        const int b = j & 1;
        if (!mbar_wait_warp(smem_u32(&sh->acc1_full[b]), n_acc[b] & 1, abort)) {
          if (lane == 0) give_up(sh, p.status, 12);
          ok = false;
          break;
        }
        ++n_acc[b];
        tc_fence_after();
        uint32_t hp[32];                                    // 64 fp16 values of this row
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          uint32_t r[32];
          tmem_ld32(lane_base + acol + b * HC + grp * 64 + c, r);
          tmem_wait_ld();
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const float4 b0 = P_b0[((j * HC + grp * 64 + c) >> 2) + jj];
            const float a0 = __uint_as_float(r[4 * jj]) + b0.x, a1 = __uint_as_float(r[4 * jj + 1]) + b0.y;
            const float a2 = __uint_as_float(r[4 * jj + 2]) + b0.z, a3 = __uint_as_float(r[4 * jj + 3]) + b0.w;
            if (GELU) {
              hp[(c >> 1) + 2 * jj] = pack_half2(gelu_exact(a0), gelu_exact(a1));
              hp[(c >> 1) + 2 * jj + 1] = pack_half2(gelu_exact(a2), gelu_exact(a3));
            } else {
              hp[(c >> 1) + 2 * jj] = pack_half2(fmaxf(a0, 0.f), fmaxf(a1, 0.f));
              hp[(c >> 1) + 2 * jj + 1] = pack_half2(fmaxf(a2, 0.f), fmaxf(a3, 0.f));
            }
          }
        }
        // this half of sH is free once the previous chunk's FFN-down MMAs on it have retired
        if (!mbar_wait_warp(smem_u32(&sh->hid_free[grp]), (n_free & 1) ^ 1, abort)) {
          if (lane == 0) give_up(sh, p.status, 14);
          ok = false;
          break;
        }
        ++n_free;
        {
          uint8_t* rowp = sH_g + grp * CHUNK_BYTES + (trow >> 3) * 1024 + (trow & 7) * 128;
#pragma unroll
          for (int pc = 0; pc < 8; ++pc)
            *reinterpret_cast<uint4*>(rowp + ((pc ^ (trow & 7)) << 4)) =
                make_uint4(hp[4 * pc], hp[4 * pc + 1], hp[4 * pc + 2], hp[4 * pc + 3]);
        }
        publish_smem();
        signal(&sh->hid_ready[grp]);
      }
      if (!ok) break;
      // ---- all MMAs of the tile have retired: X holds x1 + FFN, sH and both hidden buffers are free
      TAIL_WAIT_WARP(&sh->x_done, par, 13);
      tc_fence_after();
      // pre-store the next tile's x over the hidden buffers; its out-projection then runs under the drain
      if (t_next < t_end) {
        ok = prestore(t_next, acol);
        signal(&sh->x_ready);
        if (!ok) break;
      }
      // ---- final: xo = X + b2 -> fp32 out, then LayerNorm / fp16 outputs, as TMA stores of 32-row blocks
      {
        const int row0 = t * BM + q * 32;                   // first row of this warp
        const bool want_stats = p.g16[0] || p.g16[1];
        float sum = 0.f, sq = 0.f;
        uint32_t n_st = 0;                                  // blocks stored by this warp in this drain
        // buffer of the next block, once the store that used it three blocks ago has read it
        auto next_buf = [&]() -> uint8_t* {
          if (n_st >= 3) {
            if (lane == 0) bulk_wait_read<2>();
            __syncwarp();
          }
          return io_buf(n_st % 3);
        };
        // the warp's writes to the buffer -> one TMA store of 32 rows x 64 bytes (rows >= M are clipped)
        auto store_block = [&](const CUtensorMap* map, int x) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(map, x, row0, smem_u32(io_buf(n_st % 3)));
            bulk_commit();
          }
          ++n_st;
        };
        if (p.x_out || want_stats) {
          for (int c = c_lo; c < c_lo + dh2; c += 32) {
            uint32_t r[32];
            tmem_ld32(lane_base + xcol + c, r);
            tmem_wait_ld();
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
              uint8_t* buf = p.x_out ? next_buf() : nullptr;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float4 b2 = P_b2[((c + 16 * hb) >> 2) + j];
                float4 v = make_float4(__uint_as_float(r[16 * hb + 4 * j]) + b2.x, __uint_as_float(r[16 * hb + 4 * j + 1]) + b2.y,
                                       __uint_as_float(r[16 * hb + 4 * j + 2]) + b2.z, __uint_as_float(r[16 * hb + 4 * j + 3]) + b2.w);
                sum += (v.x + v.y) + (v.z + v.w);
                sq = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sq))));
                if (p.x_out)
                  buf_write(buf, lane, j, make_uint4(__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z),
                                                     __float_as_uint(v.w)));
              }
              if (p.x_out) store_block(&tm_xo, c + 16 * hb);
            }
          }
        }
        float mean = 0.f, rstd = 1.f;
        if (want_stats) row_stats(1, sum, sq, mean, rstd);
#pragma unroll 1
        for (int o = 0; o < 2; ++o) {
          if (!p.out16[o]) continue;
          const bool ln = p.g16[o] != nullptr;
          const float sc = ln ? rstd : 1.f, sh0 = ln ? -mean * rstd : 0.f;
          const float4 *P_go = prm4 + 256 + 128 * o, *P_bo16 = prm4 + 320 + 128 * o;
          const CUtensorMap* tm_o = o ? &tm_o1 : &tm_o0;
          for (int c = c_lo; c < c_lo + dh2; c += 32) {     // 32 columns = 64 bytes of fp16 per row
            uint32_t r[32];
            tmem_ld32(lane_base + xcol + c, r);
            tmem_wait_ld();
            uint8_t* buf = next_buf();
#pragma unroll
            for (int j = 0; j < 4; ++j) {                   // 8 columns -> one 16-byte fp16 piece
              float y[8];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int f4 = (c >> 2) + 2 * j + e;
                const float4 b2 = P_b2[f4], g = P_go[f4], bb = P_bo16[f4];
                y[4 * e] = fmaf(fmaf(__uint_as_float(r[8 * j + 4 * e]) + b2.x, sc, sh0), g.x, bb.x);
                y[4 * e + 1] = fmaf(fmaf(__uint_as_float(r[8 * j + 4 * e + 1]) + b2.y, sc, sh0), g.y, bb.y);
                y[4 * e + 2] = fmaf(fmaf(__uint_as_float(r[8 * j + 4 * e + 2]) + b2.z, sc, sh0), g.z, bb.z);
                y[4 * e + 3] = fmaf(fmaf(__uint_as_float(r[8 * j + 4 * e + 3]) + b2.w, sc, sh0), g.w, bb.w);
              }
              buf_write(buf, lane, j, make_uint4(pack_half2(y[0], y[1]), pack_half2(y[2], y[3]),
                                                 pack_half2(y[4], y[5]), pack_half2(y[6], y[7])));
            }
            store_block(tm_o, c);
          }
        }
        // the buffers (two of them inside sH) are reused by the next tile: all stores have read them
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
      }
      tc_fence_before();
    }
    if (lane == 0) bulk_wait_all();                         // the stores are complete before the CTA exits
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}
#undef tile0
#undef tstep
#undef t_end
}  // namespace

bool block_tail_ok(const BlockTailArgs& a) {
  if (a.d % 64 != 0 || a.d < 64 || a.d > 256) return false;
  if (a.F % 256 != 0 || a.F < 256 || a.F > 1024) return false;
  if (a.M < 1 || a.M > 0x7fffff00) return false;          // TMA row coordinates are 32-bit
  if (!aligned16(a.att) || !aligned16(a.x) || (a.ldx % 4) || (a.ld_att % 8)) return false;
  if (a.x_out && !aligned16(a.x_out)) return false;
  for (int o = 0; o < 2; ++o)
    if (a.out16[o] && (!aligned16(a.out16[o]) || (a.ld16[o] % 8))) return false;
  return true;
}

int block_tail(const BlockTailArgs& a, cudaStream_t stream) {
  if (!block_tail_ok(a)) {
    set_error("block_tail: shape d=%d F=%d m=%lld does not fit the fused kernel", a.d, a.F, (long long)a.M);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (!a.att || !a.x || !a.wo || !a.w0 || !a.w2 || !a.bo || !a.b0 || !a.b2 || !a.ln_g || !a.ln_b) {
    set_error("block_tail: NULL operand");
    return BSRL_ERR_NULL;
  }
  int* status = device_status_ptr();
  if (!status) return BSRL_ERR_CUDA;
  const int n_tiles = (int)((a.M + BM - 1) / BM);
  CUtensorMap tm_att, tm_wo, tm_w0, tm_w2;
  if (!make_tmap_f16(&tm_att, a.att, a.M, a.d, a.ld_att, BM)) return BSRL_ERR_CUDA;
  if (!make_tmap_f16(&tm_wo, a.wo, a.d, a.d, a.d, a.d)) return BSRL_ERR_CUDA;
  if (!make_tmap_f16(&tm_w0, a.w0, a.F, a.d, a.d, HC)) return BSRL_ERR_CUDA;
  if (!make_tmap_f16(&tm_w2, a.w2, a.d, a.F, a.F, a.d)) return BSRL_ERR_CUDA;
  // residual rows in and the outputs move as 32-row x 64-byte TMA boxes; a map that is not needed
  // aliases the attention tile's (the kernel only prefetches its descriptor)
  const bool x_tma = a.xmap.group == 0x7fffffff && a.xmap.stride == 0 && a.xmap.first == 0;
  CUtensorMap tm_x = tm_att, tm_xo = tm_att, tm_o[2] = {tm_att, tm_att};
  if (x_tma && !make_tmap_rows64(&tm_x, a.x, 4, a.M, a.d, a.ldx, 32)) return BSRL_ERR_CUDA;
  if (a.x_out && !make_tmap_rows64(&tm_xo, a.x_out, 4, a.M, a.d, a.d, 32)) return BSRL_ERR_CUDA;
  for (int o = 0; o < 2; ++o)
    if (a.out16[o] && !make_tmap_rows64(&tm_o[o], a.out16[o], 2, a.M, a.d, a.ld16[o], 32)) return BSRL_ERR_CUDA;
  static DeviceOnce once;
  int rc = once.run("block_tail_kernel set-up", [] {
    cudaError_t e = cudaFuncSetAttribute(block_tail_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(block_tail_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  if (rc != BSRL_OK) return rc;
  TailParams p;
  p.d = a.d; p.F = a.F; p.M = a.M;
  p.x = a.x; p.ldx = a.ldx; p.xmap = a.xmap;
  p.bo = a.bo; p.ln_g = a.ln_g; p.ln_b = a.ln_b; p.b0 = a.b0; p.b2 = a.b2; p.eps = a.eps;
  p.x_out = a.x_out;
  for (int o = 0; o < 2; ++o) {
    p.out16[o] = a.out16[o]; p.ld16[o] = a.ld16[o]; p.g16[o] = a.g16[o]; p.b16[o] = a.b16[o];
  }
  p.n_tiles = n_tiles;
  p.x_tma = x_tma ? 1 : 0;
  p.status = status;
  int grid = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
  if (a.gelu) block_tail_kernel<true><<<grid, THREADS, SMEM_BYTES, stream>>>(tm_att, tm_wo, tm_w0, tm_w2, tm_x, tm_xo, tm_o[0], tm_o[1], p);
  else block_tail_kernel<false><<<grid, THREADS, SMEM_BYTES, stream>>>(tm_att, tm_wo, tm_w0, tm_w2, tm_x, tm_xo, tm_o[0], tm_o[1], p);
  BSRL_LAUNCH_OK("block_tail_kernel");
  return BSRL_OK;
}


}  // namespace bsrl
