// tcgen05 linear layer: C = act(A W^T + bias) (+ residual) on the 5th-generation tensor cores.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: streams (128 x 64) A tiles and (BN x 64) W tiles, both K-major
//               with the 128-byte swizzle, through a 4-stage shared-memory ring;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M = 128, N <= 256, K = 16) on the
//               shared-memory descriptors, accumulating in TMEM; two accumulator buffers of BN
//               fp32 columns let tile t+1's MMAs overlap tile t's epilogue;
//   warps 2..9  epilogue: tcgen05.ld the accumulator (thread = output row), add bias, ReLU,
//               transpose through a per-warp swizzled staging block; dense residual-free outputs
//               leave as one TMA store per block, remapped rows and residual adds as 16-byte
//               stores that cover full 128-byte lines (residual pieces requested ahead).
// All waits are bounded: a wait that runs out sets the library's device status word, raises
// the CTA-wide abort flag, and every role falls through to the common teardown that frees TMEM.
//
// Stands in for the reference's cuBLAS / cuBLASLt calls on the fp16 stream (torch.addmm and the
// RELU_BIAS epilogue, python/fp16_linear.py:134-181; linear_relu_aux,
// python/beat_arena_env/csrc/fp16_gemm.cu:402-497).
#include "kernels.cuh"
#include "tc5.cuh"

namespace bsrl {

namespace {
__device__ int g_device_status = 0;

using namespace tc5;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;            // 16 KB
constexpr int W_BYTES = BN * BK * 2;            // 32 KB
constexpr int STAGE_BYTES = A_BYTES + W_BYTES;  // 48 KB
constexpr int EPI_WARPS = 8;
constexpr int THREADS = (2 + EPI_WARPS) * 32;
constexpr int TMEM_COLS = 2 * BN;               // two accumulator buffers = all 512 columns
constexpr int STG_BYTES = 32 * 128;             // per-warp transposition buffer: 32 rows x 128 bytes
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * STG_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct Shared {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], mma_done;
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ void give_up(Shared* sh, int* status, int role) {
  atomicCAS(status, 0, 1 * 16 + role);
  sh->abort = 1;
}

// work item w = (K split, row tile, column tile), split-major; the tile count fits 31 bits (checked on the host)
struct WorkItem {
  int split, mt, nt;
};
__device__ __forceinline__ WorkItem work_item(int64_t w, int n_tile_work, int n_tiles) {
  WorkItem it;
  int t;
  it.split = (int)div_index(w, n_tile_work, &t);
  it.mt = (int)div_index(t, n_tiles, &it.nt);
  return it;
}

// HAS_R: a residual is added in the epilogue (its prefetch registers and address arithmetic are compiled
// out otherwise: they cost the residual-free fp32 epilogue ~15 %).
template <bool HAS_R>
__global__ void __launch_bounds__(THREADS, 1)
linear_tc5_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                  const __grid_constant__ CUtensorMap tm_c, int tma_c, LinearArgs p, int m_tiles, int n_tiles,
                  int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* staging = smem_raw + (tiles_base - raw) + STAGES * STAGE_BYTES;
  Shared* sh = reinterpret_cast<Shared*>(staging + EPI_WARPS * STG_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int splits = p.k_splits > 1 ? p.k_splits : 1;
  const int kps = (k_blocks + splits - 1) / splits;          // k-blocks per split
  const int64_t n_tile_work = (int64_t)m_tiles * n_tiles;
  const int64_t n_work = n_tile_work * splits;                // work item = (split, tile): split-major
  volatile int* abort = &sh->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->tmem_full[b]), 1);
      mbar_init(smem_u32(&sh->tmem_empty[b]), EPI_WARPS);
    }
    mbar_init(smem_u32(&sh->mma_done), 1);
    sh->abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const WorkItem wi = work_item(w, (int)n_tile_work, n_tiles);
        const int kb0 = wi.split * kps, kb1 = min(k_blocks, kb0 + kps);
        const int m0 = wi.mt * BM, n0 = wi.nt * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&sh->empty[s]), ph ^ 1, abort)) { give_up(sh, status, 1); ok = false; break; }
          const uint32_t bar = smem_u32(&sh->full[s]);
          mbar_expect_tx(bar, STAGE_BYTES);
          const uint32_t dst = tiles_base + s * STAGE_BYTES;
          if (p.a_mn) tma_load_3d(dst, &tm_a, 0, kb * BK, m0 / 64, bar);
          else tma_load_2d(dst, &tm_a, kb * BK, m0, bar);
          if (p.w_mn) tma_load_3d(dst + A_BYTES, &tm_w, 0, kb * BK, n0 / 64, bar);
          else tma_load_2d(dst + A_BYTES, &tm_w, kb * BK, n0, bar);
        }
      }
      // the loads still in flight must land before this CTA may exit (also when a wait above
      // gave up): poll the full barriers of the last stages issued, bounded, ignoring abort
      const uint32_t issued = it;
      for (uint32_t j = issued > STAGES ? issued - STAGES : 0; j < issued; ++j) {
        const uint32_t bar = smem_u32(&sh->full[j % STAGES]);
        const uint32_t ph = (j / STAGES) & 1;
        uint32_t spins = 0;
        while (!mbar_try_wait(bar, ph) && ++spins < kSpinLimit) {}
        if (spins >= kSpinLimit) give_up(sh, status, 2);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int64_t w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++tile_i) {
        const WorkItem wi = work_item(w, (int)n_tile_work, n_tiles);
        const int kb0 = wi.split * kps, kb1 = min(k_blocks, kb0 + kps);
        const int n0 = wi.nt * BN;
        int n_cols = p.N - n0;
        if (n_cols > BN) n_cols = BN;
        const uint32_t idesc = idesc_f16(BM, n_cols, p.a_mn, p.w_mn);
        // 16-byte units a K step of 16 advances an operand's start address by: 32 bytes along a K-major row,
        // two 8-row groups of an MN-major tile
        const uint32_t a_step = p.a_mn ? 128u : 2u, w_step = p.w_mn ? 128u : 2u;
        const int buf = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(smem_u32(&sh->tmem_empty[buf]), acc_ph ^ 1, abort)) { give_up(sh, status, 3); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&sh->full[s]), ph, abort)) { give_up(sh, status, 4); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = tiles_base + s * STAGE_BYTES;
          const uint64_t a_desc = p.a_mn ? smem_desc_mn_sw128(a_addr, BK * 128) : smem_desc_sw128(a_addr);
          const uint64_t w_desc = p.w_mn ? smem_desc_mn_sw128(a_addr + A_BYTES, BK * 128) : smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            mma_f16_ss(d_tmem, a_desc + a_step * k, w_desc + w_step * k, idesc, (kb != kb0 || k) ? 1u : 0u);
          tc_commit(smem_u32(&sh->empty[s]));
        }
        if (ok) tc_commit(smem_u32(&sh->tmem_full[buf]));
      }
      // every MMA issued must have retired before TMEM is freed (bounded, ignoring abort)
      tc_commit(smem_u32(&sh->mma_done));
      uint32_t spins = 0;
      while (!mbar_try_wait(smem_u32(&sh->mma_done), 0) && ++spins < kSpinLimit) {}
      if (spins >= kSpinLimit) give_up(sh, status, 6);
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    // Each warp drains a 32-row x 128-column slab of the tile in blocks of 128 bytes per row
    // (64 fp16 or 32 fp32 columns).  TMEM hands every thread one ROW; writing rows straight to
    // HBM would touch 32 different 128-byte lines per store instruction, so the block is first
    // transposed through a per-warp 4 KB staging buffer (16-byte pieces, XOR-swizzled) and then
    // written -- and the residual read -- with 8 lanes covering one full 128-byte line.
    const int q = warp & 3;                    // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;          // which half of the tile's columns
    uint8_t* stg = staging + (warp - 2) * STG_BYTES;
    const bool wide = p.out_f32 || HAS_R;        // stage fp32 (32 columns per block) instead of fp16 (64)
    const int cw = wide ? 32 : 64;
    const int sub = lane >> 3, piece = lane & 7;   // transposed phase: row sub + 4 i, 16-byte piece
    uint32_t tile_i = 0;
    bool ok = true;
    for (int64_t w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++tile_i) {
      const WorkItem wi = work_item(w, (int)n_tile_work, n_tiles);
      const bool first_split = w < n_tile_work;              // the piece that carries the bias
      const int64_t m0 = (int64_t)wi.mt * BM;
      const int n0 = wi.nt * BN;
      const int buf = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      // output / residual row offsets of the 8 rows this lane writes in the transposed phase
      int64_t crow[8], rrow[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t row = m0 + q * 32 + i * 4 + sub;
        crow[i] = row < p.M ? p.cmap(row) * (int64_t)p.ldc : -1;
        rrow[i] = (HAS_R && row < p.M) ? p.rmap(row) * (int64_t)p.ldr : 0;
      }
      if (!mbar_wait_warp(smem_u32(&sh->tmem_full[buf]), acc_ph, abort)) {
        if (lane == 0) give_up(sh, status, 5);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * (BN / 2);
#pragma unroll 1
      for (int c = 0; c < BN / 2; c += cw) {
        const int col = n0 + half * (BN / 2) + c;     // first column of this block
        if (col >= p.N) break;                         // warp-uniform
        // residual pieces of this block, requested before the accumulator is read so that their latency
        // hides behind the TMEM load and the staging pass (fetched inside the store loop they made the
        // epilogue 3.6x slower than the residual-free one)
        float4 rv[8];
        if (HAS_R) {
          const int pc = col + piece * 4;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            rv[i] = (crow[i] >= 0 && pc < p.N) ? *reinterpret_cast<const float4*>(p.R + rrow[i] + pc)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        uint32_t r[32];
        // ---- phase 1: own row, 32 columns at a time -> bias / ReLU -> staging
        for (int s32 = 0; s32 < cw; s32 += 32) {
          if (col + s32 >= p.N) break;
          uint4 mk[4];                                   // this row's 32 mask entries, requested ahead of the accumulator
          const int64_t mrow = m0 + q * 32 + lane;
          const bool masked = p.mask != nullptr && mrow < p.M;
          if (masked) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              mk[j] = col + s32 + 8 * j < p.N ? *reinterpret_cast<const uint4*>(p.mask + mrow * p.ldm + col + s32 + 8 * j)
                                              : make_uint4(0, 0, 0, 0);
          }
          tmem_ld32(tbase + c + s32, r);
          tmem_wait_ld();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (p.bias && first_split) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              // columns past N read the zero padding of the accumulator; clamp the bias index
              const int cb = min(col + s32 + j, p.N - 4);
              float4 bv = *reinterpret_cast<const float4*>(p.bias + cb);
              v[j] += bv.x; v[j + 1] += bv.y; v[j + 2] += bv.z; v[j + 3] += bv.w;
            }
          }
          if (p.relu == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          } else if (p.relu == 2) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_exact(v[j]);
          }
          if (masked) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __half* mh = reinterpret_cast<const __half*>(&mk[j]);
#pragma unroll
              for (int t = 0; t < 8; ++t)
                if (!(__half2float(mh[t]) > 0.f)) v[8 * j + t] = 0.f;
            }
          }
          if (tma_c && s32 == 0) {   // the previous block's TMA store has read the staging buffer
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
          }
          if (wide) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                  make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(stg + lane * 128 + ((((s32 >> 3) + j) ^ (lane & 7)) << 4)) =
                  make_uint4(pack_half2(v[8 * j], v[8 * j + 1]), pack_half2(v[8 * j + 2], v[8 * j + 3]),
                             pack_half2(v[8 * j + 4], v[8 * j + 5]), pack_half2(v[8 * j + 6], v[8 * j + 7]));
          }
        }
        if (tma_c) {
          // ---- phase 2 (dense output, no residual): the staged 32 x 128-byte block leaves as one TMA
          // store; rows past M and columns past N are clipped by the tensor map
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && m0 + q * 32 < p.M) {
            tma_store_2d(&tm_c, col, (int)(m0 + q * 32), smem_u32(stg));
            bulk_commit();
          }
          continue;
        }
        __syncwarp();
        // ---- phase 2: 8 lanes per row, one 16-byte piece each
        const int pcol = col + piece * (wide ? 4 : 8);   // first column of this lane's piece
        if (pcol < p.N) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (crow[i] < 0) continue;
            const int rr = i * 4 + sub;
            const uint4 raw16 = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((piece ^ (rr & 7)) << 4));
            if (!wide) {
              *reinterpret_cast<uint4*>(static_cast<__half*>(p.C) + crow[i] + pcol) = raw16;
            } else {
              float4 f = make_float4(__uint_as_float(raw16.x), __uint_as_float(raw16.y),
                                     __uint_as_float(raw16.z), __uint_as_float(raw16.w));
              if (HAS_R) {
                f.x += rv[i].x; f.y += rv[i].y; f.z += rv[i].z; f.w += rv[i].w;
              }
              if (splits > 1) {
                float* dst = static_cast<float*>(p.C) + crow[i] + pcol;
                atomicAdd(dst, f.x); atomicAdd(dst + 1, f.y); atomicAdd(dst + 2, f.z); atomicAdd(dst + 3, f.w);
              } else if (p.out_f32)
                *reinterpret_cast<float4*>(static_cast<float*>(p.C) + crow[i] + pcol) = f;
              else
                *reinterpret_cast<uint2*>(static_cast<__half*>(p.C) + crow[i] + pcol) =
                    make_uint2(pack_half2(f.x, f.y), pack_half2(f.z, f.w));
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->tmem_empty[buf]));
    }
    if (tma_c && lane == 0) bulk_wait_all();      // the stores are complete before the CTA exits
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}
}  // namespace

// ---------------------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

bool make_tmap_f16(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld_elems,
                   int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_elems * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (%d) for a (%lld x %lld) fp16 matrix, ld %lld", (int)r,
              (long long)rows, (long long)cols, (long long)ld_elems);
    return false;
  }
  return true;
}

bool make_tmap_rows64(CUtensorMap* map, const void* base, int elem_bytes, int64_t rows, int64_t cols,
                      int64_t ld_elems, int box_rows) {
  return make_tmap_rows(map, base, elem_bytes, rows, cols, ld_elems, box_rows, 64);
}

bool make_tmap_rows(CUtensorMap* map, const void* base, int elem_bytes, int64_t rows, int64_t cols,
                    int64_t ld_elems, int box_rows, int row_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_elems * (cuuint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(row_bytes / elem_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (%d) for a (%lld x %lld) matrix of %d-byte elements, ld %lld", (int)r,
              (long long)rows, (long long)cols, elem_bytes, (long long)ld_elems);
    return false;
  }
  return true;
}

bool make_tmap_env3d(CUtensorMap* map, const void* base, int64_t n_envs, int tokens_per_env, int64_t cols,
                     int64_t ld_elems, int box_cols, int box_tokens, int box_envs) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)tokens_per_env, (cuuint64_t)n_envs};
  cuuint64_t strides[2] = {(cuuint64_t)ld_elems * 2, (cuuint64_t)ld_elems * 2 * (cuuint64_t)tokens_per_env};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_tokens, (cuuint32_t)box_envs};
  cuuint32_t estr[3] = {1, 1, 1};
  const int row_bytes = box_cols * 2;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (%d) for a (%lld envs x %d tokens x %lld) fp16 view, ld %lld", (int)r,
              (long long)n_envs, tokens_per_env, (long long)cols, (long long)ld_elems);
    return false;
  }
  return true;
}

// (k_rows, cols) fp16 row-major matrix seen as {64 columns, k rows, cols / 64 blocks}: one load of a
// {64, box_k, box_blocks} box brings box_blocks tiles of box_k x 128 bytes, each with the 128-byte swizzle
static bool make_tmap_mn(CUtensorMap* map, const void* base, int64_t k_rows, int64_t cols, int64_t ld_elems, int box_k,
                         int box_blocks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t dims[3] = {64, (cuuint64_t)k_rows, (cuuint64_t)(cols / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld_elems * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)box_k, (cuuint32_t)box_blocks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (%d) for a (%lld x %lld) fp16 matrix read in 64-column blocks, ld %lld", (int)r,
              (long long)k_rows, (long long)cols, (long long)ld_elems);
    return false;
  }
  return true;
}

bool linear_tc5_ok(const LinearArgs& p) {
  if (!p.A || !p.W || !p.C || p.M < 1) return false;
  if (p.N % 16 != 0 || p.N < 16 || p.K < 1) return false;
  if (!p.a_mn && !p.w_mn && p.K % BK != 0) return false;
  if (p.K % 8 != 0) return false;                                // columns past K of a K-major operand read as zero
  if (p.a_mn && (p.M % 64 != 0 || p.lda < p.M)) return false;
  if (p.w_mn && (p.N % 64 != 0 || p.ldw < p.N)) return false;
  if (p.amap.group != 0x7fffffff || p.amap.first != 0) return false;      // TMA reads A rows in order
  if (!aligned16(p.A) || !aligned16(p.W) || !aligned16(p.C) || (p.lda % 8) || (p.ldw % 8)) return false;
  if (p.ldc % (p.out_f32 ? 4 : 8)) return false;
  if (p.bias && !aligned16(p.bias)) return false;
  if (p.R && (!aligned16(p.R) || (p.ldr % 4))) return false;
  if (p.k_splits > 1 && (!p.out_f32 || p.relu || p.R || p.mask)) return false;   // split-K adds raw fp32 partial products
  if (p.mask && (!aligned16(p.mask) || (p.ldm % 8) || p.cmap.group != 0x7fffffff || p.cmap.first != 0)) return false;
  return true;
}

int linear_tc5(const LinearArgs& p_in, cudaStream_t stream) {
  LinearArgs p = p_in;
  if (p.k_splits > 1) {   // no piece may be empty: an empty piece would add an unwritten accumulator
    const int k_blocks = (p.K + BK - 1) / BK;
    if (p.k_splits > k_blocks) p.k_splits = k_blocks;
    if (p.k_splits > 1) {
      const int kps = (k_blocks + p.k_splits - 1) / p.k_splits;
      p.k_splits = (k_blocks + kps - 1) / kps;
    }
  }
  if (!linear_tc5_ok(p)) {
    set_error("linear: shape m=%lld n=%d k=%d does not fit the tcgen05 engine", (long long)p.M, p.N, p.K);
    return BSRL_ERR_UNSUPPORTED;
  }
  int* status = device_status_ptr();
  if (!status) return BSRL_ERR_CUDA;
  CUtensorMap tm_a, tm_w;
  if (p.a_mn ? !make_tmap_mn(&tm_a, p.A, p.K, p.M, p.lda, BK, BM / 64) : !make_tmap_f16(&tm_a, p.A, p.M, p.K, p.lda, BM))
    return BSRL_ERR_CUDA;
  if (p.w_mn ? !make_tmap_mn(&tm_w, p.W, p.K, p.N, p.ldw, BK, BN / 64) : !make_tmap_f16(&tm_w, p.W, p.N, p.K, p.ldw, BN))
    return BSRL_ERR_CUDA;
  // dense output rows without a residual leave as TMA stores of the epilogue's 32 x 128-byte staging blocks
  const bool tma_c = !p.R && p.k_splits <= 1 && p.cmap.group == 0x7fffffff && p.cmap.stride == 0 && p.cmap.first == 0 &&
                     p.M <= 0x7fffff00;
  CUtensorMap tm_c = tm_a;
  if (tma_c && !make_tmap_rows(&tm_c, p.C, p.out_f32 ? 4 : 2, p.M, p.N, p.ldc, 32, 128)) return BSRL_ERR_CUDA;
  static DeviceOnce once;
  int rc = once.run("linear_tc5_kernel set-up", [] {
    cudaError_t e = cudaFuncSetAttribute(linear_tc5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(linear_tc5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  if (rc != BSRL_OK) return rc;
  const int64_t m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  if (m_tiles > 0x7fffffff / n_tiles) {
    set_error("linear: too many tiles");
    return BSRL_ERR_SHAPE;
  }
  int64_t grid = m_tiles * n_tiles * (p.k_splits > 1 ? p.k_splits : 1);
  if (grid > sm_count()) grid = sm_count();
  if (p.R)
    linear_tc5_kernel<true><<<(unsigned)grid, THREADS, SMEM_BYTES, stream>>>(tm_a, tm_w, tm_c, 0, p, (int)m_tiles, n_tiles, status);
  else
    linear_tc5_kernel<false><<<(unsigned)grid, THREADS, SMEM_BYTES, stream>>>(tm_a, tm_w, tm_c, tma_c ? 1 : 0, p, (int)m_tiles,
                                                                             n_tiles, status);
  BSRL_LAUNCH_OK("linear_tc5_kernel");
  return BSRL_OK;
}

int* device_status_ptr() {
  static DeviceOnce once;
  static int* cached[kMaxDevices] = {};
  int rc = once.run("device status word", [] {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_device_status);     // address on the CURRENT device
    if (e == cudaSuccess) cached[dev] = static_cast<int*>(p);
    return e;
  });
  if (rc != BSRL_OK) return nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  return cached[dev];
}

namespace {
__global__ void wait_selftest_kernel(int* status, uint32_t polls) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_barrier_init();
    // phase 0 of this barrier never completes: no thread arrives and no copy is counted on it
    if (!mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, polls)) atomicCAS(status, 0, kSelfTestKernel * 16 + 1);
  }
}
}  // namespace

int wait_selftest(uint32_t polls, cudaStream_t stream) {
  int* status = device_status_ptr();
  if (!status) return BSRL_ERR_CUDA;
  wait_selftest_kernel<<<1, 32, 0, stream>>>(status, polls);
  BSRL_LAUNCH_OK("wait_selftest_kernel");
  return BSRL_OK;
}

int device_status_take() {
  int* p = device_status_ptr();
  int v = 0, zero = 0;
  if (!p || cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
  return v;
}

}  // namespace bsrl
