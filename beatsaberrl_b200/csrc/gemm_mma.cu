// Warp-MMA linear layer: C = act(A W^T + bias) (+ residual), fp16 operands, fp32 accumulate.
//
// This is the general-shape GEMM of the forward: any M, N % 8 == 0, K % 32 == 0, row-remapped
// operands.  The large token-stream GEMMs run on the tcgen05 kernels instead; this one serves
// the narrow/odd shapes (token encoders' first layers, heads, critic tail) and is the
// cross-check for the tcgen05 kernels in the unit tests.
//
// Reference call sites this stands in for: fp16_linear / fp16_linear_relu / fp16_packed_linear
// (python/fp16_linear.py:506-517, :633-641, :794-805), i.e. torch.addmm and the cuBLASLt
// RELU_BIAS epilogue (python/beat_arena_env/csrc/fp16_gemm.cu:402-497).
#include "kernels.cuh"

namespace bsrl {

namespace {
constexpr int BM = 128, BN = 128, BK = 32, STAGES = 4, THREADS = 256;
constexpr int STAGE_BYTES = (BM + BN) * BK * 2;  // 16 KB

// 16-byte chunk (row, kc) of a [rows][32 halfs] tile, XOR-swizzled so that the 8 rows of an
// ldmatrix phase hit 8 distinct bank groups.
__device__ __forceinline__ uint32_t tile_off(int row, int kc) {
  return static_cast<uint32_t>((row * 4 + (kc ^ ((row >> 1) & 3))) * 16);
}

__global__ void __launch_bounds__(THREADS) linear_mma_kernel(LinearArgs p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps, warp tile 64 x 32
  const int n_tiles = (p.N + BN - 1) / BN;
  const int64_t tile = blockIdx.x;
  const int nt = static_cast<int>(tile % n_tiles);
  const int64_t mt = tile / n_tiles;
  const int64_t m0 = mt * BM;
  const int n0 = nt * BN;
  const uint32_t sbase = smem_u32(smem);

  // each thread moves two 16-byte chunks of A and two of W per stage
  const __half* a_src[2];
  const __half* w_src[2];
  bool a_ok[2], w_ok[2];
  uint32_t a_dst[2], w_dst[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int c = tid + i * THREADS;
    int row = c >> 2, kc = c & 3;
    int64_t gm = m0 + row;
    a_ok[i] = gm < p.M;
    a_src[i] = p.A + (a_ok[i] ? p.amap(gm) : 0) * (int64_t)p.lda + kc * 8;
    a_dst[i] = tile_off(row, kc);
    int gn = n0 + row;
    w_ok[i] = gn < p.N;
    w_src[i] = p.W + (int64_t)(w_ok[i] ? gn : 0) * p.ldw + kc * 8;
    w_dst[i] = BM * BK * 2 + tile_off(row, kc);
  }
  const int ksteps = p.K / BK;
  auto issue = [&](int ks) {
    if (ks < ksteps) {
      uint32_t s = sbase + (ks % STAGES) * STAGE_BYTES;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        cp_async16(s + a_dst[i], a_src[i] + (int64_t)ks * BK, a_ok[i]);
        cp_async16(s + w_dst[i], w_src[i] + (int64_t)ks * BK, w_ok[i]);
      }
    }
    cp_async_commit();
  };

  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue(s);

  for (int ks = 0; ks < ksteps; ++ks) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    issue(ks + STAGES - 1);
    const uint32_t sa = sbase + (ks % STAGES) * STAGE_BYTES;
    const uint32_t sw = sa + BM * BK * 2;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      uint32_t af[4][4], bf[2][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int row = wm * 64 + i * 16 + (lane & 15);
        ldmatrix_x4(af[i], sa + tile_off(row, kk * 2 + (lane >> 4)));
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        int row = wn * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldmatrix_x4(bf[j], sw + tile_off(row, kk * 2 + ((lane >> 3) & 1)));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          mma_f16(acc[i][j], af[i], bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]);
    }
  }
  cp_async_wait<0>();

  // epilogue: bias, activation, residual, store
  const int g = lane >> 2, tig = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int64_t gm = m0 + wm * 64 + i * 16 + g + hh * 8;
      if (gm >= p.M) continue;
      const int64_t crow = p.cmap(gm) * (int64_t)p.ldc;
      const float* rrow = p.R ? p.R + p.rmap(gm) * (int64_t)p.ldr : nullptr;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int col = n0 + wn * 32 + j * 8 + tig * 2;
        if (col >= p.N) continue;
        float v0 = acc[i][j][hh * 2], v1 = acc[i][j][hh * 2 + 1];
        if (p.bias) {
          v0 += p.bias[col];
          v1 += p.bias[col + 1];
        }
        if (p.relu == 1) {
          v0 = fmaxf(v0, 0.f);
          v1 = fmaxf(v1, 0.f);
        } else if (p.relu == 2) {
          v0 = gelu_exact(v0);
          v1 = gelu_exact(v1);
        }
        if (rrow) {
          float2 r = *reinterpret_cast<const float2*>(rrow + col);
          v0 += r.x;
          v1 += r.y;
        }
        if (p.out_f32) {
          *reinterpret_cast<float2*>(static_cast<float*>(p.C) + crow + col) = make_float2(v0, v1);
        } else {
          *reinterpret_cast<uint32_t*>(static_cast<__half*>(p.C) + crow + col) = pack_half2(v0, v1);
        }
      }
    }
  }
}
}  // namespace

int linear_mma(const LinearArgs& p, cudaStream_t stream) {
  if (!p.A || !p.W || !p.C) {
    set_error("linear: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (p.M < 0 || p.N <= 0 || p.K <= 0 || p.K % BK != 0 || p.N % 8 != 0) {
    set_error("linear: unsupported shape m=%lld n=%d k=%d (need k %% 32 == 0, n %% 8 == 0)",
              (long long)p.M, p.N, p.K);
    return BSRL_ERR_SHAPE;
  }
  if (!aligned16(p.A) || !aligned16(p.W) || !aligned16(p.C) || (p.lda % 8) || (p.ldw % 8) ||
      (p.ldc % 2) || (p.R && ((p.ldr % 2) || (reinterpret_cast<uintptr_t>(p.R) & 7)))) {
    set_error("linear: operands must be 16-byte aligned with leading dimensions %% 8 == 0");
    return BSRL_ERR_ALIGN;
  }
  if (p.M == 0) return BSRL_OK;
  static DeviceOnce once;
  int rc = once.run("linear_mma_kernel set-up", [] {
    return cudaFuncSetAttribute(linear_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STAGES * STAGE_BYTES);
  });
  if (rc != BSRL_OK) return rc;
  int64_t tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  if (tiles > 0x7fffffffLL) {
    set_error("linear: too many tiles");
    return BSRL_ERR_SHAPE;
  }
  linear_mma_kernel<<<static_cast<unsigned>(tiles), THREADS, STAGES * STAGE_BYTES, stream>>>(p);
  BSRL_LAUNCH_OK("linear_mma_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
