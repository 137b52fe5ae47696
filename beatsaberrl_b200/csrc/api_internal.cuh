// Pieces of the forward's launch sequence shared by the inference entry points (api.cu) and the
// training entry points (train.cu): the per-call context, byte-offset helpers and the stage-labelled
// wrappers of the GEMM / LayerNorm / attention launchers.
#pragma once
#include <functional>
#include "kernels.cuh"
#include "layout.h"

namespace bsrl {
namespace fwd {

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }
template <typename T>
inline T* at(void* base, int64_t off) {
  return reinterpret_cast<T*>(static_cast<uint8_t*>(base) + off);
}
template <typename T>
inline const T* at(const void* base, int64_t off) {
  return reinterpret_cast<const T*>(static_cast<const uint8_t*>(base) + off);
}

#define BSRL_TRY(expr)             \
  do {                             \
    int rc__ = (expr);             \
    if (rc__ != BSRL_OK) return rc__; \
  } while (0)

constexpr int kMaxBlocks = 32;

// Where a grad-mode forward keeps what the backward needs (all caller memory): the tokenizer's feature
// rows, the key bias, the residual stream ENTERING every block (block i reads x[i] and writes x[i + 1]
// instead of updating one buffer in place), the readout rows and the head / value-bin outputs.
struct TrainPtrs {
  __half* feat;          // (29 B, 64) f16
  float* key_bias;       // (B, 29) f32
  float* x[kMaxBlocks];  // (29 B, d) f32, x[i] = stream entering block i
  __half* lead16;        // (B, 5 d) f16 readout
  float* raw;            // (B, head_cols_pad) f32
  float* vraw;           // (B, bins_pad) f32
};

struct Ctx {
  const bsrl_config* cfg;
  Layout l;
  Paths paths;
  Workspace w;
  const void* arena;
  void* ws;
  int64_t B;
  cudaStream_t st;
  __half* obs16 = nullptr;          // optional fp16 copy of the obs rows, written by the tokenizer kernel
  const TrainPtrs* train = nullptr; // grad-mode forward: intermediates the backward needs go here
  const __half* W(const Mat& m, int row0 = 0) const { return at<__half>(arena, m.w) + (int64_t)row0 * m.pitch; }
  const float* Bv(const Mat& m, int row0 = 0) const { return at<float>(arena, m.b) + row0; }
  const float* G(const Norm& n) const { return at<float>(arena, n.g); }
  const float* Be(const Norm& n) const { return at<float>(arena, n.b); }
};

int make_ctx(Ctx& c, const bsrl_config* cfg, const void* arena, int64_t n_envs, void* ws, int64_t ws_bytes, void* stream);
int run_embed(const Ctx& c, const void* obs, int obs_dtype, float* x, float* key_bias, __half* h_out = nullptr,
              bool* have_h = nullptr);
int run_forward(const Ctx& c, const void* obs, int obs_dtype, const HeadTailArgs& tail_in);
void head_shape(const bsrl_config& cfg, const Layout& l, HeadTailArgs& t);

// makes the calling thread's launch wrappers follow the process-wide engine choice (bsrl_set_engine)
void use_process_engine();
int process_engine();

// stage labels of the optional per-launch profiler (names in api.cu, same order)
enum Stage { kStGather = 0, kStEncoder, kStEncoderFused, kStLayerNorm, kStQkv, kStAttention, kStOutProj, kStFfnUp,
             kStFfnDown, kStBlockTail, kStAttnBlock, kStTrunk, kStCritic, kStHeadTail, kStCount };
void set_stage(int stage);            // label of the launches that follow on this thread
int timed_call(cudaStream_t st, double flops, double bytes, const std::function<int()>& fn);
int fused_tail(const BlockTailArgs& a, cudaStream_t st);
int fused_attn(const AttnBlockArgs& a, cudaStream_t st);
int out_proj_ln(const LinearLnArgs& a, cudaStream_t st);

// stage-labelled launch wrappers (timed when the calling thread has the profiler on)
int linear(const LinearArgs& p, cudaStream_t st);
// a product with row-contraction operands (a_mn / w_mn) can run as asked (engine and shape)
bool linear_rows_ok(const LinearArgs& p);
int layernorm(const float* x, int64_t ldx, RowMap xmap, const float* g, const float* b, float eps, int64_t rows, int d,
              __half* y, int64_t ldy, cudaStream_t st);
int attention(const __half* qkv, int ld, const float* kb, int64_t B, int d, int H, int q0, int nq, __half* out, int ldo,
              cudaStream_t st);

}  // namespace fwd
}  // namespace bsrl
