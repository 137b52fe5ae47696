// Host-side launchers of every kernel in the library (one translation unit each).
#pragma once
#include "common.cuh"

namespace bsrl {

// C = act(A W^T + bias) (+ R).  A (M, K) f16 and W (N, K) f16, both K-contiguous.
struct LinearArgs {
  const __half* A;
  int lda;
  RowMap amap;
  const __half* W;
  int ldw;
  const float* bias;   // (N) or nullptr
  const float* R;      // residual f32 or nullptr
  int ldr;
  RowMap rmap;
  void* C;             // f16 or f32
  int ldc;
  RowMap cmap;
  int out_f32;
  int relu;            // activation: 0 none, 1 ReLU, 2 exact GELU
  int64_t M;
  int N, K;
  // Split-K (weight gradients: few output tiles, a very long K): the K range is cut into k_splits
  // pieces that run as separate work items and ADD their partial products into the fp32 output with
  // atomics (the caller zeroes C first; bias goes in with the first piece).  0 or 1 = off.
  int k_splits = 0;
  // Operands stored with the contraction index as ROWS (tcgen05 engine only): a_mn = A is a (K, M)
  // row-major matrix with pitch lda, w_mn = W is a (K, N) row-major matrix with pitch ldw.  The tiles
  // are fetched as 64-column blocks and handed to the tensor cores as MN-major operands, so weight
  // gradients (g^T x: the contraction runs over token rows) and input gradients (g W) need no
  // transposed copies.  M % 64 == 0 (a_mn), N % 64 == 0 (w_mn); K is free (rows past K read as zero).
  int a_mn = 0, w_mn = 0;
  // ReLU backward in the epilogue (tcgen05 engine): entries of C whose counterpart in `mask` (fp16, M rows of
  // pitch ldm, dense rows) is not positive are written as zero.
  const __half* mask = nullptr;
  int ldm = 0;
};
LinearArgs linear_args(const __half* A, int lda, const __half* W, int ldw, const float* bias,
                       void* C, int ldc, int out_f32, int relu, int64_t M, int N, int K);

int linear_mma(const LinearArgs& p, cudaStream_t stream);   // warp-MMA engine
int linear_tc5(const LinearArgs& p, cudaStream_t stream);   // tcgen05 / TMEM engine
bool linear_tc5_ok(const LinearArgs& p);                     // shape fits the tcgen05 engine

// Projection + residual + LayerNorm in one kernel (gemm_ln_tc5.cu): x_out = R + A W^T + bias (fp32), h =
// LayerNorm(x_out) (fp16).  N a multiple of 64 up to 512 (of 128 above 256), K a multiple of 64.  R and x_out
// may be the same buffer.
struct LinearLnArgs {
  const __half* A;
  int lda;
  const __half* W;      // (N, K)
  int ldw;
  const float* bias;    // (N) or nullptr
  const float* R;       // (M, ldr) f32
  int64_t ldr;
  float* x_out;         // (M, ldx) f32
  int64_t ldx;
  const float* gamma;   // LayerNorm weight / bias (N)
  const float* beta;
  float eps;
  __half* h;            // (M, ldh) f16
  int64_t ldh;
  int64_t M;
  int N, K;
};
bool linear_ln_ok(const LinearLnArgs& a);
int linear_ln(const LinearLnArgs& a, cudaStream_t stream);

// Fused block tail (out-projection + residual + LayerNorm + FFN + residual + output LayerNorms).
struct BlockTailArgs {
  int d, F;
  int64_t M;
  const __half* att;   // (M, d) f16
  int ld_att;
  const float* x;      // residual stream in, f32, rows mapped by xmap
  int64_t ldx;
  RowMap xmap;
  const __half* wo;    // (d, d)
  const float* bo;
  const float* ln_g;   // ln_ffn
  const float* ln_b;
  const __half* w0;    // (F, d)
  const float* b0;
  const __half* w2;    // (d, F)
  const float* b2;
  float eps;
  float* x_out;        // (M, d) f32 or nullptr
  __half* out16[2];    // fp16 outputs: LayerNorm(xo) with (g16, b16), or plain cast when g16 is null
  int64_t ld16[2];
  const float* g16[2];
  const float* b16[2];
  int gelu;            // 1: the FFN activation is the exact GELU instead of ReLU
};
bool block_tail_ok(const BlockTailArgs& a);
int block_tail(const BlockTailArgs& a, cudaStream_t stream);

// Fused q|k|v projection + masked attention (head_dim 32), weights regrouped per head group.
struct AttnBlockArgs {
  int d, n_heads;
  int64_t n_envs;
  const __half* h;       // (n_envs*29, d) LayerNorm rows
  int ldh;
  const __half* wg;      // regrouped [q|k|v] weight (3d, d)
  const float* bg;       // regrouped bias (3d)
  const float* key_bias; // (n_envs, 29)
  int q_first, n_q;      // query rows of each env
  __half* out;           // (n_envs*n_q, ldo)
  int ldo;
  // value residual (all optional): the block's own values written to v_out (n_envs*29, d) f16; values
  // replaced by vres[0] * v + vres[1] * v0 before the attention (v0 (n_envs*29, d) f16, vres 2 device floats)
  __half* v_out = nullptr;
  const __half* v0 = nullptr;
  const float* vres = nullptr;
  // Single-body-token layout: envs of `tokens` = 33 rows in h / key_bias / out; the 32 object tokens (rows 1..32)
  // are the env's tile, the body token (row 0) is folded in from qkv0 (n_envs, 3d) f16 = its q | k | v in the
  // plain column order (a small projection the caller runs first).  n_q = tokens: out (n_envs*tokens, ldo);
  // n_q = 1: the body row only, out (n_envs, ldo).
  int body = 0, tokens = 29;
  const __half* qkv0 = nullptr;
};
// v columns of a packed projection: copy out (v_out) and / or mix with v0 in place (value residual)
int vres_mix(__half* v, int ld, int64_t rows, int d, __half* v_out, const __half* v0, const float* vres,
             cudaStream_t stream);
bool attn_block_ok(const AttnBlockArgs& a);
int attn_block(const AttnBlockArgs& a, cudaStream_t stream);

// y(f16, ldy) = LayerNorm(x(f32, ldx)) per row, fp32 statistics; layernorm_rows_f32 writes fp32 rows
// (in place allowed).
int layernorm_rows(const float* x, int64_t ldx, RowMap xmap, const float* gamma, const float* beta,
                   float eps, int64_t rows, int d, __half* y, int64_t ldy, cudaStream_t stream);
int layernorm_rows_f32(const float* x, int64_t ldx, const float* gamma, const float* beta, float eps,
                       int64_t rows, int d, float* y, int64_t ldy, cudaStream_t stream);

// SimBaV2 trunk rows (python/policy.py:1140-1155).  mode 0: x = l2n(in * vec) -> x (fp32) and out16;
// mode 1: y = l2n(in), x' = l2n(x + vec c_alpha (y - x)), out16 = sqrt(d) x'.  scale_relu_rows: relu(in * s).
int simba2_rows(int mode, const float* in, float* x, const float* vec, float c_alpha, int64_t rows, int d,
                __half* out16, int64_t ld16, cudaStream_t stream);
int scale_relu_rows(const float* in, const float* s, int64_t rows, int n, __half* out16, cudaStream_t stream);

// Tokenizer: obs -> per-encoder fp16 feature rows + additive key bias.
struct EmbedBuffers {
  __half* saber;  // (2B, ks)
  __half* torso;  // (B, kt)
  __half* leg;    // (2B, kl)
  __half* note;   // (24B, kn)
  float* key_bias;  // (B, 29)
  int ks, kt, kl, kn;
  __half* obs16 = nullptr;   // optional (B, 630) fp16 copy of the observation rows (rollout buffer row)
};
int embed_gather(const void* obs, int obs_dtype, int64_t n_envs, int note_geo, int flux, float z_asinh,
                 const EmbedBuffers& out, cudaStream_t stream);
int token_lane_host(int tok, int k);

// Fused token encoders (both layers of the four MLPs + block 0's LayerNorm), one tcgen05 kernel.
// Encoder order everywhere: saber, torso, leg, note.
struct EncoderArgs {
  int d;
  int64_t n_envs;
  const __half* feat;    // (29 n_envs, 64) f16: 2 n_envs saber rows, n_envs torso, 2 n_envs leg, 24 n_envs note rows
  const __half* w0[4];   // (d, 64) first layers, K-padded
  const float* b0[4];
  int k0[4];             // padded input widths (all 64)
  const __half* w1[4];   // (d, d) second layers
  const float* b1[4];
  const float* ln_g;     // block 0's ln_attn (used when h is given)
  const float* ln_b;
  float eps;
  float* x;              // (29 n_envs, d) f32 token stream out
  __half* h;             // (29 n_envs, d) f16 LayerNorm rows out, or nullptr
};
bool encoder_fused_ok(const EncoderArgs& a);
int encoder_fused(const EncoderArgs& a, cudaStream_t stream);

// Masked MHA over the `tokens` keys of each env (1..96); attention29 is the 29-token case.
int attention_tokens(const __half* qkv, int ld_qkv, const float* key_bias, int64_t n_envs, int tokens, int d,
                     int n_heads, int q_first, int n_q, __half* out, int ldo, cudaStream_t stream);
// Masked MHA over the 29 keys of each env.
int attention29(const __half* qkv, int ld_qkv, const float* key_bias, int64_t n_envs, int d,
                int n_heads, int q_first, int n_q, __half* out, int ldo, cudaStream_t stream);

// Head tail: masked-lane fill, log-softmax, log-prob of given actions, entropy; HL-Gauss value.
struct HeadTailArgs {
  const float* raw;      // (B, ld_raw) packed head outputs, bias included
  int ld_raw;
  const float* vraw;     // (B, ld_v) value-bin logits
  int ld_v;
  int bins;
  float vmax;
  int k_max;
  int gears[kActHeads];
  int first[kActHeads];  // first packed column of each head
  const void* actions;   // (B, 29) or nullptr
  int act_dtype;
  const unsigned long long* rng;   // device [seed, offset]: sample actions (Gumbel-max) when actions is null
  long long* action_out;           // (B, 29) sampled actions
  unsigned char* action_u8;        // (B, 29) the same actions as bytes (rollout buffer row) or nullptr
  float* value_buf;                // (B) value * ret_sigma + ret_mu (rollout buffer row) or nullptr
  const float* ret_sigma;          // device scalars of the return normaliser; nullptr = 1 / 0
  const float* ret_mu;
  float* logits;         // (B, 29, k_max) or nullptr
  float* logprob;        // (B) or nullptr
  float* entropy;        // (B) or nullptr
  float* ent_head;       // (B, 29) or nullptr
  float* value;          // (B)
  float* value_logits;   // (B, bins) or nullptr
  int64_t n_envs;
};
int head_tail(const HeadTailArgs& a, cudaStream_t stream);

// Stand-in for the simulator's step kernel (graph tests / tick benchmarks): actions in, the env's obs row,
// reward and done flag rewritten in place.
int standin_env_step(const long long* actions, int64_t n_envs, uint32_t* state, float* obs, float* reward,
                     unsigned char* done, cudaStream_t stream);

// Scatter of every fp32 master into the packed arena (a few launches), with an optional Adam / AdamW
// step applied to the masters that come with a gradient first (optim.cu).  lr / wd: one value per
// parameter (host arrays) or nullptr; step: 1-based step count for the bias corrections (0: none).
struct Layout;
int multi_pack(const bsrl_config& cfg, const Layout& l, float* const* params, const float* const* grads,
               float* const* exp_avg, float* const* exp_avg_sq, const float* lr, const float* wd, float beta1,
               float beta2, float eps, int step, const float* inv_scale, const float* found_inf, void* arena,
               cudaStream_t stream);

}  // namespace bsrl
