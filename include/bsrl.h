/*
 * bsrl.h -- C ABI of the B200 policy-forward library (libbsrl.so).
 *
 * Every entry point takes plain pointers and sizes.  Device buffers are owned by the
 * caller; the library never allocates or frees device memory and never synchronises
 * the host with the device: work is enqueued on the stream passed in (a cudaStream_t
 * passed as void*; NULL = the legacy default stream).  Return value: 0 on success, a
 * negative bsrl_status otherwise, with a thread-local message behind bsrl_last_error().
 * All argument checks happen on the host before the first launch.
 *
 * Threads and devices: entry points may be called from several host threads, each on its own
 * stream / device; the stage profiler is per host thread; per-device set-up (kernel attributes,
 * device-symbol addresses) is done once per device under a lock and belongs to the device's
 * primary context, so do not call cudaDeviceReset between calls.
 *
 * The entry points replace, for the policy-forward path, what the reference binds through
 * its two pybind11 torch extensions and the torch library calls around them:
 *   layer_norm_cuda {ln_fwd, ln_fwd_add}   python/beat_arena_env/csrc/layer_norm.cu:733-749
 *   fp16_gemm {attn29_fwd, ffn_fused, linear_relu_aux, bias_relu_}
 *                                          python/beat_arena_env/csrc/fp16_gemm.cu:535-566
 *   torch.addmm / F.linear / SDPA on the fp16 stream      python/fp16_linear.py:134-181, :866-909
 */
#ifndef BSRL_H_
#define BSRL_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSRL_ABI_VERSION 3
#define BSRL_OBS_DIM 630
#define BSRL_N_TOKENS 29
#define BSRL_N_LEAD 5
#define BSRL_N_SLOTS 24
#define BSRL_N_ACT_HEADS 29

typedef enum bsrl_status {
  BSRL_OK = 0,
  BSRL_ERR_NULL = -1,        /* a required pointer is NULL */
  BSRL_ERR_SHAPE = -2,       /* a size is out of range for the configuration */
  BSRL_ERR_ALIGN = -3,       /* a pointer is not aligned as required (16 bytes) */
  BSRL_ERR_WORKSPACE = -4,   /* workspace or arena smaller than the *_bytes() figure */
  BSRL_ERR_UNSUPPORTED = -5, /* valid in the reference, not built here */
  BSRL_ERR_CUDA = -6,        /* a CUDA call or launch failed */
  BSRL_ERR_TIMEOUT = -7      /* a bounded device-side wait ran out */
} bsrl_status;

typedef enum bsrl_dtype {
  BSRL_F32 = 0, BSRL_F16 = 1, BSRL_U8 = 2, BSRL_I32 = 3, BSRL_I64 = 4
} bsrl_dtype;

/* Shape of the network: the keyword arguments of the reference constructor that change
 * the forward (NotePolicy.__init__, python/policy.py:795-806). */
typedef struct bsrl_config {
  int32_t embed;         /* d */
  int32_t n_heads;       /* attention heads, head_dim = embed / n_heads in {32, 48, 64} */
  int32_t n_blocks;      /* transformer blocks (>= 1); the last runs on the lead rows */
  int32_t ffn_mult;      /* FFN hidden = ffn_mult * embed */
  int32_t trunk_dim;     /* D */
  int32_t trunk_hidden;  /* SimBa trunk hidden width */
  int32_t value_bins;    /* HL-Gauss bins */
  int32_t note_geo;      /* 1 = append the 22 hand-relative geometry lanes to each slot */
  int32_t head_gears[BSRL_N_ACT_HEADS]; /* action ids per head, each in [3, 7] */
  float z_asinh;         /* obs z encoding constant (metres) */
  float value_vmax;      /* bin centres = linspace(-vmax, vmax, bins) */
  float eps;             /* LayerNorm epsilon */
  /* A/B options of the reference constructor, all 0 by default (python/policy.py:804-805): */
  int32_t emb_ln;        /* 1 = LayerNorm on the token embeddings (--emb-ln, :1261-1262) */
  int32_t final_ln;      /* 1 = LayerNorm on the lead rows leaving the last block (--final-ln, :1306-1307) */
  int32_t game_flux;     /* 1 = the Flux game's note-geo variant: bar slots aim at lanes 12, 13 (:357-360) */
  int32_t value_residual; /* 1 = blocks after the first mix block 0's attention values in,
                           * v <- vres_a v + vres_b v0 (--value-residual, :512-520, :604-615) */
  int32_t trunk_v2;      /* 1 = SimBaV2 readout trunk (--trunk-arch simbav2, :984-1021, :1140-1155):
                           * parameters trunk_in / trunk_w1 / trunk_w2, trunk_s_in, trunk_s_1, trunk_alpha */
} bsrl_config;

/* --- library -------------------------------------------------------------------- */
int bsrl_abi_version(void);
const char* bsrl_last_error(void);

/* Checks a configuration against what the kernels are built for.
 * Mirrors the constructor checks at python/policy.py:808-850. */
int bsrl_config_validate(const bsrl_config* cfg);

/* Multiply-accumulates of one env-forward (dense over all 29 keys). */
int64_t bsrl_mac_per_env(const bsrl_config* cfg);

/* --- weights -------------------------------------------------------------------- *
 * The packed arena plays the role of the reference's flat fp16 replica buffer
 * (flatten_fp16_replicas / flat_refresh, python/fp16_linear.py:220-427;
 * NotePolicy.flatten_fp16 / refresh_fp16_caches, python/policy.py:1405-1461):
 * fp16 GEMM operands with q|k|v, critic k|v and the 29 heads stacked, fp32 biases and
 * LayerNorm parameters.  Re-running bsrl_pack_weights refreshes it in place. */
int32_t bsrl_param_count(const bsrl_config* cfg);
/* i-th fp32 master in reference state_dict naming ("blocks.0.q_proj.weight", ...);
 * rows x cols of the master (cols = 1 for vectors). */
int bsrl_param_desc(const bsrl_config* cfg, int32_t i, char* name, int32_t name_cap,
                    int64_t* rows, int64_t* cols);
int64_t bsrl_weights_bytes(const bsrl_config* cfg);
int bsrl_pack_weights(const bsrl_config* cfg, const float* const* params, int32_t n_params,
                      void* arena, int64_t arena_bytes, void* stream);

/* Optimizer step and arena refresh in one pass: an Adam / AdamW update of every fp32 master that has
 * a gradient, written straight into the master AND into its fp16 / fp32 places in the arena by the
 * same kernel, so that no separate refresh follows opt.step().  Replaces the pair
 * "fused Adam step, then bump_weights_version() + flat fp16 recast" of the reference trainer
 * (python/train_batch.py:2847-2854, python/fp16_linear.py:236-246).  Arithmetic of torch.optim.AdamW:
 *   g' = g * *inv_scale;  p *= 1 - lr wd;  m = b1 m + (1 - b1) g';  v = b2 v + (1 - b2) g'^2;
 *   p -= lr / (1 - b1^step) * m / (sqrt(v) / sqrt(1 - b2^step) + eps)
 * params / grads / exp_avg / exp_avg_sq: n_params DEVICE pointers each, in bsrl_param_desc order;
 * grads[i] == NULL leaves master i unchanged and only re-scatters it (frozen parameters, or ones
 * another optimizer owns).  lr and weight_decay: n_params HOST floats (weight_decay may be NULL = 0).
 * inv_scale / found_inf: optional DEVICE scalars of a loss scaler (non-zero found_inf skips every
 * update).  The arena must have been packed once by bsrl_pack_weights (which also zeroes its padding).
 * A handful of launches for the whole model; nothing allocated. */
int bsrl_adam_step_pack(const bsrl_config* cfg, float* const* params, const float* const* grads,
                        float* const* exp_avg, float* const* exp_avg_sq, int32_t n_params, const float* lr,
                        const float* weight_decay, float beta1, float beta2, float eps, int32_t step,
                        const float* inv_scale, const float* found_inf, void* arena, int64_t arena_bytes,
                        void* stream);

/* The last stage of an optimizer whose update direction is computed by the caller (the Muon half of the reference's
 * hybrid optimizer, python/train_batch.py:854-931: momentum, Newton-Schulz orthogonalisation, scale): params[i] +=
 * updates[i] (fp32, in place; NULL = untouched) and every parameter's places in the arena are rewritten in the same
 * kernel, as in bsrl_adam_step_pack.  found_inf (device float, may be NULL): non-zero skips the updates. */
int bsrl_apply_updates_pack(const bsrl_config* cfg, float* const* params, const float* const* updates, int32_t n_params,
                            const float* found_inf, void* arena, int64_t arena_bytes, void* stream);

/* --- forward -------------------------------------------------------------------- */
int64_t bsrl_workspace_bytes(const bsrl_config* cfg, int64_t n_envs);

/* NotePolicy.forward_stacked (python/policy.py:1179-1344): obs (n_envs, 630) f32 or f16
 * -> logits (n_envs, 29, k_max) f32 with -1e9 on lanes past a head's gear count, value
 * (n_envs) f32.  value_logits (n_envs, value_bins) f32 is optional (NULL to skip): the
 * reference keeps it as NotePolicy._value_logits (python/policy.py:1402). */
int bsrl_forward(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                 int64_t n_envs, float* logits, float* value, float* value_logits,
                 void* workspace, int64_t workspace_bytes, void* stream);

/* bsrl_forward for callers that cannot hand over a workspace.  Same inputs, outputs and
 * arithmetic as bsrl_forward, but the intermediates live in a 32 MiB scratch array built into
 * the library (bsrl_fixed_scratch_bytes()), so this call needs no workspace argument and
 * allocates nothing -- no cudaMalloc, no cudaFree, no allocating library routine.  It is meant
 * for hosts that own no device allocator of their own or may not allocate where they call from:
 * a simulator-side C/C++ thread or a replay/evaluation tool that wants a handful of policy
 * forwards without linking torch, or code running under a fixed device-memory budget in which
 * any late cudaMalloc could fail or stall the other streams.
 *   - Batches whose bsrl_workspace_bytes() exceeds the built-in scratch are refused with
 *     BSRL_ERR_WORKSPACE (about 190 envs at embed 256, about 390 at embed 128).
 *   - The first call on each device looks up the scratch's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before any stream
 *     capture begins.
 *   - All calls on a device share the one scratch and it keeps the last call's contents.  Nothing
 *     in it needs clearing between calls, but two calls whose kernels overlap on the GPU (two
 *     streams, two host threads) race on it: serialise them, or use bsrl_forward.
 *   - Every GPU that loads the library holds the 32 MiB until the process exits.
 * This entry point has no counterpart in the reference (its extensions allocate through torch). */
int64_t bsrl_fixed_scratch_bytes(void);
int bsrl_forward_fixed(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                       int64_t n_envs, float* logits, float* value, void* stream);

/* NotePolicy.get_action_and_value with given actions (python/policy.py:1467-1516), the PPO
 * recompute call: same forward, then log-softmax, summed log-prob of the given actions and
 * entropy fused into the head kernel.  actions (n_envs, 29) u8 / i32 / i64.
 * logits, entropy, ent_head (n_envs, 29) and value_logits may be NULL. */
int bsrl_forward_act(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                     int64_t n_envs, const void* actions, int32_t act_dtype,
                     float* logits, float* logprob, float* entropy, float* ent_head,
                     float* value, float* value_logits,
                     void* workspace, int64_t workspace_bytes, void* stream);

/* NotePolicy.get_action_and_value with action=None (python/policy.py:1475-1490), the rollout call:
 * same forward, then actions are drawn in the head kernel by Gumbel-max on the log-softmax
 * (argmax_i logsm_i - log E_i, E ~ Exp(1); lanes past a head's gear count never win), with the
 * summed log-prob of the drawn actions and the entropy.  Random numbers are Philox4x32-10 keyed by
 * rng_state[0] (seed) and counted by (env, head, rng_state[1]); rng_state is a DEVICE pointer to
 * two uint64 that the caller advances between calls (e.g. rng_state[1] += 1 on the same stream),
 * so a captured CUDA graph draws fresh numbers on every replay.  The stream of numbers differs from
 * torch's generator, as the reference's own switch to Gumbel-max did.
 * action_out (n_envs, 29) i64; logits, entropy, ent_head may be NULL. */
int bsrl_forward_sample(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                        int64_t n_envs, const uint64_t* rng_state, int64_t* action_out, float* logits,
                        float* logprob, float* entropy, float* ent_head, float* value, void* workspace,
                        int64_t workspace_bytes, void* stream);

/* One rollout tick with the trainer's per-tick buffer stores fused in -- the loop body of the
 * rollout (python/train_batch.py:2299-2350: b_obs[t] = obs; a, logp, _, v = get_action_and_value(obs);
 * b_act[t], b_logp[t] = a, logp; b_val[t].copy_(v).mul_(ret_sig).add_(ret_mu)).  Samples like
 * bsrl_forward_sample and writes, from the same kernels:
 *   act_u8    (n_envs, 29) u8   row t of the uint8 action buffer (python/train_batch.py:1963-1970)
 *   logprob   (n_envs)     f32  row t of b_logp
 *   value_buf (n_envs)     f32  row t of b_val: value * *ret_sigma + *ret_mu (DEVICE scalars of the
 *                               return normaliser, python/train_batch.py:1986-1988; NULL = 1 / 0)
 *   obs16     (n_envs, 630) f16 row t of the half-precision obs buffer (--fp16 all,
 *                               python/train_batch.py:1953-1962), written by the tokenizer kernel that
 *                               reads the row anyway
 * action_out (n_envs, 29) i64 feeds the env step.  action_out or act_u8 must be given; act_u8,
 * value_buf, obs16, entropy and ent_head may be NULL. */
int bsrl_forward_rollout(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                         int64_t n_envs, const uint64_t* rng_state, int64_t* action_out, uint8_t* act_u8,
                         float* logprob, float* entropy, float* ent_head, float* value, float* value_buf,
                         const float* ret_sigma, const float* ret_mu, void* obs16, void* workspace,
                         int64_t workspace_bytes, void* stream);

/* --- training: grad-mode forward and backward --------------------------------------- *
 * The PPO update's recompute (python/train_batch.py:2669-2741): get_action_and_value(obs, action) in
 * grad mode, then loss.backward().  The reference gets its backward from autograd over its
 * autograd.Functions (python/fp16_linear.py:461-767, :931-1064, :1197-1251; python/fused_ln.py:58-107)
 * and their kernels (ln_bwd*, attn29_bwd, wgrad / wgrad_bgrad / dgrad_drelu / relu_bwd); here the two
 * halves are two calls.  Not built for emb_ln / final_ln / value_residual / trunk_v2 (BSRL_ERR_UNSUPPORTED).
 *
 * bsrl_forward_train: same arguments and outputs as bsrl_forward_act, computed by the same kernels
 * (outputs are bit-identical to bsrl_forward_act's), plus a caller-owned `save` buffer of
 * bsrl_train_save_bytes() that receives what the backward needs: the tokenizer's feature rows, the key
 * bias, the residual stream entering every block, the readout rows, the head outputs. */
int64_t bsrl_train_save_bytes(const bsrl_config* cfg, int64_t n_envs);
int bsrl_forward_train(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype, int64_t n_envs,
                       const void* actions, int32_t act_dtype, float* logits, float* logprob, float* entropy,
                       float* ent_head, float* value, float* value_logits, void* save, int64_t save_bytes,
                       void* workspace, int64_t workspace_bytes, void* stream);

/* bsrl_backward: gradients of every parameter given the upstream gradients (DEVICE fp32, any may be
 * NULL = zero) of logprob (n_envs), entropy (n_envs), value (n_envs), value_logits (n_envs, value_bins)
 * and logits (n_envs, 29, k_max).  grads: ONE flat fp32 buffer of bsrl_grad_floats() floats; parameter i
 * (bsrl_param_desc order, master shape) starts at offsets[i] (every slot 16-byte aligned); the call
 * zeroes it first.  Each block's intermediates are recomputed from the saved block input; matrix
 * products run on the tcgen05 GEMM (weight gradients as split-K products over the token rows).
 * Activation gradients travel as fp16 multiplied by loss_scale, and the parameter gradients come out
 * multiplied by loss_scale too: divide by it (pick it so that loss_scale * |upstream| stays well inside
 * fp16 range; 1024-65536 for mean-reduced PPO losses).  workspace: bsrl_backward_workspace_bytes(). */
int64_t bsrl_backward_workspace_bytes(const bsrl_config* cfg, int64_t n_envs);
int64_t bsrl_grad_floats(const bsrl_config* cfg, int64_t* offsets, int32_t n_offsets);
int bsrl_backward(const bsrl_config* cfg, const void* arena, int64_t n_envs, const void* actions, int32_t act_dtype,
                  const void* save, int64_t save_bytes, const float* g_logprob, const float* g_entropy,
                  const float* g_value, const float* g_value_logits, const float* g_logits, float loss_scale,
                  float* grads, int64_t grad_floats, void* workspace, int64_t workspace_bytes, void* stream);

/* Single stages of the backward, for unit tests.
 * bsrl_layernorm_bwd: gx = (g_residual ? g_residual : 0) + dLayerNorm(gy; x, gamma), g_gamma / g_beta
 *   ACCUMULATE (zero them first); all fp32, rows x d (ln_bwd with the fused residual gradient,
 *   python/beat_arena_env/csrc/layer_norm.cu:289-519).
 * bsrl_attention_bwd: gradients of the packed projection for g_out (n_envs*n_q, d) f16: gq (n_envs*n_q, d),
 *   gkv (n_envs*29, 2d) = [gk | gv], fp16 (attn29_bwd, python/beat_arena_env/csrc/small_attn.cu:345-463).
 * bsrl_head_tail_bwd: gradients (fp16, times `scale`) of the packed head outputs and value-bin logits from
 *   the upstream gradients of logprob / entropy / value / value_logits / logits (any may be NULL).
 * bsrl_linear_bwd: for y = x w^T + b with x (m, k), w (n, k), g = dL/dy (m, n) fp16: g_weight (n, k) f32 +=
 *   g^T x (split-K tcgen05 product over the m rows; zero it first), g_bias (n) += column sums, g_x (m, k) =
 *   g w (fp16 or fp32); any output may be NULL (wgrad / wgrad_bgrad / dgrad of
 *   python/beat_arena_env/csrc/fp16_gemm.cu:252-373, :499-518). */
int bsrl_layernorm_bwd(const float* x, const float* gamma, float eps, const float* gy, const float* g_residual,
                       int64_t rows, int32_t d, float* gx, float* g_gamma, float* g_beta, void* stream);
int bsrl_attention_bwd(const void* qkv_f16, const float* key_bias, int64_t n_envs, int32_t d, int32_t n_heads,
                       int32_t q_first, int32_t n_q, const void* g_out_f16, void* gq_f16, void* gkv_f16, void* stream);
int bsrl_head_tail_bwd(const bsrl_config* cfg, const float* head_out, const float* value_bin_logits, int64_t n_envs,
                       const void* actions, int32_t act_dtype, const float* g_logprob, const float* g_entropy,
                       const float* g_value, const float* g_value_logits, const float* g_logits, float scale,
                       void* g_head_out_f16, int32_t ld_g_head, void* g_value_bins_f16, int32_t ld_g_bins, void* stream);
int64_t bsrl_linear_bwd_scratch_bytes(int64_t m, int32_t n, int32_t k);
int bsrl_linear_bwd(const void* g_f16, const void* x_f16, const void* w_f16, int64_t m, int32_t n, int32_t k,
                    float* g_weight, float* g_bias, void* g_x, int32_t g_x_f32, void* scratch, int64_t scratch_bytes,
                    void* stream);

/* --- the single-body-token layout ---------------------------------------------------- *
 * A second front / back end around the same transformer core, for policies laid out as one body token
 * plus n_obj object tokens (T = 1 + n_obj, e.g. 17 / 33 / 65):
 *   obs (n_envs, body_dim + n_obj * obj_dim + n_obj) f32 = body | objects | per-object live flag (0 / 1)
 *   token 0 = Linear(body_dim, embed)(body);  token 1 + j = Linear(obj_dim, embed)(object j)
 *   n_blocks pre-LN blocks with an exact-GELU FFN, absent objects masked as keys, the last block on the
 *   body row only;  heads Linear(embed, 29 * n_gears) -> logits (n_envs, 29, n_gears);  value Linear(embed, 1)
 * The reference has no such tokenizer or readout (python/policy.py:174-275, :940-952, :1107-1138, :1346-1403
 * are fixed at 29 tokens, 2-layer ReLU encoders, a SimBa trunk and a distributional critic); its blocks are
 * the reference's Block (python/policy.py:524-715) with the FFN activation swapped, which is what this
 * layout's parity oracle composes.  Parameter names: body_enc, obj_enc, blocks.i.{ln_attn, q_proj, k_proj,
 * v_proj, out_proj, ln_ffn, ffn.0, ffn.2}, heads, value. */
typedef struct bsrl_gconfig {
  int32_t embed, n_heads, n_blocks, ffn_mult;
  int32_t n_obj;       /* object tokens (1..95) */
  int32_t n_gears;     /* logits per action head (3..7) */
  int32_t body_dim;    /* e.g. 340 */
  int32_t obj_dim;     /* e.g. 16 (<= 64) */
  float eps;           /* LayerNorm epsilon */
} bsrl_gconfig;
int bsrl_g_config_validate(const bsrl_gconfig* cfg);
int32_t bsrl_g_obs_dim(const bsrl_gconfig* cfg);
int64_t bsrl_g_mac_per_env(const bsrl_gconfig* cfg);
int32_t bsrl_g_param_count(const bsrl_gconfig* cfg);
int bsrl_g_param_desc(const bsrl_gconfig* cfg, int32_t i, char* name, int32_t name_cap, int64_t* rows, int64_t* cols);
int64_t bsrl_g_weights_bytes(const bsrl_gconfig* cfg);
int bsrl_g_pack_weights(const bsrl_gconfig* cfg, const float* const* params, int32_t n_params, void* arena,
                        int64_t arena_bytes, void* stream);
int64_t bsrl_g_workspace_bytes(const bsrl_gconfig* cfg, int64_t n_envs);
/* Forward; with actions (n_envs, 29) u8 / i32 / i64 also the summed log-prob, entropy and per-head entropy
 * from the fused head kernel.  logits, logprob, entropy, ent_head may be NULL (logits or logprob must be given). */
int bsrl_g_forward(const bsrl_gconfig* cfg, const void* arena, const float* obs, int64_t n_envs, const void* actions,
                   int32_t act_dtype, float* logits, float* logprob, float* entropy, float* ent_head, float* value,
                   void* workspace, int64_t workspace_bytes, void* stream);

/* --- single stages (unit tests and profiling) -------------------------------------- */

/* Obs lane of feature k of lead token tok (0..4), or -1 past the token's width
 * (index tables at python/policy.py:211-266). */
int32_t bsrl_token_lane(int32_t tok, int32_t k);

/* Tokenizer + four encoders: obs -> resolved token stream x (n_envs*29, d) f32 and additive
 * key bias (n_envs, 29) f32 (python/policy.py:1198-1260). */
int bsrl_embed(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
               int64_t n_envs, float* x, float* key_bias,
               void* workspace, int64_t workspace_bytes, void* stream);

/* LayerNorm rows of x (rows, d) f32 -> y (rows, d) f16, fp32 statistics
 * (FusedLayerNorm.forward, python/fused_ln.py:126-138). */
int bsrl_layernorm(const float* x, const float* gamma, const float* beta, float eps,
                   int64_t rows, int32_t d, void* y_f16, int64_t ldy, void* stream);

/* y = act(a @ w^T + bias) (+ residual): a (m, k) f16 row-major, w (n, k) f16 row-major,
 * bias (n) f32 or NULL, residual (m, n) f32 or NULL; out f16 (out_f32 = 0) or f32.
 * k % 32 == 0, n % 8 == 0.  (fp16_linear / fp16_linear_relu, python/fp16_linear.py:633-641,
 * :794-805.)  engine 0 = warp-MMA kernel, 1 = tcgen05/TMEM kernel (k % 64 == 0). */
int bsrl_linear(const void* a_f16, const void* w_f16, const float* bias, const float* residual,
                void* out, int32_t out_f32, int32_t relu, int64_t m, int32_t n, int32_t k,
                int32_t engine, void* stream);

/* x_out = residual + a @ w^T + bias (fp32) and h = LayerNorm(x_out; gamma, beta, eps) (fp16) in one tcgen05
 * kernel: a (m, k) f16, w (n, k) f16, residual / x_out (m, n) f32 (may be the same buffer), h (m, n) f16.
 * n a multiple of 64 up to 512 (of 128 above 256), k a multiple of 64.  (out_proj + ln_ffn.forward_add,
 * python/policy.py:655-668, for rows wider than the fused block tail takes.) */
int bsrl_linear_ln(const void* a_f16, const void* w_f16, const float* bias, const float* residual, const float* gamma,
                   const float* beta, float eps, int64_t m, int32_t n, int32_t k, float* x_out, void* h_f16, void* stream);

/* Masked multi-head attention over 29 keys: qkv (n_envs*29, 3d) f16 packed [q|k|v],
 * key_bias (n_envs, 29) f32, queries = token rows [q_first, q_first + n_q) of each env
 * -> out (n_envs*n_q, d) f16 (attn29_fwd, python/beat_arena_env/csrc/small_attn.cu:515-536;
 * reference arithmetic python/policy.py:686-690). */
int bsrl_attention(const void* qkv_f16, const float* key_bias, int64_t n_envs, int32_t d,
                   int32_t n_heads, int32_t q_first, int32_t n_q, void* out_f16, void* stream);
/* The same over `tokens` (1..96) token rows per env: qkv (n_envs*tokens, 3d), key_bias (n_envs, tokens).
 * With 17 / 33 / 65 tokens (one body token + 16 / 32 / 64 object tokens), all rows or the first row only,
 * the object tokens fill whole tensor-core tiles and the body token is folded in beside them. */
int bsrl_attention_tokens(const void* qkv_f16, const float* key_bias, int64_t n_envs, int32_t tokens, int32_t d,
                          int32_t n_heads, int32_t q_first, int32_t n_q, void* out_f16, void* stream);

/* Fused packed projection + attention of one block (head_dim 32 with an even head count, or head_dim
 * 48; embed <= 256), one tcgen05 kernel:
 *   out = MHA(h Wq^T + bq, h Wk^T + bk, h Wv^T + bv; key_bias), queries = rows [q_first, q_first + n_q)
 * h (n_envs*29, d) f16 -> out (n_envs*n_q, d) f16.  The weights come REGROUPED per head group (two
 * heads of 32, or one head of 48; w = the group's width, 64 or 48): rows [3 w g, 3 w g + w) = Wq rows
 * of group g, the next w = its Wk rows, the next w = its Wv rows; the bias likewise
 * (bsrl_pack_weights builds these copies in the arena).
 * Replaces fp16_packed_linear + attn29_packed / packed_sdpa (python/policy.py:586-600, :645-692). */
int bsrl_qkv_attention(const void* h_f16, const void* w_grouped_f16, const float* b_grouped,
                       const float* key_bias, int64_t n_envs, int32_t d, int32_t n_heads, int32_t q_first,
                       int32_t n_q, void* out_f16, void* stream);
/* The same for the single-body-token layout with 33 tokens per env (one body token + 32 object tokens): h
 * (n_envs*33, d), key_bias (n_envs, 33); qkv0 (n_envs, 3d) f16 = the body rows' own projection [q | k | v] in the
 * plain column order (bsrl_linear on every 33rd row of h).  n_q = 33: out (n_envs*33, d); n_q = 1: the body row
 * only, out (n_envs, d).  head_dim 32, even head count, d <= 256.  No counterpart kernel in the reference. */
int bsrl_qkv_attention_body(const void* h_f16, const void* w_grouped_f16, const float* b_grouped, const void* qkv0_f16,
                            const float* key_bias, int64_t n_envs, int32_t d, int32_t n_heads, int32_t n_q,
                            void* out_f16, void* stream);

/* Fused tail of one transformer block on a (m, d) token stream, one tcgen05 kernel:
 *   x1 = x + att Wo^T + bo;  xo = x1 + relu(LN(x1; ln_g, ln_b) W0^T + b0) W2^T + b2
 * att (m, d) f16, x (m, d) f32, Wo (d, d), W0 (f, d), W2 (d, f) f16 row-major.  Outputs (either
 * may be NULL): x_out (m, d) f32 (may alias x), ln_out (m, d) f16 = LayerNorm(xo; out_g, out_b),
 * or fp16(xo) when out_g is NULL.  d in {64, 128, 192, 256}, f % 256 == 0.
 * Replaces out_proj + ln_ffn.forward_add + fused_ffn (python/policy.py:655-715; ffn_fused,
 * python/beat_arena_env/csrc/fused_ffn.cu:551-619). */
int bsrl_block_tail(const void* att_f16, const float* x, const void* wo_f16, const float* bo,
                    const float* ln_g, const float* ln_b, const void* w0_f16, const float* b0,
                    const void* w2_f16, const float* b2, float eps, int64_t m, int32_t d, int32_t f,
                    float* x_out, void* ln_out_f16, const float* out_g, const float* out_b, void* stream);

/* Readout trunk + packed action heads alone (NotePolicy._trunk and the packed head GEMM,
 * python/policy.py:1107-1155, :1311-1335): readout (n_envs, 5 * embed) f16 = the lead rows leaving the
 * last block -> head_out (n_envs, head_cols_pad) f32, the 29 heads' outputs side by side (bias
 * included, before the masked-lane fill; bsrl_head_layout gives the pitch and each head's first
 * column).  trunk_h (n_envs, trunk_dim) f16 is optional: the trunk output the reference stashes as
 * NotePolicy._diag_h (python/policy.py:1309-1310).  Uses the forward's workspace. */
int bsrl_trunk_heads(const bsrl_config* cfg, const void* arena, const void* readout_f16, int64_t n_envs,
                     float* head_out, void* trunk_h_f16, void* workspace, int64_t workspace_bytes, void* stream);

/* Head tail alone: masked-lane fill, log-softmax, summed log-prob of the given actions, entropy,
 * HL-Gauss value (python/policy.py:1337-1344, :1399-1403, :1473-1516).  head_out (n_envs,
 * head_cols_pad) f32 and value_bin_logits (n_envs, bins_pad) f32 as the forward's GEMMs leave them;
 * actions, logits, logprob, entropy, ent_head may be NULL. */
int bsrl_head_tail(const bsrl_config* cfg, const float* head_out, const float* value_bin_logits, int64_t n_envs,
                   const void* actions, int32_t act_dtype, float* logits, float* logprob, float* entropy,
                   float* ent_head, float* value, void* stream);
/* Row pitches of head_out and value_bin_logits, and the first packed column of each of the 29 heads. */
int bsrl_head_layout(const bsrl_config* cfg, int32_t* head_cols_pad, int32_t* bins_pad, int32_t* head_first);

/* Where a named intermediate of the last forward sits in the caller's workspace (valid until the next
 * call on that workspace): "trunk_h" (the reference's _diag_h), "x_resolved" (the residual stream
 * entering the last block, the critic's input; python/policy.py:1302-1305), "key_bias", "readout",
 * "head_out".  dtype is a bsrl_dtype; ld_elems the row pitch in elements. */
int bsrl_workspace_region(const bsrl_config* cfg, int64_t n_envs, const char* name, int64_t* byte_offset,
                          int64_t* rows, int64_t* cols, int64_t* ld_elems, int32_t* dtype);

/* Stand-in for the simulator's per-tick step kernel (step_kernel,
 * python/beat_arena_env/csrc/beat_arena_cuda.cu:6188-6245), for graph-capture tests and rollout-tick
 * benchmarks only: it has the real kernel's memory behaviour -- reads actions (n_envs, 29) i64,
 * rewrites obs (n_envs, 630) f32, reward (n_envs) f32 and done (n_envs) u8 IN PLACE, advances state
 * (n_envs) u32 -- and none of its physics (the next obs is a hash of state and actions, clipped to
 * +-5, slot-mask lanes 0 or 1).  reward and done may be NULL. */
int bsrl_standin_env_step(const int64_t* actions, int64_t n_envs, uint32_t* state, float* obs, float* reward,
                          uint8_t* done, void* stream);

/* Self-test of the bounded waits: launches a one-CTA kernel whose only thread waits, for at most
 * `polls` polls, on an mbarrier that nothing ever arrives on.  The wait runs out, the kernel sets the
 * device status word (kernel 15, role 1) and returns; the next bsrl_device_status() therefore reports
 * BSRL_ERR_TIMEOUT, and the GPU and the context stay usable.  Nothing traps or hangs.  No counterpart
 * in the reference. */
int bsrl_selftest_wait_timeout(int32_t polls, void* stream);

/* Which GEMM kernel the forward's linear layers use: 0 (default) = the tcgen05/TMEM kernel
 * wherever the shape fits it (and the fused block-tail kernel), the warp-MMA kernel elsewhere;
 * 1 = the warp-MMA kernel and separate LayerNorm kernels everywhere.
 * Both are CUDA kernels of this library; 1 exists so tests can cross-check one against the
 * other.  The choice is process-wide: set it before the first forward and before asking for
 * bsrl_workspace_bytes (the unfused kernels need more workspace).  No counterpart in the reference. */
int bsrl_set_engine(int32_t engine);

/* Synchronises the current device, then reads and clears its status word: BSRL_OK, or
 * BSRL_ERR_TIMEOUT when a bounded wait inside a tcgen05 kernel (on an mbarrier fed by TMA or by
 * the tensor core) ran out since the last call -- the results of that launch are then invalid.
 * The kernels never spin without a limit and never trap.  No counterpart in the reference. */
int bsrl_device_status(void);

/* --- stage timing (benchmarks) ------------------------------------------------------- *
 * When enabled, every launch of a forward is bracketed by CUDA events on the caller's stream
 * and accounted to a stage ("ffn_down_gemm", "attention", ...).  Enabling clears earlier
 * records.  Read the totals after synchronising the stream.  Leave it off while capturing a
 * CUDA graph.  Counterpart in the reference: the per-tick CUDA-event timers of its --bench
 * mode (python/train_batch.py:2120-2124, :2309-2352). */
int bsrl_profile_enable(int32_t on);
int32_t bsrl_profile_stage_count(void);
const char* bsrl_profile_stage_name(int32_t i);
int bsrl_profile_stage(int32_t i, double* ms_total, int64_t* launches, double* flops_total,
                       double* bytes_total);

#ifdef __cplusplus
}
#endif
#endif /* BSRL_H_ */
