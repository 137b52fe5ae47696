// Byte layout of the packed weight arena and of the forward workspace (host only).
//
// The arena is this library's form of the reference's flat fp16 replica buffer
// (flatten_fp16_replicas, python/fp16_linear.py:220-427): fp16 GEMM operands in nn.Linear's
// (out, in) layout -- K-contiguous, which is what both MMA engines want for the B operand --
// with q|k|v, the critic's k|v and the 29 heads stacked into single matrices, first-layer
// encoder weights K-padded with zero columns, and fp32 biases / LayerNorm parameters.
#pragma once
#include <string>
#include <vector>

#include "common.cuh"
#include "obs_layout.h"

namespace bsrl {

struct Mat {          // fp16 (rows, pitch) matrix + fp32 bias(rows) in the arena
  int64_t w = 0, b = 0;
  int rows = 0, cols = 0, pitch = 0;
};
struct Norm {         // fp32 gamma, beta
  int64_t g = 0, b = 0;
  int width = 0;
};
struct BlockW {
  Norm ln_attn, ln_ffn;
  Mat qkv, out, up, down;
  Mat qkv_g;   // q|k|v rows regrouped per head group for the fused attention kernel (see attn_G)
  int64_t vres = -1;   // value residual: fp32 {vres_a, vres_b} of this block (blocks after the first), or -1
};
struct Encoder {
  Mat l0, l1;
};

struct Layout {
  int d, H, L, F, D, Hh, bins, bins_pad, k_max, n_head_cols, head_cols_pad, note_in, note_k;
  Encoder note, saber, torso, leg;
  std::vector<BlockW> blocks;
  Mat trunk_proj, trunk_fc1, trunk_fc2, heads;
  Norm trunk_ln1, trunk_ln2, critic_ln;
  Norm emb_ln, final_ln;   // optional (width 0 when the option is off)
  Mat critic_q, critic_kv, critic_out, critic_m0, critic_m1, critic_m2;
  Mat critic_qkv_g;   // critic q|k|v regrouped like BlockW::qkv_g
  int attn_G = 0;     // heads per group of the fused QKV+attention kernel; 0 = shape not supported
  int value_residual = 0;
  int trunk_v2 = 0;                    // SimBaV2 trunk: trunk_proj / fc1 / fc2 hold W_in / W1 / W2 ...
  int64_t v2_s_in = -1, v2_s_1 = -1, v2_alpha = -1;   // ... and these its fp32 scalers (D, Hh, D)
  int head_first[kActHeads];
  int64_t bytes = 0;
};

// One fp32 master parameter and where it lands in the arena.
struct ParamSlot {
  std::string name;
  int64_t rows, cols;      // master shape (cols = 1 for vectors)
  int64_t dst;             // byte offset in the arena
  int64_t dst_pitch;       // elements per destination row (fp16 matrices); 0 for fp32 vectors
  bool half;
};

// A second destination for (a row range of) a master parameter: the regrouped q|k|v copies.
struct CopySlot {
  int param;               // index into make_param_slots()
  int64_t src_row0, n_rows, cols;
  int64_t dst, dst_pitch;
  bool half;
};

// scatter (and optionally AdamW-update) a list of masters into an arena (optim.cu)
int multi_pack_slots(const std::vector<ParamSlot>& slots, const std::vector<CopySlot>& copies, float* const* params,
                     const float* const* grads, float* const* exp_avg, float* const* exp_avg_sq, const float* lr,
                     const float* wd, float beta1, float beta2, float eps, int step, const float* inv_scale,
                     const float* found_inf, void* arena, cudaStream_t stream);

int validate_config(const bsrl_config* c);
Layout make_layout(const bsrl_config& c);
std::vector<ParamSlot> make_param_slots(const bsrl_config& c, const Layout& l);
std::vector<CopySlot> make_copy_slots(const bsrl_config& c, const Layout& l, const std::vector<ParamSlot>& params);

// Which kernels a forward of this shape runs: the fused tcgen05 kernels where the widths fit them
// (and the engine override allows), separate GEMM / LayerNorm / attention kernels otherwise.  The
// workspace only holds the intermediates of the path taken.
struct Paths {
  bool attn_fused;   // q|k|v projection + attention in one kernel (no (rows, 3d) buffer)
  bool tail_fused;   // out-projection + LayerNorm + FFN in one kernel (no (rows, 4d) hidden buffer)
  bool enc_fused;    // both encoder layers + block 0's LayerNorm in one kernel
};
Paths plan_paths(const Layout& l, int engine);

// Workspace carve-up for a batch of n_envs (offsets of buffers the path does not use are -1).
struct Workspace {
  int64_t key_bias, f_saber, f_torso, f_leg, f_note, enc_hid, x, h, qkv, att, hid;
  int64_t x_lead, h_lead, lead16, xt, u, r, z, m1, m2, raw, vraw, att_c;
  int64_t v0;   // block 0's attention values (B*29, d) fp16 (value residual only)
  int64_t t32;  // SimBaV2 trunk: fp32 GEMM outputs (B, max(D, Hh))
  int64_t bytes;
};
Workspace make_workspace(const Layout& l, int64_t n_envs, const Paths& paths);

}  // namespace bsrl
