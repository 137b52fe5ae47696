// C ABI of the library: argument checks, then the launch sequence of one policy forward.
//
// The sequence restates NotePolicy._forward_stacked (python/policy.py:1198-1344) as a fixed
// list of kernel launches on the caller's stream, with every intermediate in the caller's
// workspace; nothing here allocates, frees or synchronises, so the whole call can be captured
// in a CUDA graph next to the simulator's step kernel (python/rollout_graph.py:45-74).
#include <string.h>

#include <atomic>
#include <functional>
#include <vector>

#include "api_internal.cuh"
#include "tc5.cuh"

namespace bsrl {
const char* last_error();

namespace fwd {

// ---------------------------------------------------------------- stage profiler
// Optional CUDA-event timing of every launch of a forward, grouped by stage.  Off by default
// (a captured graph must not contain it); the benchmark switches it on to time the dominant
// kernel live, on the stream the kernels run on.
const char* const kStageNames[kStCount] = {"embed_gather", "encoder_gemm", "encoder_fused", "layernorm", "qkv_gemm",
                                           "attention", "out_proj_gemm", "ffn_up_gemm", "ffn_down_gemm", "block_tail", "attn_block",
                                           "trunk", "critic", "head_tail"};
struct Profiler {
  bool on = false;
  struct Rec { int stage; cudaEvent_t e0, e1; double flops, bytes; };
  std::vector<Rec> recs;
  std::vector<cudaEvent_t> pool;
  size_t used = 0;
  cudaEvent_t get() {
    if (used == pool.size()) {
      cudaEvent_t e;
      if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
      pool.push_back(e);
    }
    return pool[used++];
  }
  void reset() { recs.clear(); used = 0; }
};
// Per host thread: each thread that enables the profiler times its own forwards, and forwards
// running on other threads are not affected.
thread_local Profiler g_prof;
thread_local int g_stage = kStGather;   // stage label of the launches that follow

double linear_bytes(const LinearArgs& p) {
  double b = (double)p.M * p.K * 2 + (double)p.N * p.K * 2 + (double)p.M * p.N * (p.out_f32 ? 4 : 2);
  if (p.R) b += (double)p.M * p.N * 4;
  return b;
}

template <typename Fn>
int timed(cudaStream_t st, double flops, double bytes, Fn&& fn) {
  if (!g_prof.on) return fn();
  cudaEvent_t e0 = g_prof.get(), e1 = g_prof.get();
  if (!e0 || !e1) return fn();
  cudaEventRecord(e0, st);
  int rc = fn();
  cudaEventRecord(e1, st);
  g_prof.recs.push_back({g_stage, e0, e1, flops, bytes});
  return rc;
}

// engine choice for one linear layer: tcgen05 where the shape fits, warp-MMA otherwise
// 0 = automatic, 1 = warp-MMA kernel only (cross-check runs).  Process-wide test knob: set it before
// the first forward; each forward reads it once (Ctx::engine), so a change never splits a forward.
std::atomic<int> g_engine{0};
thread_local int g_call_engine = 0;   // the engine of the forward running on this thread
void use_process_engine() { g_call_engine = g_engine.load(std::memory_order_relaxed); }
int process_engine() { return g_engine.load(std::memory_order_relaxed); }
int linear(const LinearArgs& p, cudaStream_t st) {
  return timed(st, 2.0 * p.M * p.N * p.K, linear_bytes(p), [&] {
    if (p.a_mn || p.w_mn || p.mask) {      // row-contraction operands and the epilogue mask: the tcgen05 engine only
      if (g_call_engine == 0 && linear_tc5_ok(p)) return linear_tc5(p, st);
      set_error("linear: row-contraction operands need the tcgen05 engine and M, N multiples of 64 (m=%lld n=%d k=%d)",
                (long long)p.M, p.N, p.K);
      return (int)BSRL_ERR_UNSUPPORTED;
    }
    if (g_call_engine == 0 && p.M >= 128 && linear_tc5_ok(p)) return linear_tc5(p, st);
    return linear_mma(p, st);
  });
}
bool linear_rows_ok(const LinearArgs& p) { return g_call_engine == 0 && linear_tc5_ok(p); }
int layernorm(const float* x, int64_t ldx, RowMap xmap, const float* g, const float* b, float eps,
              int64_t rows, int d, __half* y, int64_t ldy, cudaStream_t st) {
  int keep = g_stage;
  if (g_stage != kStTrunk && g_stage != kStCritic) g_stage = kStLayerNorm;
  int rc = timed(st, 0.0, (double)rows * d * 6, [&] { return layernorm_rows(x, ldx, xmap, g, b, eps, rows, d, y, ldy, st); });
  g_stage = keep;
  return rc;
}
int attention(const __half* qkv, int ld, const float* kb, int64_t B, int d, int H, int q0, int nq,
              __half* out, int ldo, cudaStream_t st) {
  int keep = g_stage;
  if (g_stage != kStCritic) g_stage = kStAttention;
  double fl = 4.0 * B * nq * kT * d;
  double by = (double)B * (kT * 2 * d + nq * d * 2) * 2 + (double)B * kT * 4;
  int rc = timed(st, fl, by, [&] { return attention29(qkv, ld, kb, B, d, H, q0, nq, out, ldo, st); });
  g_stage = keep;
  return rc;
}

void set_stage(int stage) { g_stage = stage; }
int timed_call(cudaStream_t st, double flops, double bytes, const std::function<int()>& fn) { return timed(st, flops, bytes, fn); }

int fused_tail(const BlockTailArgs& a, cudaStream_t st) {
  int keep = g_stage;
  g_stage = kStBlockTail;
  double fl = 2.0 * a.M * ((double)a.d * a.d + 2.0 * a.d * a.F);
  double by = (double)a.M * a.d * (2 + 4 + (a.x_out ? 4 : 0) + (a.out16[0] ? 2 : 0) + (a.out16[1] ? 2 : 0));
  int rc = timed(st, fl, by, [&] { return block_tail(a, st); });
  g_stage = keep;
  return rc;
}

// out-projection + residual + LayerNorm as one kernel where it pays (rows wider than the fused block tail takes, K =
// d: the kernel is HBM-bound and saves the LayerNorm pass), else as the GEMM and the LayerNorm kernel
int out_proj_ln(const LinearLnArgs& a, cudaStream_t st) {
  int keep = g_stage;
  g_stage = kStOutProj;
  int rc;
  if (g_call_engine == 0 && a.N > 256 && a.M >= 128 && linear_ln_ok(a)) {
    rc = timed(st, 2.0 * a.M * a.N * a.K, (double)a.M * (a.K * 2 + a.N * 10.0), [&] { return linear_ln(a, st); });
  } else {
    LinearArgs po = linear_args(a.A, a.lda, a.W, a.ldw, a.bias, a.x_out, (int)a.ldx, 1, 0, a.M, a.N, a.K);
    po.R = a.R; po.ldr = (int)a.ldr;
    rc = linear(po, st);
    if (rc == BSRL_OK) rc = layernorm(a.x_out, a.ldx, identity_map(), a.gamma, a.beta, a.eps, a.M, a.N, a.h, a.ldh, st);
  }
  g_stage = keep;
  return rc;
}

int fused_attn(const AttnBlockArgs& a, cudaStream_t st) {
  int keep = g_stage;
  g_stage = kStAttnBlock;
  const int tokens = a.body ? a.tokens : kT;
  const double rows = (double)a.n_envs * tokens;
  double fl = 2.0 * rows * 3.0 * a.d * a.d + 4.0 * a.n_envs * a.n_q * tokens * a.d;
  double by = rows * a.d * 2 + (double)a.n_envs * a.n_q * a.d * 2 + (double)a.n_envs * tokens * 4;
  int rc = timed(st, fl, by, [&] { return attn_block(a, st); });
  g_stage = keep;
  return rc;
}

// obs -> x (B*29, d) f32 + key bias; with h_out (and the fused encoder kernel) also block 0's LayerNorm rows.
// Returns through *have_h whether h_out was written.
int run_embed(const Ctx& c, const void* obs, int obs_dtype, float* x, float* key_bias, __half* h_out,
              bool* have_h) {
  const Layout& l = c.l;
  const Workspace& w = c.w;
  const int d = l.d;
  const int64_t B = c.B;
  EmbedBuffers eb;
  // one (29 B, 64) feature matrix: saber | torso | leg | note rows (kept for the backward in a grad-mode forward)
  eb.saber = c.train ? c.train->feat : at<__half>(c.ws, w.f_saber);
  eb.torso = eb.saber + 2 * B * 64;
  eb.leg = eb.torso + B * 64;
  eb.note = eb.leg + 2 * B * 64;
  eb.key_bias = key_bias;
  eb.obs16 = c.obs16;
  eb.ks = kSaberK; eb.kt = kTorsoK; eb.kl = kLegK; eb.kn = l.note_k;
  g_stage = kStGather;
  BSRL_TRY(timed(c.st, 0.0, (double)B * (kObs * 4 + (2 * kSaberK + kTorsoK + 2 * kLegK + kSlots * l.note_k) * 2 + kT * 4),
                 [&] { return embed_gather(obs, obs_dtype, B, c.cfg->note_geo, c.cfg->game_flux, c.cfg->z_asinh, eb, c.st); }));
  if (have_h) *have_h = false;
  if (c.paths.enc_fused) {
    EncoderArgs ea;
    ea.d = d; ea.n_envs = B; ea.feat = eb.saber;
    const Encoder* encs[4] = {&l.saber, &l.torso, &l.leg, &l.note};
    const int kpad[4] = {kSaberK, kTorsoK, kLegK, l.note_k};
    for (int e = 0; e < 4; ++e) {
      ea.w0[e] = c.W(encs[e]->l0); ea.b0[e] = c.Bv(encs[e]->l0); ea.k0[e] = kpad[e];
      ea.w1[e] = c.W(encs[e]->l1); ea.b1[e] = c.Bv(encs[e]->l1);
    }
    const BlockW& b0 = l.blocks[0];
    ea.ln_g = c.G(b0.ln_attn); ea.ln_b = c.Be(b0.ln_attn); ea.eps = c.cfg->eps;
    ea.x = x; ea.h = h_out;
    g_stage = kStEncoderFused;
    const double rows = (double)B * kT;
    BSRL_TRY(timed(c.st, 2.0 * rows * d * (64 + d), rows * (128 + 4.0 * d + (h_out ? 2.0 * d : 0.0)),
                   [&] { return encoder_fused(ea, c.st); }));
    if (have_h) *have_h = h_out != nullptr;
    return BSRL_OK;
  }
  g_stage = kStEncoder;
  __half* hid = at<__half>(c.ws, w.enc_hid);
  struct Part { const Encoder* e; const __half* f; int kpad; int64_t rows; int64_t row0; int group; int first; };
  const Part parts[4] = {
      {&l.saber, eb.saber, kSaberK, 2 * B, 0, 2, 0},
      {&l.torso, eb.torso, kTorsoK, B, 2 * B, 1, 2},
      {&l.leg, eb.leg, kLegK, 2 * B, 3 * B, 2, 3},
      {&l.note, eb.note, l.note_k, (int64_t)kSlots * B, 5 * B, kSlots, kLead},
  };
  for (const Part& p : parts) {
    __half* hp = hid + p.row0 * d;
    LinearArgs a0 = linear_args(p.f, p.kpad, c.W(p.e->l0), p.e->l0.pitch, c.Bv(p.e->l0), hp, d, 0, 1,
                                p.rows, d, p.kpad);
    BSRL_TRY(linear(a0, c.st));
    LinearArgs a1 = linear_args(hp, d, c.W(p.e->l1), p.e->l1.pitch, c.Bv(p.e->l1), x, d, 1, 0, p.rows, d, d);
    a1.cmap = RowMap{p.group, kT, p.first};
    BSRL_TRY(linear(a1, c.st));
  }
  if (c.cfg->emb_ln) {   // tokens = emb_ln(tokens), in place on the fp32 stream (python/policy.py:1261-1262)
    g_stage = kStLayerNorm;
    BSRL_TRY(timed(c.st, 0.0, (double)B * kT * d * 8, [&] {
      return layernorm_rows_f32(x, d, c.G(l.emb_ln), c.Be(l.emb_ln), c.cfg->eps, B * kT, d, x, d, c.st);
    }));
  }
  return BSRL_OK;
}

// head sizes, packed-column offsets and value bins of the configuration
void head_shape(const bsrl_config& cfg, const Layout& l, HeadTailArgs& t) {
  t.bins = l.bins; t.vmax = cfg.value_vmax; t.k_max = l.k_max;
  for (int j = 0; j < kActHeads; ++j) {
    t.gears[j] = cfg.head_gears[j];
    t.first[j] = l.head_first[j];
  }
}

// readout (B, 5d) f16 -> SimBa / SimBaV2 trunk -> h (f16, in z[:, d:]) -> packed head outputs raw (B, head_cols_pad) f32
// (NotePolicy._trunk + the packed head GEMM, python/policy.py:1107-1155, :1311-1335)
int run_trunk(const Ctx& c, const __half* lead16, float* raw) {
  const Layout& l = c.l;
  const Workspace& w = c.w;
  const int d = l.d, D = l.D;
  const int64_t B = c.B;
  const float eps = c.cfg->eps;
  const RowMap ident = identity_map();
  float* xt = at<float>(c.ws, w.xt);
  __half* u = at<__half>(c.ws, w.u);
  __half* r = at<__half>(c.ws, w.r);
  __half* z = at<__half>(c.ws, w.z);
  const int ldz = d + D;
  g_stage = kStTrunk;
  BSRL_TRY(linear(linear_args(lead16, kLead * d, c.W(l.trunk_proj), kLead * d, c.Bv(l.trunk_proj), xt, D, 1, 0, B, D, kLead * d), c.st));
  if (l.trunk_v2) {
    // SimBaV2 (python/policy.py:1140-1155): x = l2n(s_in W_in z); y = l2n(W2 relu(s_1 W1 x));
    // x = l2n(x + alpha (y - x)); h = sqrt(D) x.  GEMMs on fp16 operands, everything else fp32.
    float* t32 = at<float>(c.ws, w.t32);
    BSRL_TRY(simba2_rows(0, xt, xt, at<float>(c.arena, l.v2_s_in), 0.f, B, D, u, D, c.st));
    BSRL_TRY(linear(linear_args(u, D, c.W(l.trunk_fc1), D, c.Bv(l.trunk_fc1), t32, l.Hh, 1, 0, B, l.Hh, D), c.st));
    BSRL_TRY(scale_relu_rows(t32, at<float>(c.arena, l.v2_s_1), B, l.Hh, r, c.st));
    BSRL_TRY(linear(linear_args(r, l.Hh, c.W(l.trunk_fc2), l.Hh, c.Bv(l.trunk_fc2), t32, D, 1, 0, B, D, l.Hh), c.st));
    BSRL_TRY(simba2_rows(1, t32, xt, at<float>(c.arena, l.v2_alpha), 0.5f * sqrtf((float)D), B, D, z + d, ldz, c.st));
  } else {
    BSRL_TRY(layernorm(xt, D, ident, c.G(l.trunk_ln1), c.Be(l.trunk_ln1), eps, B, D, u, D, c.st));
    BSRL_TRY(linear(linear_args(u, D, c.W(l.trunk_fc1), D, c.Bv(l.trunk_fc1), r, l.Hh, 0, 1, B, l.Hh, D), c.st));
    LinearArgs p2 = linear_args(r, l.Hh, c.W(l.trunk_fc2), l.Hh, c.Bv(l.trunk_fc2), xt, D, 1, 0, B, D, l.Hh);
    p2.R = xt; p2.ldr = D;
    BSRL_TRY(linear(p2, c.st));
    BSRL_TRY(layernorm(xt, D, ident, c.G(l.trunk_ln2), c.Be(l.trunk_ln2), eps, B, D, z + d, ldz, c.st));
  }
  return linear(linear_args(z + d, ldz, c.W(l.heads), D, c.Bv(l.heads), raw, l.head_cols_pad, 1, 0, B, l.head_cols_pad, D), c.st);
}

int run_forward(const Ctx& c, const void* obs, int obs_dtype, const HeadTailArgs& tail_in) {
  const Layout& l = c.l;
  const Workspace& w = c.w;
  const int d = l.d, F = l.F, D = l.D;
  const int64_t B = c.B, R = B * kT, Rl = B * kLead;
  const float eps = c.cfg->eps;
  // the residual stream: one buffer updated in place, or -- in a grad-mode forward -- one buffer per
  // block input, so that the backward can recompute every block from what entered it
  float* x = c.train ? c.train->x[0] : at<float>(c.ws, w.x);
  float* key_bias = c.train ? c.train->key_bias : at<float>(c.ws, w.key_bias);
  __half* h = at<__half>(c.ws, w.h);
  __half* qkv = w.qkv >= 0 ? at<__half>(c.ws, w.qkv) : nullptr;   // unfused attention path only
  __half* att = at<__half>(c.ws, w.att);
  __half* hid = w.hid >= 0 ? at<__half>(c.ws, w.hid) : nullptr;   // unfused FFN path only
  const RowMap lead_rows{kLead, kT, 0};
  const RowMap ident = identity_map();

  bool have_h = false, have_hv = false;
  BSRL_TRY(run_embed(c, obs, obs_dtype, x, key_bias, h, &have_h));

  // Fused block tail (out-projection + LayerNorm + FFN in one tcgen05 kernel) where the widths fit;
  // it also emits the next block's LayerNorm rows (and the critic's), so the standalone LayerNorm
  // kernel only runs ahead of block 0.
  auto tail_args = [&](const BlockW& b, int64_t M) {
    BlockTailArgs a;
    memset(&a, 0, sizeof(a));
    a.d = d; a.F = F; a.M = M;
    a.att = att; a.ld_att = d;
    a.x = x; a.ldx = d; a.xmap = ident;
    a.wo = c.W(b.out); a.bo = c.Bv(b.out);
    a.ln_g = c.G(b.ln_ffn); a.ln_b = c.Be(b.ln_ffn);
    a.w0 = c.W(b.up); a.b0 = c.Bv(b.up);
    a.w2 = c.W(b.down); a.b2 = c.Bv(b.down);
    a.eps = eps;
    return a;
  };
  const bool fused = c.paths.tail_fused;
  if (fused && !block_tail_ok(tail_args(l.blocks[0], R))) {
    set_error("forward: the fused block-tail kernel does not take this shape (d=%d, F=%d)", d, F);
    return BSRL_ERR_UNSUPPORTED;
  }
  // Fused q|k|v projection + attention where head_dim is 32 (weights regrouped per head pair).
  auto attn_args = [&](const __half* rows, const Mat& wg, int q_first, int n_q, __half* out) {
    AttnBlockArgs a;
    a.d = d; a.n_heads = l.H; a.n_envs = B;
    a.h = rows; a.ldh = d;
    a.wg = c.W(wg); a.bg = c.Bv(wg);
    a.key_bias = key_bias; a.q_first = q_first; a.n_q = n_q;
    a.out = out; a.ldo = d;
    return a;
  };
  const bool fused_qkv = c.paths.attn_fused;
  if (fused_qkv && !attn_block_ok(attn_args(h, l.blocks[0].qkv_g, 0, kT, att))) {
    set_error("forward: the fused attention kernel does not take this shape (d=%d, heads=%d)", d, l.H);
    return BSRL_ERR_UNSUPPORTED;
  }
  __half* hv = at<__half>(c.ws, w.enc_hid);   // critic LayerNorm rows (encoder scratch is free by now)
  // value residual (python/policy.py:1263-1275): block 0 hands its attention values to every later block
  __half* v0buf = l.value_residual ? at<__half>(c.ws, w.v0) : nullptr;
  auto vres_fused = [&](AttnBlockArgs a, int i) {
    if (v0buf && i == 0) a.v_out = v0buf;
    if (v0buf && i > 0) { a.v0 = v0buf; a.vres = at<float>(c.arena, l.blocks[i].vres); }
    return a;
  };
  auto vres_unfused = [&](int i) -> int {     // on the packed q|k|v buffer, between projection and attention
    if (!v0buf) return BSRL_OK;
    return vres_mix(qkv + 2 * d, 3 * d, R, d, i == 0 ? v0buf : nullptr, i > 0 ? v0buf : nullptr,
                    i > 0 ? at<float>(c.arena, l.blocks[i].vres) : nullptr, c.st);
  };

  for (int i = 0; i + 1 < l.L; ++i) {
    const BlockW& b = l.blocks[i];
    float* x_next = c.train ? c.train->x[i + 1] : x;
    if (!have_h) BSRL_TRY(layernorm(x, d, ident, c.G(b.ln_attn), c.Be(b.ln_attn), eps, R, d, h, d, c.st));
    if (fused_qkv) {
      BSRL_TRY(fused_attn(vres_fused(attn_args(h, b.qkv_g, 0, kT, att), i), c.st));
    } else {
      g_stage = kStQkv;
      BSRL_TRY(linear(linear_args(h, d, c.W(b.qkv), d, c.Bv(b.qkv), qkv, 3 * d, 0, 0, R, 3 * d, d), c.st));
      BSRL_TRY(vres_unfused(i));
      BSRL_TRY(attention(qkv, 3 * d, key_bias, B, d, l.H, 0, kT, att, d, c.st));
    }
    if (fused) {
      const BlockW& nb = l.blocks[i + 1];
      BlockTailArgs a = tail_args(b, R);
      a.x_out = x_next;
      a.out16[0] = h; a.ld16[0] = d; a.g16[0] = c.G(nb.ln_attn); a.b16[0] = c.Be(nb.ln_attn);
      if (i + 2 == l.L) {
        a.out16[1] = hv; a.ld16[1] = d; a.g16[1] = c.G(l.critic_ln); a.b16[1] = c.Be(l.critic_ln);
        have_hv = true;
      }
      BSRL_TRY(fused_tail(a, c.st));
      have_h = true;
      x = x_next;
      continue;
    }
    {
      LinearLnArgs po{att, d, c.W(b.out), d, c.Bv(b.out), x, d, x_next, d, c.G(b.ln_ffn), c.Be(b.ln_ffn), eps, h, d, R, d, d};
      BSRL_TRY(out_proj_ln(po, c.st));
    }
    x = x_next;
    g_stage = kStFfnUp;
    BSRL_TRY(linear(linear_args(h, d, c.W(b.up), d, c.Bv(b.up), hid, F, 0, 1, R, F, d), c.st));
    LinearArgs pd = linear_args(hid, F, c.W(b.down), F, c.Bv(b.down), x, d, 1, 0, R, d, F);
    pd.R = x; pd.ldr = d;
    g_stage = kStFfnDown;
    BSRL_TRY(linear(pd, c.st));
  }

  // final block: keys/values over all 29 rows, everything else on the 5 lead rows
  float* x_lead = at<float>(c.ws, w.x_lead);
  __half* h_lead = at<__half>(c.ws, w.h_lead);
  __half* lead16 = c.train ? c.train->lead16 : at<__half>(c.ws, w.lead16);
  {
    const BlockW& b = l.blocks[l.L - 1];
    if (!have_h) BSRL_TRY(layernorm(x, d, ident, c.G(b.ln_attn), c.Be(b.ln_attn), eps, R, d, h, d, c.st));
    if (fused_qkv) {
      // q is projected for all 29 rows (a third of this kernel's MMAs, no extra HBM traffic);
      // only the 5 lead rows are attended and written
      BSRL_TRY(fused_attn(vres_fused(attn_args(h, b.qkv_g, 0, kLead, att), l.L - 1), c.st));
    } else {
      g_stage = kStQkv;
      BSRL_TRY(linear(linear_args(h, d, c.W(b.qkv, d), d, c.Bv(b.qkv, d), qkv + d, 3 * d, 0, 0, R, 2 * d, d), c.st));
      LinearArgs pq = linear_args(h, d, c.W(b.qkv), d, c.Bv(b.qkv), qkv, 3 * d, 0, 0, Rl, d, d);
      pq.amap = lead_rows;
      pq.cmap = lead_rows;
      BSRL_TRY(linear(pq, c.st));
      BSRL_TRY(vres_unfused(l.L - 1));
      BSRL_TRY(attention(qkv, 3 * d, key_bias, B, d, l.H, 0, kLead, att, d, c.st));
    }
    if (fused) {
      BlockTailArgs a = tail_args(b, Rl);
      a.xmap = lead_rows;
      a.out16[0] = lead16; a.ld16[0] = d;     // plain fp16 rows: the trunk's GEMM operand
      if (c.cfg->final_ln) {                  // ... or final_ln of them (python/policy.py:1306-1307)
        a.g16[0] = c.G(l.final_ln); a.b16[0] = c.Be(l.final_ln);
      }
      BSRL_TRY(fused_tail(a, c.st));
    } else {
      LinearArgs po = linear_args(att, d, c.W(b.out), d, c.Bv(b.out), x_lead, d, 1, 0, Rl, d, d);
      po.R = x; po.ldr = d; po.rmap = lead_rows;
      g_stage = kStOutProj;
      BSRL_TRY(linear(po, c.st));
      BSRL_TRY(layernorm(x_lead, d, ident, c.G(b.ln_ffn), c.Be(b.ln_ffn), eps, Rl, d, h_lead, d, c.st));
      g_stage = kStFfnUp;
      BSRL_TRY(linear(linear_args(h_lead, d, c.W(b.up), d, c.Bv(b.up), hid, F, 0, 1, Rl, F, d), c.st));
      LinearArgs pd = linear_args(hid, F, c.W(b.down), F, c.Bv(b.down), lead16, d, 0, 0, Rl, d, F);
      pd.R = x_lead; pd.ldr = d;
      if (c.cfg->final_ln) {   // keep the fp32 rows and normalise them into the trunk operand
        pd.C = x_lead; pd.ldc = d; pd.out_f32 = 1;
      }
      g_stage = kStFfnDown;
      BSRL_TRY(linear(pd, c.st));
      if (c.cfg->final_ln)
        BSRL_TRY(layernorm(x_lead, d, ident, c.G(l.final_ln), c.Be(l.final_ln), eps, Rl, d, lead16, d, c.st));
    }
  }

  // SimBa trunk on the (B, 5d) readout; its output h lands in z[:, d:]; then the packed heads
  __half* z = at<__half>(c.ws, w.z);
  const int ldz = d + D;
  float* raw = c.train ? c.train->raw : at<float>(c.ws, w.raw);
  BSRL_TRY(run_trunk(c, lead16, raw));

  // adapool critic over the resolved stream entering the final block (still in x)
  __half* att_c = at<__half>(c.ws, w.att_c);
  __half* m1 = at<__half>(c.ws, w.m1);
  __half* m2 = at<__half>(c.ws, w.m2);
  float* vraw = c.train ? c.train->vraw : at<float>(c.ws, w.vraw);
  {
    const RowMap torso_rows{1, kT, 2};
    g_stage = kStCritic;
    const __half* hc = have_hv ? hv : h;
    if (!have_hv) BSRL_TRY(layernorm(x, d, ident, c.G(l.critic_ln), c.Be(l.critic_ln), eps, R, d, h, d, c.st));
    if (fused_qkv) {
      BSRL_TRY(fused_attn(attn_args(hc, l.critic_qkv_g, 2, 1, att_c), c.st));
    } else {
      BSRL_TRY(linear(linear_args(hc, d, c.W(l.critic_kv), d, c.Bv(l.critic_kv), qkv + d, 3 * d, 0, 0, R, 2 * d, d), c.st));
      LinearArgs pq = linear_args(hc, d, c.W(l.critic_q), d, c.Bv(l.critic_q), qkv, 3 * d, 0, 0, B, d, d);
      pq.amap = torso_rows;
      pq.cmap = torso_rows;
      BSRL_TRY(linear(pq, c.st));
      BSRL_TRY(attention(qkv, 3 * d, key_bias, B, d, l.H, 2, 1, att_c, d, c.st));
    }
    BSRL_TRY(linear(linear_args(att_c, d, c.W(l.critic_out), d, c.Bv(l.critic_out), z, ldz, 0, 0, B, d, d), c.st));
    BSRL_TRY(linear(linear_args(z, ldz, c.W(l.critic_m0), ldz, c.Bv(l.critic_m0), m1, D, 0, 1, B, D, ldz), c.st));
    BSRL_TRY(linear(linear_args(m1, D, c.W(l.critic_m1), D, c.Bv(l.critic_m1), m2, D, 0, 1, B, D, D), c.st));
    BSRL_TRY(linear(linear_args(m2, D, c.W(l.critic_m2), D, c.Bv(l.critic_m2), vraw, l.bins_pad, 1, 0, B, l.bins_pad, D), c.st));
  }

  HeadTailArgs t = tail_in;
  t.raw = raw; t.ld_raw = l.head_cols_pad;
  t.vraw = vraw; t.ld_v = l.bins_pad;
  head_shape(*c.cfg, l, t);
  t.n_envs = B;
  g_stage = kStHeadTail;
  return timed(c.st, 0.0, (double)B * 4 * (l.head_cols_pad + l.bins_pad + kActHeads * l.k_max + 1),
               [&] { return head_tail(t, c.st); });
}

int make_ctx(Ctx& c, const bsrl_config* cfg, const void* arena, int64_t n_envs, void* ws,
             int64_t ws_bytes, void* stream) {
  BSRL_TRY(validate_config(cfg));
  if (!arena || !ws) {
    set_error("forward: NULL arena or workspace");
    return BSRL_ERR_NULL;
  }
  if (n_envs < 0 || n_envs > (int64_t)1 << 26) {
    set_error("forward: n_envs %lld out of range", (long long)n_envs);
    return BSRL_ERR_SHAPE;
  }
  if ((reinterpret_cast<uintptr_t>(arena) & 255) || (reinterpret_cast<uintptr_t>(ws) & 255)) {
    set_error("forward: arena and workspace must be 256-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  c.cfg = cfg;
  c.l = make_layout(*cfg);
  use_process_engine();
  c.paths = plan_paths(c.l, g_call_engine);
  c.w = make_workspace(c.l, n_envs, c.paths);
  if (ws_bytes < c.w.bytes) {
    set_error("forward: workspace %lld bytes < required %lld", (long long)ws_bytes, (long long)c.w.bytes);
    return BSRL_ERR_WORKSPACE;
  }
  c.arena = arena;
  c.ws = ws;
  c.B = n_envs;
  c.st = as_stream(stream);
  return BSRL_OK;
}

}  // namespace fwd
}  // namespace bsrl

using namespace bsrl;
using namespace bsrl::fwd;

extern "C" {

int bsrl_abi_version(void) { return BSRL_ABI_VERSION; }
const char* bsrl_last_error(void) { return bsrl::last_error(); }
int bsrl_config_validate(const bsrl_config* cfg) { return validate_config(cfg); }

int64_t bsrl_mac_per_env(const bsrl_config* cfg) {
  if (validate_config(cfg) != BSRL_OK) return -1;
  Layout l = make_layout(*cfg);
  const int64_t d = l.d, T = kT, ld = kLead, D = l.D, Hh = l.Hh, f = cfg->ffn_mult;
  int64_t enc = d * (kSlots * l.note_in + 2 * (kSaberFeat + 2) + kTorsoFeat + 2 * (kLegFeat + 2)) + T * d * d;
  int64_t blk = (4 + 2 * f) * T * d * d + 2 * T * T * d;
  int64_t last = 2 * T * d * d + (2 + 2 * f) * ld * d * d + 2 * ld * T * d;
  int64_t tr = ld * d * D + 2 * D * Hh;
  int64_t heads = D * l.n_head_cols;
  int64_t cr = 2 * T * d * d + 2 * d * d + 2 * T * d + (d + D) * D + D * D + l.bins * D;
  return enc + (l.L - 1) * blk + last + tr + heads + cr;
}

int32_t bsrl_param_count(const bsrl_config* cfg) {
  if (validate_config(cfg) != BSRL_OK) return -1;
  Layout l = make_layout(*cfg);
  return (int32_t)make_param_slots(*cfg, l).size();
}

int bsrl_param_desc(const bsrl_config* cfg, int32_t i, char* name, int32_t name_cap, int64_t* rows,
                    int64_t* cols) {
  BSRL_TRY(validate_config(cfg));
  Layout l = make_layout(*cfg);
  std::vector<ParamSlot> s = make_param_slots(*cfg, l);
  if (i < 0 || i >= (int32_t)s.size()) {
    set_error("param_desc: index %d out of range [0, %d)", i, (int)s.size());
    return BSRL_ERR_SHAPE;
  }
  if (name && name_cap > 0) {
    strncpy(name, s[i].name.c_str(), name_cap - 1);
    name[name_cap - 1] = 0;
  }
  if (rows) *rows = s[i].rows;
  if (cols) *cols = s[i].cols;
  return BSRL_OK;
}

int64_t bsrl_weights_bytes(const bsrl_config* cfg) {
  if (validate_config(cfg) != BSRL_OK) return -1;
  return make_layout(*cfg).bytes;
}

int bsrl_pack_weights(const bsrl_config* cfg, const float* const* params, int32_t n_params, void* arena,
                      int64_t arena_bytes, void* stream) {
  BSRL_TRY(validate_config(cfg));
  Layout l = make_layout(*cfg);
  std::vector<ParamSlot> s = make_param_slots(*cfg, l);
  if (!params || !arena) {
    set_error("pack_weights: NULL argument");
    return BSRL_ERR_NULL;
  }
  if (n_params != (int32_t)s.size()) {
    set_error("pack_weights: %d parameters given, %d expected", n_params, (int)s.size());
    return BSRL_ERR_SHAPE;
  }
  if (arena_bytes < l.bytes) {
    set_error("pack_weights: arena %lld bytes < required %lld", (long long)arena_bytes, (long long)l.bytes);
    return BSRL_ERR_WORKSPACE;
  }
  if (reinterpret_cast<uintptr_t>(arena) & 255) {
    set_error("pack_weights: arena must be 256-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  for (int32_t i = 0; i < n_params; ++i)
    if (!params[i]) {
      set_error("pack_weights: parameter %d (%s) is NULL", i, s[i].name.c_str());
      return BSRL_ERR_NULL;
    }
  cudaStream_t st = as_stream(stream);
  // padding columns / rows of the stacked matrices must read as zero
  BSRL_CUDA_OK(cudaMemsetAsync(arena, 0, l.bytes, st));
  return multi_pack(*cfg, l, const_cast<float* const*>(params), nullptr, nullptr, nullptr, nullptr, nullptr, 0.f, 0.f,
                    0.f, 0, nullptr, nullptr, arena, st);
}

int bsrl_adam_step_pack(const bsrl_config* cfg, float* const* params, const float* const* grads,
                        float* const* exp_avg, float* const* exp_avg_sq, int32_t n_params, const float* lr,
                        const float* weight_decay, float beta1, float beta2, float eps, int32_t step,
                        const float* inv_scale, const float* found_inf, void* arena, int64_t arena_bytes,
                        void* stream) {
  BSRL_TRY(validate_config(cfg));
  Layout l = make_layout(*cfg);
  const int32_t want = (int32_t)make_param_slots(*cfg, l).size();
  if (!params || !grads || !exp_avg || !exp_avg_sq || !lr || !arena) {
    set_error("adam_step_pack: NULL argument");
    return BSRL_ERR_NULL;
  }
  if (n_params != want) {
    set_error("adam_step_pack: %d parameters given, %d expected", n_params, want);
    return BSRL_ERR_SHAPE;
  }
  if (arena_bytes < l.bytes) {
    set_error("adam_step_pack: arena %lld bytes < required %lld", (long long)arena_bytes, (long long)l.bytes);
    return BSRL_ERR_WORKSPACE;
  }
  if (reinterpret_cast<uintptr_t>(arena) & 255) {
    set_error("adam_step_pack: arena must be 256-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  if (step < 1 || !(beta1 >= 0.f && beta1 < 1.f) || !(beta2 >= 0.f && beta2 < 1.f) || !(eps > 0.f)) {
    set_error("adam_step_pack: step must be >= 1, betas in [0, 1), eps > 0");
    return BSRL_ERR_SHAPE;
  }
  for (int32_t i = 0; i < n_params; ++i)
    if (!params[i]) {
      set_error("adam_step_pack: parameter %d is NULL", i);
      return BSRL_ERR_NULL;
    }
  return multi_pack(*cfg, l, params, grads, exp_avg, exp_avg_sq, lr, weight_decay, beta1, beta2, eps, step, inv_scale,
                    found_inf, arena, as_stream(stream));
}

int bsrl_apply_updates_pack(const bsrl_config* cfg, float* const* params, const float* const* updates, int32_t n_params,
                            const float* found_inf, void* arena, int64_t arena_bytes, void* stream) {
  BSRL_TRY(validate_config(cfg));
  Layout l = make_layout(*cfg);
  const int32_t want = (int32_t)make_param_slots(*cfg, l).size();
  if (!params || !updates || !arena) {
    set_error("apply_updates_pack: NULL argument");
    return BSRL_ERR_NULL;
  }
  if (n_params != want) {
    set_error("apply_updates_pack: %d parameters given, %d expected", n_params, want);
    return BSRL_ERR_SHAPE;
  }
  if (arena_bytes < l.bytes || (reinterpret_cast<uintptr_t>(arena) & 255)) {
    set_error("apply_updates_pack: arena too small (%lld < %lld) or not 256-byte aligned", (long long)arena_bytes, (long long)l.bytes);
    return BSRL_ERR_WORKSPACE;
  }
  for (int32_t i = 0; i < n_params; ++i)
    if (!params[i]) {
      set_error("apply_updates_pack: parameter %d is NULL", i);
      return BSRL_ERR_NULL;
    }
  // step 0 + gradients given = additive mode of the pack kernel
  return multi_pack(*cfg, l, params, updates, nullptr, nullptr, nullptr, nullptr, 0.f, 0.f, 1.f, 0, nullptr, found_inf, arena,
                    as_stream(stream));
}

int64_t bsrl_workspace_bytes(const bsrl_config* cfg, int64_t n_envs) {
  if (validate_config(cfg) != BSRL_OK) return -1;
  if (n_envs < 0) return -1;
  Layout l = make_layout(*cfg);
  return make_workspace(l, n_envs, plan_paths(l, g_engine.load(std::memory_order_relaxed))).bytes;
}

int bsrl_forward(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                 int64_t n_envs, float* logits, float* value, float* value_logits, void* workspace,
                 int64_t workspace_bytes, void* stream) {
  Ctx c;
  BSRL_TRY(make_ctx(c, cfg, arena, n_envs, workspace, workspace_bytes, stream));
  if (!obs || !logits || !value) {
    set_error("forward: NULL obs / logits / value");
    return BSRL_ERR_NULL;
  }
  if (n_envs == 0) return BSRL_OK;
  HeadTailArgs t;
  memset(&t, 0, sizeof(t));
  t.logits = logits;
  t.value = value;
  t.value_logits = value_logits;
  return run_forward(c, obs, obs_dtype, t);
}

int bsrl_forward_act(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                     int64_t n_envs, const void* actions, int32_t act_dtype, float* logits,
                     float* logprob, float* entropy, float* ent_head, float* value, float* value_logits,
                     void* workspace, int64_t workspace_bytes, void* stream) {
  Ctx c;
  BSRL_TRY(make_ctx(c, cfg, arena, n_envs, workspace, workspace_bytes, stream));
  if (!obs || !actions || !logprob || !value) {
    set_error("forward_act: NULL obs / actions / logprob / value");
    return BSRL_ERR_NULL;
  }
  if (act_dtype != BSRL_U8 && act_dtype != BSRL_I32 && act_dtype != BSRL_I64) {
    set_error("forward_act: actions must be u8, i32 or i64");
    return BSRL_ERR_UNSUPPORTED;
  }
  if (n_envs == 0) return BSRL_OK;
  HeadTailArgs t;
  memset(&t, 0, sizeof(t));
  t.actions = actions;
  t.act_dtype = act_dtype;
  t.logits = logits;
  t.logprob = logprob;
  t.entropy = entropy;
  t.ent_head = ent_head;
  t.value = value;
  t.value_logits = value_logits;
  return run_forward(c, obs, obs_dtype, t);
}

int bsrl_forward_sample(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                        int64_t n_envs, const uint64_t* rng_state, int64_t* action_out, float* logits,
                        float* logprob, float* entropy, float* ent_head, float* value, void* workspace,
                        int64_t workspace_bytes, void* stream) {
  Ctx c;
  BSRL_TRY(make_ctx(c, cfg, arena, n_envs, workspace, workspace_bytes, stream));
  if (!obs || !rng_state || !action_out || !logprob || !value) {
    set_error("forward_sample: NULL obs / rng_state / action_out / logprob / value");
    return BSRL_ERR_NULL;
  }
  if (n_envs == 0) return BSRL_OK;
  HeadTailArgs t;
  memset(&t, 0, sizeof(t));
  t.rng = reinterpret_cast<const unsigned long long*>(rng_state);
  t.action_out = reinterpret_cast<long long*>(action_out);
  t.logits = logits;
  t.logprob = logprob;
  t.entropy = entropy;
  t.ent_head = ent_head;
  t.value = value;
  return run_forward(c, obs, obs_dtype, t);
}

int bsrl_forward_rollout(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                         int64_t n_envs, const uint64_t* rng_state, int64_t* action_out, uint8_t* act_u8,
                         float* logprob, float* entropy, float* ent_head, float* value, float* value_buf,
                         const float* ret_sigma, const float* ret_mu, void* obs16, void* workspace,
                         int64_t workspace_bytes, void* stream) {
  Ctx c;
  BSRL_TRY(make_ctx(c, cfg, arena, n_envs, workspace, workspace_bytes, stream));
  if (!obs || !rng_state || !logprob || !value || (!action_out && !act_u8)) {
    set_error("forward_rollout: NULL obs / rng_state / logprob / value, or no action output");
    return BSRL_ERR_NULL;
  }
  if (obs16 && (reinterpret_cast<uintptr_t>(obs16) & 3)) {
    set_error("forward_rollout: obs16 must be 4-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  if (n_envs == 0) return BSRL_OK;
  c.obs16 = static_cast<__half*>(obs16);
  HeadTailArgs t;
  memset(&t, 0, sizeof(t));
  t.rng = reinterpret_cast<const unsigned long long*>(rng_state);
  t.action_out = reinterpret_cast<long long*>(action_out);
  t.action_u8 = act_u8;
  t.logprob = logprob;
  t.entropy = entropy;
  t.ent_head = ent_head;
  t.value = value;
  t.value_buf = value_buf;
  t.ret_sigma = ret_sigma;
  t.ret_mu = ret_mu;
  return run_forward(c, obs, obs_dtype, t);
}

int32_t bsrl_token_lane(int32_t tok, int32_t k) { return token_lane_host(tok, k); }

// ---- forward on the library's own fixed scratch (no caller workspace, nothing allocated) ----
// The scratch is a file-scope device array, so every GPU that loads the library holds these
// 32 MiB until the process exits.  g_fixed_scratch names the array for DEVICE code only; on the
// host the same name is just a handle, so the real device address is looked up once per device
// with cudaGetSymbolAddress and that pointer is what the kernels get.
#define BSRL_FIXED_SCRATCH_BYTES (32ll << 20)
static __device__ __align__(256) unsigned char g_fixed_scratch[BSRL_FIXED_SCRATCH_BYTES];

static int fixed_scratch_ptr(void** out) {
  static DeviceOnce once;
  static void* cached[kMaxDevices] = {};
  BSRL_TRY(once.run("forward_fixed: scratch address", [] {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_fixed_scratch);   // address on the CURRENT device
    if (e == cudaSuccess) cached[dev] = ptr;
    return e;
  }));
  int dev = 0;
  BSRL_CUDA_OK(cudaGetDevice(&dev));
  *out = cached[dev];
  return BSRL_OK;
}

int64_t bsrl_fixed_scratch_bytes(void) { return BSRL_FIXED_SCRATCH_BYTES; }

int bsrl_forward_fixed(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
                       int64_t n_envs, float* logits, float* value, void* stream) {
  BSRL_TRY(validate_config(cfg));
  if (n_envs < 0) {
    set_error("forward_fixed: n_envs %lld is negative", (long long)n_envs);
    return BSRL_ERR_SHAPE;
  }
  const int64_t need = bsrl_workspace_bytes(cfg, n_envs);
  if (need > BSRL_FIXED_SCRATCH_BYTES) {
    set_error("forward_fixed: %lld envs need %lld bytes of scratch, the built-in scratch holds %lld; "
              "use bsrl_forward with a caller workspace for larger batches",
              (long long)n_envs, (long long)need, (long long)BSRL_FIXED_SCRATCH_BYTES);
    return BSRL_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  BSRL_TRY(fixed_scratch_ptr(&scratch));
  // Nothing in the scratch has to start at zero: every region a kernel reads was written earlier
  // in the same call, so the previous call's contents are simply overwritten.
  return bsrl_forward(cfg, arena, obs, obs_dtype, n_envs, logits, value, nullptr, scratch,
                      BSRL_FIXED_SCRATCH_BYTES, stream);
}

int bsrl_set_engine(int32_t engine) {
  if (engine < 0 || engine > 1) {
    set_error("set_engine: 0 (automatic) or 1 (warp-MMA only)");
    return BSRL_ERR_UNSUPPORTED;
  }
  g_engine.store(engine, std::memory_order_relaxed);
  return BSRL_OK;
}

int bsrl_device_status(void) {
  int v = device_status_take();
  if (v < 0) {
    set_error("device_status: could not read the status word");
    return BSRL_ERR_CUDA;
  }
  if (v != 0) {
    set_error("a bounded device-side wait ran out (kernel %d, role %d)", v / 16, v % 16);
    return BSRL_ERR_TIMEOUT;
  }
  return BSRL_OK;
}

int bsrl_profile_enable(int32_t on) {
  g_prof.reset();
  g_prof.on = on != 0;
  return BSRL_OK;
}
int32_t bsrl_profile_stage_count(void) { return kStCount; }
const char* bsrl_profile_stage_name(int32_t i) { return (i >= 0 && i < kStCount) ? kStageNames[i] : ""; }
int bsrl_profile_stage(int32_t i, double* ms_total, int64_t* launches, double* flops_total,
                       double* bytes_total) {
  if (i < 0 || i >= kStCount) {
    set_error("profile_stage: index %d out of range", i);
    return BSRL_ERR_SHAPE;
  }
  double ms = 0, fl = 0, by = 0;
  int64_t n = 0;
  for (const Profiler::Rec& r : g_prof.recs) {
    if (r.stage != i) continue;
    float t = 0.f;
    cudaError_t e = cudaEventElapsedTime(&t, r.e0, r.e1);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventElapsedTime (synchronise the stream before reading the profile)");
    ms += t; fl += r.flops; by += r.bytes; ++n;
  }
  if (ms_total) *ms_total = ms;
  if (launches) *launches = n;
  if (flops_total) *flops_total = fl;
  if (bytes_total) *bytes_total = by;
  return BSRL_OK;
}

int bsrl_embed(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype,
               int64_t n_envs, float* x, float* key_bias, void* workspace, int64_t workspace_bytes,
               void* stream) {
  Ctx c;
  BSRL_TRY(make_ctx(c, cfg, arena, n_envs, workspace, workspace_bytes, stream));
  if (!obs || !x || !key_bias) {
    set_error("embed: NULL obs / x / key_bias");
    return BSRL_ERR_NULL;
  }
  if (!aligned16(x)) {
    set_error("embed: x must be 16-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  if (n_envs == 0) return BSRL_OK;
  return run_embed(c, obs, obs_dtype, x, key_bias);
}

int bsrl_trunk_heads(const bsrl_config* cfg, const void* arena, const void* readout_f16, int64_t n_envs,
                     float* head_out, void* trunk_h_f16, void* workspace, int64_t workspace_bytes, void* stream) {
  Ctx c;
  BSRL_TRY(make_ctx(c, cfg, arena, n_envs, workspace, workspace_bytes, stream));
  if (!readout_f16 || !head_out) {
    set_error("trunk_heads: NULL readout / head_out");
    return BSRL_ERR_NULL;
  }
  if (!aligned16(readout_f16) || !aligned16(head_out) || (trunk_h_f16 && !aligned16(trunk_h_f16))) {
    set_error("trunk_heads: readout, head_out and trunk_h must be 16-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  if (n_envs == 0) return BSRL_OK;
  BSRL_TRY(run_trunk(c, static_cast<const __half*>(readout_f16), head_out));
  if (trunk_h_f16) {   // h sits in the workspace as the right-hand columns of the critic MLP's input rows
    const int d = c.l.d, D = c.l.D;
    BSRL_CUDA_OK(cudaMemcpy2DAsync(trunk_h_f16, (size_t)D * 2, at<__half>(c.ws, c.w.z) + d, (size_t)(d + D) * 2,
                                   (size_t)D * 2, (size_t)n_envs, cudaMemcpyDeviceToDevice, c.st));
  }
  return BSRL_OK;
}

int bsrl_head_tail(const bsrl_config* cfg, const float* head_out, const float* value_bin_logits, int64_t n_envs,
                   const void* actions, int32_t act_dtype, float* logits, float* logprob, float* entropy,
                   float* ent_head, float* value, void* stream) {
  BSRL_TRY(validate_config(cfg));
  if (!head_out || !value_bin_logits || !value) {
    set_error("head_tail: NULL head_out / value_bin_logits / value");
    return BSRL_ERR_NULL;
  }
  if (n_envs < 0) {
    set_error("head_tail: n_envs %lld is negative", (long long)n_envs);
    return BSRL_ERR_SHAPE;
  }
  Layout l = make_layout(*cfg);
  HeadTailArgs t;
  memset(&t, 0, sizeof(t));
  t.raw = head_out; t.ld_raw = l.head_cols_pad;
  t.vraw = value_bin_logits; t.ld_v = l.bins_pad;
  head_shape(*cfg, l, t);
  t.actions = actions; t.act_dtype = act_dtype;
  t.logits = logits; t.logprob = logprob; t.entropy = entropy; t.ent_head = ent_head; t.value = value;
  t.n_envs = n_envs;
  return head_tail(t, as_stream(stream));
}

int bsrl_head_layout(const bsrl_config* cfg, int32_t* head_cols_pad, int32_t* bins_pad, int32_t* head_first) {
  BSRL_TRY(validate_config(cfg));
  Layout l = make_layout(*cfg);
  if (head_cols_pad) *head_cols_pad = l.head_cols_pad;
  if (bins_pad) *bins_pad = l.bins_pad;
  if (head_first)
    for (int j = 0; j < kActHeads; ++j) head_first[j] = l.head_first[j];
  return BSRL_OK;
}

int bsrl_workspace_region(const bsrl_config* cfg, int64_t n_envs, const char* name, int64_t* byte_offset,
                          int64_t* rows, int64_t* cols, int64_t* ld_elems, int32_t* dtype) {
  BSRL_TRY(validate_config(cfg));
  if (!name || n_envs < 0) {
    set_error("workspace_region: NULL name or negative n_envs");
    return BSRL_ERR_NULL;
  }
  Layout l = make_layout(*cfg);
  Workspace w = make_workspace(l, n_envs, plan_paths(l, g_engine.load(std::memory_order_relaxed)));
  int64_t off = -1, r = 0, cc = 0, ld = 0;
  int32_t dt = BSRL_F16;
  if (!strcmp(name, "trunk_h")) { off = w.z + (int64_t)l.d * 2; r = n_envs; cc = l.D; ld = l.d + l.D; }
  else if (!strcmp(name, "x_resolved")) { off = w.x; r = n_envs * kT; cc = l.d; ld = l.d; dt = BSRL_F32; }
  else if (!strcmp(name, "key_bias")) { off = w.key_bias; r = n_envs; cc = kT; ld = kT; dt = BSRL_F32; }
  else if (!strcmp(name, "readout")) { off = w.lead16; r = n_envs; cc = kLead * l.d; ld = kLead * l.d; }
  else if (!strcmp(name, "head_out")) { off = w.raw; r = n_envs; cc = l.head_cols_pad; ld = l.head_cols_pad; dt = BSRL_F32; }
  else {
    set_error("workspace_region: unknown region '%s' (trunk_h, x_resolved, key_bias, readout, head_out)", name);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (byte_offset) *byte_offset = off;
  if (rows) *rows = r;
  if (cols) *cols = cc;
  if (ld_elems) *ld_elems = ld;
  if (dtype) *dtype = dt;
  return BSRL_OK;
}

int bsrl_selftest_wait_timeout(int32_t polls, void* stream) {
  if (polls < 1 || polls > (1 << 20)) {
    set_error("selftest_wait_timeout: polls must be in [1, 2^20]");
    return BSRL_ERR_SHAPE;
  }
  return wait_selftest((uint32_t)polls, as_stream(stream));
}

int bsrl_standin_env_step(const int64_t* actions, int64_t n_envs, uint32_t* state, float* obs, float* reward,
                          uint8_t* done, void* stream) {
  return standin_env_step(reinterpret_cast<const long long*>(actions), n_envs, state, obs, reward, done,
                          as_stream(stream));
}

int bsrl_layernorm(const float* x, const float* gamma, const float* beta, float eps, int64_t rows,
                   int32_t d, void* y_f16, int64_t ldy, void* stream) {
  return layernorm_rows(x, d, identity_map(), gamma, beta, eps, rows, d, static_cast<__half*>(y_f16), ldy,
                        as_stream(stream));
}

int bsrl_linear(const void* a_f16, const void* w_f16, const float* bias, const float* residual, void* out,
                int32_t out_f32, int32_t relu, int64_t m, int32_t n, int32_t k, int32_t engine,
                void* stream) {
  LinearArgs p = linear_args(static_cast<const __half*>(a_f16), k, static_cast<const __half*>(w_f16), k, bias,
                             out, n, out_f32, relu, m, n, k);
  p.R = residual;
  p.ldr = n;
  if (engine == 0) return linear_mma(p, as_stream(stream));
  if (engine == 1) {
    if (!linear_tc5_ok(p)) {
      set_error("linear: shape m=%lld n=%d k=%d does not fit the tcgen05 engine", (long long)m, n, k);
      return BSRL_ERR_UNSUPPORTED;
    }
    return linear_tc5(p, as_stream(stream));
  }
  set_error("linear: engine must be 0 (warp-MMA) or 1 (tcgen05)");
  return BSRL_ERR_UNSUPPORTED;
}

int bsrl_block_tail(const void* att_f16, const float* x, const void* wo_f16, const float* bo,
                    const float* ln_g, const float* ln_b, const void* w0_f16, const float* b0,
                    const void* w2_f16, const float* b2, float eps, int64_t m, int32_t d, int32_t f,
                    float* x_out, void* ln_out_f16, const float* out_g, const float* out_b, void* stream) {
  BlockTailArgs a;
  memset(&a, 0, sizeof(a));
  a.d = d; a.F = f; a.M = m;
  a.att = static_cast<const __half*>(att_f16); a.ld_att = d;
  a.x = x; a.ldx = d; a.xmap = identity_map();
  a.wo = static_cast<const __half*>(wo_f16); a.bo = bo; a.ln_g = ln_g; a.ln_b = ln_b;
  a.w0 = static_cast<const __half*>(w0_f16); a.b0 = b0;
  a.w2 = static_cast<const __half*>(w2_f16); a.b2 = b2;
  a.eps = eps;
  a.x_out = x_out;
  a.out16[0] = static_cast<__half*>(ln_out_f16); a.ld16[0] = d; a.g16[0] = out_g; a.b16[0] = out_b;
  return block_tail(a, as_stream(stream));
}

int bsrl_qkv_attention(const void* h_f16, const void* w_grouped_f16, const float* b_grouped,
                       const float* key_bias, int64_t n_envs, int32_t d, int32_t n_heads, int32_t q_first,
                       int32_t n_q, void* out_f16, void* stream) {
  AttnBlockArgs a;
  a.d = d; a.n_heads = n_heads; a.n_envs = n_envs;
  a.h = static_cast<const __half*>(h_f16); a.ldh = d;
  a.wg = static_cast<const __half*>(w_grouped_f16); a.bg = b_grouped;
  a.key_bias = key_bias; a.q_first = q_first; a.n_q = n_q;
  a.out = static_cast<__half*>(out_f16); a.ldo = d;
  return attn_block(a, as_stream(stream));
}

int bsrl_linear_ln(const void* a_f16, const void* w_f16, const float* bias, const float* residual, const float* gamma,
                   const float* beta, float eps, int64_t m, int32_t n, int32_t k, float* x_out, void* h_f16, void* stream) {
  LinearLnArgs a{static_cast<const __half*>(a_f16), k, static_cast<const __half*>(w_f16), k, bias, residual, n, x_out, n,
                 gamma, beta, eps, static_cast<__half*>(h_f16), n, m, n, k};
  return linear_ln(a, as_stream(stream));
}

int bsrl_qkv_attention_body(const void* h_f16, const void* w_grouped_f16, const float* b_grouped, const void* qkv0_f16,
                            const float* key_bias, int64_t n_envs, int32_t d, int32_t n_heads, int32_t n_q, void* out_f16,
                            void* stream) {
  AttnBlockArgs a;
  a.d = d; a.n_heads = n_heads; a.n_envs = n_envs;
  a.h = static_cast<const __half*>(h_f16); a.ldh = d;
  a.wg = static_cast<const __half*>(w_grouped_f16); a.bg = b_grouped;
  a.key_bias = key_bias; a.q_first = 0; a.n_q = n_q;
  a.out = static_cast<__half*>(out_f16); a.ldo = d;
  a.body = 1; a.tokens = 33; a.qkv0 = static_cast<const __half*>(qkv0_f16);
  return attn_block(a, as_stream(stream));
}

int bsrl_attention(const void* qkv_f16, const float* key_bias, int64_t n_envs, int32_t d, int32_t n_heads,
                   int32_t q_first, int32_t n_q, void* out_f16, void* stream) {
  return attention29(static_cast<const __half*>(qkv_f16), 3 * d, key_bias, n_envs, d, n_heads, q_first, n_q,
                     static_cast<__half*>(out_f16), d, as_stream(stream));
}

int bsrl_attention_tokens(const void* qkv_f16, const float* key_bias, int64_t n_envs, int32_t tokens, int32_t d, int32_t n_heads,
                          int32_t q_first, int32_t n_q, void* out_f16, void* stream) {
  return attention_tokens(static_cast<const __half*>(qkv_f16), 3 * d, key_bias, n_envs, tokens, d, n_heads, q_first, n_q,
                          static_cast<__half*>(out_f16), d, as_stream(stream));
}

}  // extern "C"
