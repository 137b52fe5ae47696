// The single-body-token policy ("body + objects" layout): the transformer core of the forward with a
// different front and back end.
//
//   obs (B, body_dim + n_obj * obj_dim + n_obj):  body features | n_obj x obj_dim object features | n_obj live flags
//   tokens: T = 1 + n_obj:  token 0 = Linear(body_dim, d)(body),  token 1 + j = Linear(obj_dim, d)(object j)
//   L pre-LN blocks (python/policy.py:524-715 arithmetic: masked MHA with the additive key bias, FFN with an exact
//   GELU), the last one on the body row only;  readout = the body token
//   heads: Linear(d, 29 K) -> logits (B, 29, K);  value: Linear(d, 1)
//
// This layout is not in the reference (its tokenizer is fixed at 29 tokens with 2-layer ReLU encoders, a
// SimBa trunk and a distributional critic); its blocks are the reference's Block with the FFN activation
// swapped, which is what the parity oracle of this mode composes.  The core kernels are shared with the
// reference layout: the tcgen05 GEMM, the LayerNorm rows, the attention kernel (any token count up to 96), the
// fused block tail (d <= 256, GELU variant) and the head-tail kernel.
#include <string.h>

#include "api_internal.cuh"

namespace bsrl {
namespace {
using namespace fwd;

constexpr int kBodyPadTo = 64;

struct GLayout {
  int d, H, L, F, T, n_obj, K, body_dim, obj_dim, body_k, obj_k, n_cols, cols_pad, obs_dim;
  Mat body, obj, heads;          // heads: rows [0, 29 K) the action heads, row 29 K the value
  std::vector<BlockW> blocks;
  int64_t bytes;
};
struct GWorkspace {
  int64_t key_bias, f_body, f_obj, x, h, qkv, att, hid, x_lead, h_lead, lead16, raw, bytes;
};

struct Carve {
  int64_t off = 0;
  int64_t take(int64_t bytes) {
    const int64_t at = off;
    off += round_up(bytes, 256);
    return at;
  }
};
Mat carve_mat(Carve& c, int rows, int cols, int pitch, int alloc_rows) {
  Mat m;
  m.rows = rows; m.cols = cols; m.pitch = pitch;
  m.w = c.take((int64_t)alloc_rows * pitch * 2);
  m.b = c.take((int64_t)alloc_rows * 4);
  return m;
}
Norm carve_norm(Carve& c, int width) {
  Norm n;
  n.width = width;
  n.g = c.take((int64_t)width * 4);
  n.b = c.take((int64_t)width * 4);
  return n;
}

int validate_g(const bsrl_gconfig* c) {
  if (!c) {
    set_error("gconfig: NULL");
    return BSRL_ERR_NULL;
  }
  if (c->embed < 64 || c->embed > 1024 || c->embed % 64 != 0) {
    set_error("gconfig: embed %d unsupported (multiple of 64 in [64, 1024])", c->embed);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (c->n_heads < 1 || c->embed % c->n_heads != 0 ||
      (c->embed / c->n_heads != 32 && c->embed / c->n_heads != 48 && c->embed / c->n_heads != 64)) {
    set_error("gconfig: head_dim %d unsupported (32, 48 or 64)", c->n_heads > 0 ? c->embed / c->n_heads : 0);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (c->n_blocks < 1 || c->n_blocks > kMaxBlocks || c->ffn_mult < 1 || c->ffn_mult > 8) {
    set_error("gconfig: n_blocks %d / ffn_mult %d out of range", c->n_blocks, c->ffn_mult);
    return BSRL_ERR_SHAPE;
  }
  if (c->n_obj < 1 || c->n_obj > 95) {
    set_error("gconfig: n_obj %d unsupported (1..95: at most 96 tokens)", c->n_obj);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (c->n_gears < 3 || c->n_gears > 7) {
    set_error("gconfig: n_gears %d unsupported (3..7)", c->n_gears);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (c->body_dim < 1 || c->body_dim > 4096 || c->obj_dim < 1 || c->obj_dim > 64) {
    set_error("gconfig: body_dim %d / obj_dim %d out of range", c->body_dim, c->obj_dim);
    return BSRL_ERR_SHAPE;
  }
  if (!(c->eps > 0.f)) {
    set_error("gconfig: eps must be > 0");
    return BSRL_ERR_SHAPE;
  }
  return BSRL_OK;
}

// The fused projection + attention kernel covers 33 tokens (one body token + 32 object tokens = one 32-row tile
// slot per env), head_dim 32 with an even head count, d <= 256.
bool g_attn_shape(const GLayout& l) { return l.T == 33 && l.d <= 256 && l.d % 64 == 0 && l.d / l.H == 32 && l.H % 2 == 0; }

GLayout make_glayout(const bsrl_gconfig& c) {
  GLayout l;
  l.d = c.embed; l.H = c.n_heads; l.L = c.n_blocks; l.F = c.ffn_mult * c.embed;
  l.n_obj = c.n_obj; l.T = 1 + c.n_obj; l.K = c.n_gears;
  l.body_dim = c.body_dim; l.obj_dim = c.obj_dim;
  l.body_k = (int)round_up(c.body_dim, kBodyPadTo);
  l.obj_k = 64;
  l.n_cols = kActHeads * c.n_gears + 1;
  l.cols_pad = (int)round_up(l.n_cols, 16);
  l.obs_dim = c.body_dim + c.n_obj * c.obj_dim + c.n_obj;
  Carve cv;
  const int d = l.d;
  l.body = carve_mat(cv, d, c.body_dim, l.body_k, d);
  l.obj = carve_mat(cv, d, c.obj_dim, l.obj_k, d);
  l.blocks.resize(l.L);
  for (int i = 0; i < l.L; ++i) {
    BlockW& b = l.blocks[i];
    b.ln_attn = carve_norm(cv, d);
    b.qkv = carve_mat(cv, 3 * d, d, d, 3 * d);
    b.out = carve_mat(cv, d, d, d, d);
    b.ln_ffn = carve_norm(cv, d);
    b.up = carve_mat(cv, l.F, d, d, l.F);
    b.down = carve_mat(cv, d, l.F, l.F, d);
    if (g_attn_shape(l)) b.qkv_g = carve_mat(cv, 3 * d, d, d, 3 * d);   // rows regrouped per pair of heads
  }
  l.heads = carve_mat(cv, l.n_cols, d, d, l.cols_pad);
  l.bytes = cv.off;
  return l;
}

std::vector<ParamSlot> g_slots(const GLayout& l) {
  std::vector<ParamSlot> s;
  auto lin = [&](const std::string& name, const Mat& m, int rows, int cols, int row0) {
    s.push_back({name + ".weight", rows, cols, m.w + (int64_t)row0 * m.pitch * 2, m.pitch, true});
    s.push_back({name + ".bias", rows, 1, m.b + (int64_t)row0 * 4, 0, false});
  };
  auto norm = [&](const std::string& name, const Norm& n) {
    s.push_back({name + ".weight", n.width, 1, n.g, 0, false});
    s.push_back({name + ".bias", n.width, 1, n.b, 0, false});
  };
  const int d = l.d;
  lin("body_enc", l.body, d, l.body_dim, 0);
  lin("obj_enc", l.obj, d, l.obj_dim, 0);
  for (int i = 0; i < l.L; ++i) {
    const BlockW& b = l.blocks[i];
    const std::string p = "blocks." + std::to_string(i);
    norm(p + ".ln_attn", b.ln_attn);
    lin(p + ".q_proj", b.qkv, d, d, 0);
    lin(p + ".k_proj", b.qkv, d, d, d);
    lin(p + ".v_proj", b.qkv, d, d, 2 * d);
    lin(p + ".out_proj", b.out, d, d, 0);
    norm(p + ".ln_ffn", b.ln_ffn);
    lin(p + ".ffn.0", b.up, l.F, d, 0);
    lin(p + ".ffn.2", b.down, d, l.F, 0);
  }
  lin("heads", l.heads, kActHeads * l.K, d, 0);
  lin("value", l.heads, 1, d, kActHeads * l.K);
  return s;
}

// second destinations of q / k / v rows: the per-head-pair regrouped copy the fused attention kernel reads
std::vector<CopySlot> g_copy_slots(const GLayout& l, const std::vector<ParamSlot>& params) {
  std::vector<CopySlot> out;
  if (!g_attn_shape(l)) return out;
  auto find = [&](const std::string& name) {
    for (size_t i = 0; i < params.size(); ++i)
      if (params[i].name == name) return (int)i;
    return -1;
  };
  const int d = l.d, gd = 64, n_groups = d / gd;
  for (int i = 0; i < l.L; ++i) {
    const std::string p = "blocks." + std::to_string(i);
    const std::string names[3] = {p + ".q_proj", p + ".k_proj", p + ".v_proj"};
    const Mat& m = l.blocks[i].qkv_g;
    for (int sct = 0; sct < 3; ++sct) {
      const int pw = find(names[sct] + ".weight"), pb = find(names[sct] + ".bias");
      for (int g = 0; g < n_groups; ++g) {
        const int64_t row = (int64_t)g * 3 * gd + sct * gd;
        out.push_back({pw, (int64_t)g * gd, gd, d, m.w + row * m.pitch * 2, m.pitch, true});
        out.push_back({pb, (int64_t)g * gd, gd, 1, m.b + row * 4, 0, false});
      }
    }
  }
  return out;
}

GWorkspace make_gws(const GLayout& l, int64_t B, bool tail_fused, bool attn_fused) {
  GWorkspace w;
  Carve cv;
  const int64_t R = B * l.T;
  const int d = l.d;
  w.key_bias = cv.take(R * 4);
  w.f_body = cv.take(B * (int64_t)l.body_k * 2);
  w.f_obj = cv.take(B * (int64_t)l.n_obj * l.obj_k * 2);
  w.x = cv.take(R * d * 4);
  w.h = cv.take(R * d * 2);
  w.qkv = cv.take((attn_fused ? B : R) * 3 * d * 2);    // fused attention: only the body rows' projection
  w.att = cv.take(R * d * 2);
  w.hid = tail_fused ? -1 : cv.take(R * (int64_t)l.F * 2);
  w.x_lead = cv.take(B * d * 4);
  w.h_lead = cv.take(B * d * 2);
  w.lead16 = cv.take(B * d * 2);
  w.raw = cv.take(B * (int64_t)l.cols_pad * 4);
  w.bytes = cv.off;
  return w;
}

bool g_attn_fused(const GLayout& l, int engine) { return engine == 0 && g_attn_shape(l); }
bool g_tail_fused(const GLayout& l, int engine) {
  return engine == 0 && l.d % 64 == 0 && l.d <= 256 && l.F % 256 == 0 && l.F >= 256 && l.F <= 1024;
}

// One warp per env: body lanes -> K-padded fp16 row, each object's lanes -> its 64-wide row, key bias
// (token 0 always attendable, object j by its live flag: 0 or -16384, python/policy.py:422-428)
__global__ void __launch_bounds__(256) embed_g_kernel(const float* __restrict__ obs, int64_t n_envs, int obs_dim, int body_dim,
                                                      int body_k, int n_obj, int obj_dim, __half* __restrict__ f_body,
                                                      __half* __restrict__ f_obj, float* __restrict__ key_bias) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int T = 1 + n_obj;
  for (int64_t env = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); env < n_envs; env += warps) {
    const float* o = obs + env * obs_dim;
    for (int c = lane; c < body_k; c += 32) f_body[env * body_k + c] = __float2half_rn(c < body_dim ? o[c] : 0.f);
    const float* ob = o + body_dim;
    for (int i = lane; i < n_obj * 64; i += 32) {
      const int j = i >> 6, c = i & 63;
      f_obj[(env * n_obj + j) * 64 + c] = __float2half_rn(c < obj_dim ? ob[j * obj_dim + c] : 0.f);
    }
    const float* live = ob + n_obj * obj_dim;
    for (int t = lane; t < T; t += 32) key_bias[env * T + t] = t == 0 ? 0.f : (live[t - 1] - 1.f) * kMaskBias;
  }
}

struct GCtx {
  const bsrl_gconfig* cfg;
  GLayout l;
  GWorkspace w;
  const void* arena;
  void* ws;
  int64_t B;
  bool fused, attn_fused;
  cudaStream_t st;
  const __half* W(const Mat& m, int row0 = 0) const { return at<__half>(arena, m.w) + (int64_t)row0 * m.pitch; }
  const float* Bv(const Mat& m, int row0 = 0) const { return at<float>(arena, m.b) + row0; }
  const float* G(const Norm& n) const { return at<float>(arena, n.g); }
  const float* Be(const Norm& n) const { return at<float>(arena, n.b); }
};

int g_forward(const GCtx& c, const float* obs, const HeadTailArgs& tail_in) {
  const GLayout& l = c.l;
  const GWorkspace& w = c.w;
  const int d = l.d, F = l.F, T = l.T;
  const int64_t B = c.B, R = B * T;
  const float eps = c.cfg->eps;
  cudaStream_t st = c.st;
  float* x = at<float>(c.ws, w.x);
  float* key_bias = at<float>(c.ws, w.key_bias);
  __half* h = at<__half>(c.ws, w.h);
  __half* qkv = at<__half>(c.ws, w.qkv);
  __half* att = at<__half>(c.ws, w.att);
  __half* hid = w.hid >= 0 ? at<__half>(c.ws, w.hid) : nullptr;
  __half* f_body = at<__half>(c.ws, w.f_body);
  __half* f_obj = at<__half>(c.ws, w.f_obj);
  const RowMap ident = identity_map(), body_rows{1, T, 0}, obj_rows{l.n_obj, T, 1};

  set_stage(kStGather);
  BSRL_TRY(timed_call(st, 0.0, (double)B * (l.obs_dim * 4 + (l.body_k + l.n_obj * l.obj_k) * 2 + T * 4), [&]() -> int {
    int64_t blocks = (B + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    embed_g_kernel<<<(unsigned)blocks, 256, 0, st>>>(obs, B, l.obs_dim, l.body_dim, l.body_k, l.n_obj, l.obj_dim, f_body, f_obj,
                                                     key_bias);
    BSRL_LAUNCH_OK("embed_g_kernel");
    return BSRL_OK;
  }));
  set_stage(kStEncoder);
  {
    LinearArgs a = linear_args(f_body, l.body_k, c.W(l.body), l.body.pitch, c.Bv(l.body), x, d, 1, 0, B, d, l.body_k);
    a.cmap = body_rows;
    BSRL_TRY(linear(a, st));
    LinearArgs o = linear_args(f_obj, l.obj_k, c.W(l.obj), l.obj.pitch, c.Bv(l.obj), x, d, 1, 0, B * l.n_obj, d, l.obj_k);
    o.cmap = obj_rows;
    BSRL_TRY(linear(o, st));
  }
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
    a.gelu = 1;
    return a;
  };
  // q|k|v projection + attention of block b for n_q = T (all rows) or 1 (the body row) query rows per env
  auto project_attend = [&](const BlockW& b, int n_q) -> int {
    // the body rows' own projection (B x 3d), then one kernel for the object rows' projection and all the attention
    set_stage(kStQkv);
    // (the body rows of h are every T-th row: a dense matrix of pitch T d)
    BSRL_TRY(linear(linear_args(h, T * d, c.W(b.qkv), d, c.Bv(b.qkv), qkv, 3 * d, 0, 0, B, 3 * d, d), st));
    AttnBlockArgs a;
    a.d = d; a.n_heads = l.H; a.n_envs = B;
    a.h = h; a.ldh = d;
    a.wg = c.W(b.qkv_g); a.bg = c.Bv(b.qkv_g);
    a.key_bias = key_bias; a.q_first = 0; a.n_q = n_q;
    a.out = att; a.ldo = d;
    a.body = 1; a.tokens = T; a.qkv0 = qkv;
    return fused_attn(a, st);
  };
  auto attend = [&](int n_q) -> int {        // masked attention of n_q query rows per env over its T tokens
    set_stage(kStAttention);
    return timed_call(st, 4.0 * B * n_q * T * d, (double)B * (T * 2 * d + n_q * d * 2) * 2 + (double)B * T * 4,
                      [&]() -> int { return attention_tokens(qkv, 3 * d, key_bias, B, T, d, l.H, 0, n_q, att, d, st); });
  };
  bool have_h = false;
  for (int i = 0; i + 1 < l.L; ++i) {
    const BlockW& b = l.blocks[i];
    if (!have_h) BSRL_TRY(layernorm(x, d, ident, c.G(b.ln_attn), c.Be(b.ln_attn), eps, R, d, h, d, st));
    if (c.attn_fused) {
      BSRL_TRY(project_attend(b, T));
    } else {
      set_stage(kStQkv);
      BSRL_TRY(linear(linear_args(h, d, c.W(b.qkv), d, c.Bv(b.qkv), qkv, 3 * d, 0, 0, R, 3 * d, d), st));
      BSRL_TRY(attend(T));
    }
    if (c.fused) {
      BlockTailArgs a = tail_args(b, R);
      a.x_out = x;
      const BlockW& nb = l.blocks[i + 1];
      a.out16[0] = h; a.ld16[0] = d; a.g16[0] = c.G(nb.ln_attn); a.b16[0] = c.Be(nb.ln_attn);
      BSRL_TRY(fused_tail(a, st));
      have_h = true;
      continue;
    }
    {
      LinearLnArgs po{att, d, c.W(b.out), d, c.Bv(b.out), x, d, x, d, c.G(b.ln_ffn), c.Be(b.ln_ffn), eps, h, d, R, d, d};
      BSRL_TRY(out_proj_ln(po, st));
    }
    set_stage(kStFfnUp);
    BSRL_TRY(linear(linear_args(h, d, c.W(b.up), d, c.Bv(b.up), hid, F, 0, 2, R, F, d), st));
    set_stage(kStFfnDown);
    LinearArgs pd = linear_args(hid, F, c.W(b.down), F, c.Bv(b.down), x, d, 1, 0, R, d, F);
    pd.R = x; pd.ldr = d;
    BSRL_TRY(linear(pd, st));
  }
  // last block: keys / values over all tokens, everything else on the body row
  float* x_lead = at<float>(c.ws, w.x_lead);
  __half* h_lead = at<__half>(c.ws, w.h_lead);
  __half* lead16 = at<__half>(c.ws, w.lead16);
  {
    const BlockW& b = l.blocks[l.L - 1];
    if (!have_h) BSRL_TRY(layernorm(x, d, ident, c.G(b.ln_attn), c.Be(b.ln_attn), eps, R, d, h, d, st));
    if (c.attn_fused) {
      BSRL_TRY(project_attend(b, 1));
    } else {
      set_stage(kStQkv);
      BSRL_TRY(linear(linear_args(h, d, c.W(b.qkv, d), d, c.Bv(b.qkv, d), qkv + d, 3 * d, 0, 0, R, 2 * d, d), st));
      LinearArgs pq = linear_args(h, d, c.W(b.qkv), d, c.Bv(b.qkv), qkv, 3 * d, 0, 0, B, d, d);
      pq.amap = body_rows; pq.cmap = body_rows;
      BSRL_TRY(linear(pq, st));
      BSRL_TRY(attend(1));
    }
    if (c.fused) {
      BlockTailArgs a = tail_args(b, B);
      a.xmap = body_rows;
      a.out16[0] = lead16; a.ld16[0] = d;
      BSRL_TRY(fused_tail(a, st));
    } else {
      set_stage(kStOutProj);
      LinearArgs po = linear_args(att, d, c.W(b.out), d, c.Bv(b.out), x_lead, d, 1, 0, B, d, d);
      po.R = x; po.ldr = d; po.rmap = body_rows;
      BSRL_TRY(linear(po, st));
      BSRL_TRY(layernorm(x_lead, d, ident, c.G(b.ln_ffn), c.Be(b.ln_ffn), eps, B, d, h_lead, d, st));
      BSRL_TRY(linear(linear_args(h_lead, d, c.W(b.up), d, c.Bv(b.up), hid, F, 0, 2, B, F, d), st));
      LinearArgs pd = linear_args(hid, F, c.W(b.down), F, c.Bv(b.down), lead16, d, 0, 0, B, d, F);
      pd.R = x_lead; pd.ldr = d;
      BSRL_TRY(linear(pd, st));
    }
  }
  float* raw = at<float>(c.ws, w.raw);
  set_stage(kStTrunk);
  BSRL_TRY(linear(linear_args(lead16, d, c.W(l.heads), d, c.Bv(l.heads), raw, l.cols_pad, 1, 0, B, l.cols_pad, d), st));
  HeadTailArgs t = tail_in;
  t.raw = raw; t.ld_raw = l.cols_pad;
  t.vraw = raw + kActHeads * l.K; t.ld_v = l.cols_pad;      // the value is the last packed column: one "bin"
  t.bins = 1; t.vmax = 1.f; t.k_max = l.K;
  for (int j = 0; j < kActHeads; ++j) {
    t.gears[j] = l.K;
    t.first[j] = j * l.K;
  }
  t.n_envs = B;
  set_stage(kStHeadTail);
  return timed_call(st, 0.0, (double)B * (l.cols_pad * 4 + 64), [&]() -> int { return head_tail(t, st); });
}

int make_gctx(GCtx& c, const bsrl_gconfig* cfg, const void* arena, int64_t n_envs, void* ws, int64_t ws_bytes, void* stream) {
  BSRL_TRY(validate_g(cfg));
  if (!arena || !ws) {
    set_error("g_forward: NULL arena or workspace");
    return BSRL_ERR_NULL;
  }
  if (n_envs < 0 || n_envs > (int64_t)1 << 26) {
    set_error("g_forward: n_envs %lld out of range", (long long)n_envs);
    return BSRL_ERR_SHAPE;
  }
  if ((reinterpret_cast<uintptr_t>(arena) & 255) || (reinterpret_cast<uintptr_t>(ws) & 255)) {
    set_error("g_forward: arena and workspace must be 256-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  use_process_engine();
  c.cfg = cfg;
  c.l = make_glayout(*cfg);
  c.fused = g_tail_fused(c.l, process_engine());
  c.attn_fused = g_attn_fused(c.l, process_engine());
  c.w = make_gws(c.l, n_envs, c.fused, c.attn_fused);
  if (ws_bytes < c.w.bytes) {
    set_error("g_forward: workspace %lld bytes < required %lld", (long long)ws_bytes, (long long)c.w.bytes);
    return BSRL_ERR_WORKSPACE;
  }
  c.arena = arena; c.ws = ws; c.B = n_envs; c.st = as_stream(stream);
  return BSRL_OK;
}

}  // namespace
}  // namespace bsrl

using namespace bsrl;
using namespace bsrl::fwd;

extern "C" {

int bsrl_g_config_validate(const bsrl_gconfig* cfg) { return validate_g(cfg); }

int32_t bsrl_g_obs_dim(const bsrl_gconfig* cfg) {
  if (validate_g(cfg) != BSRL_OK) return -1;
  return make_glayout(*cfg).obs_dim;
}

int64_t bsrl_g_mac_per_env(const bsrl_gconfig* cfg) {
  if (validate_g(cfg) != BSRL_OK) return -1;
  const GLayout l = make_glayout(*cfg);
  const int64_t d = l.d, T = l.T, f = cfg->ffn_mult;
  const int64_t enc = (int64_t)l.body_dim * d + (int64_t)l.n_obj * l.obj_dim * d;
  const int64_t blk = (4 + 2 * f) * T * d * d + 2 * T * T * d;
  const int64_t last = 2 * T * d * d + (2 + 2 * f) * d * d + 2 * T * d;
  return enc + (l.L - 1) * blk + last + d * l.n_cols;
}

int32_t bsrl_g_param_count(const bsrl_gconfig* cfg) {
  if (validate_g(cfg) != BSRL_OK) return -1;
  return (int32_t)g_slots(make_glayout(*cfg)).size();
}

int bsrl_g_param_desc(const bsrl_gconfig* cfg, int32_t i, char* name, int32_t name_cap, int64_t* rows, int64_t* cols) {
  BSRL_TRY(validate_g(cfg));
  const std::vector<ParamSlot> s = g_slots(make_glayout(*cfg));
  if (i < 0 || i >= (int32_t)s.size()) {
    set_error("g_param_desc: index %d out of range [0, %d)", i, (int)s.size());
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

int64_t bsrl_g_weights_bytes(const bsrl_gconfig* cfg) {
  if (validate_g(cfg) != BSRL_OK) return -1;
  return make_glayout(*cfg).bytes;
}

int bsrl_g_pack_weights(const bsrl_gconfig* cfg, const float* const* params, int32_t n_params, void* arena,
                        int64_t arena_bytes, void* stream) {
  BSRL_TRY(validate_g(cfg));
  const GLayout l = make_glayout(*cfg);
  const std::vector<ParamSlot> s = g_slots(l);
  if (!params || !arena) {
    set_error("g_pack_weights: NULL argument");
    return BSRL_ERR_NULL;
  }
  if (n_params != (int32_t)s.size()) {
    set_error("g_pack_weights: %d parameters given, %d expected", n_params, (int)s.size());
    return BSRL_ERR_SHAPE;
  }
  if (arena_bytes < l.bytes || (reinterpret_cast<uintptr_t>(arena) & 255)) {
    set_error("g_pack_weights: arena too small (%lld < %lld) or not 256-byte aligned", (long long)arena_bytes, (long long)l.bytes);
    return BSRL_ERR_WORKSPACE;
  }
  for (int32_t i = 0; i < n_params; ++i)
    if (!params[i]) {
      set_error("g_pack_weights: parameter %d (%s) is NULL", i, s[i].name.c_str());
      return BSRL_ERR_NULL;
    }
  cudaStream_t st = as_stream(stream);
  BSRL_CUDA_OK(cudaMemsetAsync(arena, 0, l.bytes, st));
  return multi_pack_slots(s, g_copy_slots(l, s), const_cast<float* const*>(params), nullptr, nullptr, nullptr, nullptr, nullptr, 0.f, 0.f, 0.f, 0,
                          nullptr, nullptr, arena, st);
}

int64_t bsrl_g_workspace_bytes(const bsrl_gconfig* cfg, int64_t n_envs) {
  if (validate_g(cfg) != BSRL_OK || n_envs < 0) return -1;
  const GLayout l = make_glayout(*cfg);
  return make_gws(l, n_envs, g_tail_fused(l, process_engine()), g_attn_fused(l, process_engine())).bytes;
}

int bsrl_g_forward(const bsrl_gconfig* cfg, const void* arena, const float* obs, int64_t n_envs, const void* actions,
                   int32_t act_dtype, float* logits, float* logprob, float* entropy, float* ent_head, float* value,
                   void* workspace, int64_t workspace_bytes, void* stream) {
  GCtx c;
  BSRL_TRY(make_gctx(c, cfg, arena, n_envs, workspace, workspace_bytes, stream));
  if (!obs || !value || (!logits && !logprob)) {
    set_error("g_forward: NULL obs / value, or neither logits nor logprob asked for");
    return BSRL_ERR_NULL;
  }
  if ((logprob || entropy || ent_head) && !actions && logprob) {
    set_error("g_forward: logprob needs the actions");
    return BSRL_ERR_NULL;
  }
  if (actions && act_dtype != BSRL_U8 && act_dtype != BSRL_I32 && act_dtype != BSRL_I64) {
    set_error("g_forward: actions must be u8, i32 or i64");
    return BSRL_ERR_UNSUPPORTED;
  }
  if (n_envs == 0) return BSRL_OK;
  HeadTailArgs t;
  memset(&t, 0, sizeof(t));
  t.actions = actions; t.act_dtype = act_dtype;
  t.logits = logits; t.logprob = logprob; t.entropy = entropy; t.ent_head = ent_head; t.value = value;
  return g_forward(c, obs, t);
}

}  // extern "C"
