// Configuration checks, arena / workspace layout and the weight packer.
#include "layout.h"

#include <stdarg.h>
#include <string.h>

#include <atomic>

#include "kernels.cuh"

namespace bsrl {

// ------------------------------------------------------------------ errors, device info
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_err; }

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
  return BSRL_ERR_CUDA;
}

int sm_count() {
  static std::atomic<int> cached[kMaxDevices];     // 0 = not read yet; racing first readers store the same value
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

LinearArgs linear_args(const __half* A, int lda, const __half* W, int ldw, const float* bias,
                       void* C, int ldc, int out_f32, int relu, int64_t M, int N, int K) {
  LinearArgs p;
  p.A = A; p.lda = lda; p.amap = identity_map();
  p.W = W; p.ldw = ldw; p.bias = bias;
  p.R = nullptr; p.ldr = 0; p.rmap = identity_map();
  p.C = C; p.ldc = ldc; p.cmap = identity_map();
  p.out_f32 = out_f32; p.relu = relu;
  p.M = M; p.N = N; p.K = K;
  return p;
}

// ------------------------------------------------------------------ configuration
int validate_config(const bsrl_config* c) {
  if (!c) {
    set_error("config: NULL");
    return BSRL_ERR_NULL;
  }
  if (c->embed < 32 || c->embed > 1024 || c->embed % 32 != 0) {
    set_error("config: embed %d unsupported (multiple of 32 in [32, 1024])", c->embed);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (c->n_heads < 1 || c->embed % c->n_heads != 0) {
    set_error("config: embed %d not divisible by %d heads", c->embed, c->n_heads);
    return BSRL_ERR_SHAPE;
  }
  const int dh = c->embed / c->n_heads;
  if (dh != 32 && dh != 48 && dh != 64) {
    set_error("config: head_dim %d unsupported (32, 48 or 64)", dh);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (c->n_blocks < 1 || c->n_blocks > 64 || c->ffn_mult < 1 || c->ffn_mult > 8) {
    set_error("config: n_blocks %d / ffn_mult %d out of range", c->n_blocks, c->ffn_mult);
    return BSRL_ERR_SHAPE;
  }
  if (c->trunk_dim < 32 || c->trunk_dim > 1024 || c->trunk_dim % 32 != 0 || c->trunk_hidden < 32 ||
      c->trunk_hidden > 4096 || c->trunk_hidden % 32 != 0) {
    set_error("config: trunk_dim %d / trunk_hidden %d unsupported (multiples of 32, trunk_dim <= 1024)",
              c->trunk_dim, c->trunk_hidden);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (c->value_bins < 2 || c->value_bins > 1024) {
    set_error("config: value_bins must be in [2, 1024], got %d", c->value_bins);
    return BSRL_ERR_SHAPE;
  }
  for (int j = 0; j < kActHeads; ++j)
    if (c->head_gears[j] < 3 || c->head_gears[j] > 7) {
      set_error("config: head_gears must be %d counts in [3, 7], got %d at head %d", kActHeads,
                c->head_gears[j], j);
      return BSRL_ERR_SHAPE;
    }
  if (!(c->z_asinh > 0.f)) {
    set_error("config: z_asinh must be > 0 (metres), got %g", c->z_asinh);
    return BSRL_ERR_SHAPE;
  }
  if ((c->emb_ln | c->final_ln | c->game_flux | c->value_residual | c->trunk_v2) & ~1) {
    set_error("config: emb_ln / final_ln / game_flux / value_residual / trunk_v2 must be 0 or 1");
    return BSRL_ERR_SHAPE;
  }
  if (!(c->value_vmax > 0.f) || !(c->eps > 0.f)) {
    set_error("config: value_vmax and eps must be > 0");
    return BSRL_ERR_SHAPE;
  }
  return BSRL_OK;
}

// ------------------------------------------------------------------ arena layout
namespace {
struct Carver {
  int64_t off = 0;
  int64_t take(int64_t bytes) {
    int64_t at = off;
    off += round_up(bytes, 256);
    return at;
  }
};
Mat carve_mat(Carver& c, int rows, int cols, int pitch = 0, int alloc_rows = 0) {
  Mat m;
  m.rows = rows;
  m.cols = cols;
  m.pitch = pitch ? pitch : cols;
  if (alloc_rows < rows) alloc_rows = rows;
  m.w = c.take((int64_t)alloc_rows * m.pitch * 2);
  m.b = c.take((int64_t)alloc_rows * 4);
  return m;
}
Norm carve_norm(Carver& c, int width) {
  Norm n;
  n.width = width;
  n.g = c.take((int64_t)width * 4);
  n.b = c.take((int64_t)width * 4);
  return n;
}
}  // namespace

Layout make_layout(const bsrl_config& c) {
  Layout l;
  l.d = c.embed;
  l.H = c.n_heads;
  l.L = c.n_blocks;
  l.F = c.ffn_mult * c.embed;
  l.D = c.trunk_dim;
  l.Hh = c.trunk_hidden;
  l.bins = c.value_bins;
  l.bins_pad = (int)round_up(c.value_bins, 16);      // multiples of 16: the packed GEMMs stay on the tcgen05 kernel
  l.note_in = kNoteFeat + (c.note_geo ? kGeoFeat : 0);
  l.note_k = note_k(c.note_geo != 0);
  l.k_max = 0;
  l.n_head_cols = 0;
  for (int j = 0; j < kActHeads; ++j) {
    l.head_first[j] = l.n_head_cols;
    l.n_head_cols += c.head_gears[j];
    if (c.head_gears[j] > l.k_max) l.k_max = c.head_gears[j];
  }
  l.head_cols_pad = (int)round_up(l.n_head_cols, 16);
  const int d = l.d;
  Carver cv;
  auto enc = [&](int in, int kpad) {
    Encoder e;
    e.l0 = carve_mat(cv, d, in, kpad);
    e.l1 = carve_mat(cv, d, d);
    return e;
  };
  l.note = enc(l.note_in, l.note_k);
  l.saber = enc(kSaberFeat + 2, kSaberK);
  l.torso = enc(kTorsoFeat, kTorsoK);
  l.leg = enc(kLegFeat + 2, kLegK);
  l.blocks.resize(l.L);
  for (int i = 0; i < l.L; ++i) {
    BlockW& b = l.blocks[i];
    b.ln_attn = carve_norm(cv, d);
    b.qkv = carve_mat(cv, 3 * d, d);
    b.out = carve_mat(cv, d, d);
    b.ln_ffn = carve_norm(cv, d);
    b.up = carve_mat(cv, l.F, d);
    b.down = carve_mat(cv, d, l.F);
    b.qkv_g = carve_mat(cv, 3 * d, d);
    if (c.value_residual && i > 0) b.vres = cv.take(8);
  }
  l.value_residual = c.value_residual;
  l.trunk_proj = carve_mat(cv, l.D, kLead * d);
  l.trunk_ln1 = carve_norm(cv, l.D);
  l.trunk_fc1 = carve_mat(cv, l.Hh, l.D);
  l.trunk_fc2 = carve_mat(cv, l.D, l.Hh);
  l.trunk_ln2 = carve_norm(cv, l.D);
  l.trunk_v2 = c.trunk_v2;
  if (c.trunk_v2) {
    l.v2_s_in = cv.take((int64_t)l.D * 4);
    l.v2_s_1 = cv.take((int64_t)l.Hh * 4);
    l.v2_alpha = cv.take((int64_t)l.D * 4);
  }
  l.heads = carve_mat(cv, l.n_head_cols, l.D, 0, l.head_cols_pad);
  l.critic_ln = carve_norm(cv, d);
  if (c.emb_ln) l.emb_ln = carve_norm(cv, d);
  if (c.final_ln) l.final_ln = carve_norm(cv, d);
  l.critic_q = carve_mat(cv, d, d);
  l.critic_kv = carve_mat(cv, 2 * d, d);
  l.critic_out = carve_mat(cv, d, d);
  l.critic_m0 = carve_mat(cv, l.D, d + l.D);
  l.critic_m1 = carve_mat(cv, l.D, l.D);
  l.critic_m2 = carve_mat(cv, l.bins, l.D, 0, l.bins_pad);
  l.critic_qkv_g = carve_mat(cv, 3 * d, d);
  // fused QKV+attention kernel: head_dim 32, two heads per group (192 output columns per group), or
  // head_dim 48, one head per group (144 columns)
  l.attn_G = 0;
  if (d % 64 == 0 && d % l.H == 0) {
    if (d <= 256 && d / l.H == 32 && l.H % 2 == 0) l.attn_G = 2;
    else if (d <= 256 && d / l.H == 48) l.attn_G = 1;
    else if (d <= 512 && d / l.H == 64) l.attn_G = 1;      // the h tile streams through the ring
  }
  l.bytes = cv.off;
  return l;
}

std::vector<ParamSlot> make_param_slots(const bsrl_config& c, const Layout& l) {
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
  auto enc = [&](const std::string& name, const Encoder& e) {
    lin(name + ".0", e.l0, d, e.l0.cols, 0);
    lin(name + ".2", e.l1, d, d, 0);
  };
  enc("note_mlp", l.note);
  enc("saber_mlp", l.saber);
  enc("torso_mlp", l.torso);
  enc("leg_mlp", l.leg);
  for (int i = 0; i < l.L; ++i) {
    const BlockW& b = l.blocks[i];
    std::string p = "blocks." + std::to_string(i);
    norm(p + ".ln_attn", b.ln_attn);
    lin(p + ".q_proj", b.qkv, d, d, 0);
    lin(p + ".k_proj", b.qkv, d, d, d);
    lin(p + ".v_proj", b.qkv, d, d, 2 * d);
    lin(p + ".out_proj", b.out, d, d, 0);
    norm(p + ".ln_ffn", b.ln_ffn);
    if (b.vres >= 0) {
      s.push_back({p + ".vres_a", 1, 1, b.vres, 0, false});
      s.push_back({p + ".vres_b", 1, 1, b.vres + 4, 0, false});
    }
    lin(p + ".ffn.0", b.up, l.F, d, 0);
    lin(p + ".ffn.2", b.down, d, l.F, 0);
  }
  if (l.trunk_v2) {
    lin("trunk_in", l.trunk_proj, l.D, kLead * d, 0);
    lin("trunk_w1", l.trunk_fc1, l.Hh, l.D, 0);
    lin("trunk_w2", l.trunk_fc2, l.D, l.Hh, 0);
    s.push_back({"trunk_s_in", l.D, 1, l.v2_s_in, 0, false});
    s.push_back({"trunk_s_1", l.Hh, 1, l.v2_s_1, 0, false});
    s.push_back({"trunk_alpha", l.D, 1, l.v2_alpha, 0, false});
  } else {
    lin("trunk_proj", l.trunk_proj, l.D, kLead * d, 0);
    norm("trunk_ln1", l.trunk_ln1);
    lin("trunk_fc1", l.trunk_fc1, l.Hh, l.D, 0);
    lin("trunk_fc2", l.trunk_fc2, l.D, l.Hh, 0);
    norm("trunk_ln2", l.trunk_ln2);
  }
  for (int j = 0; j < kActHeads; ++j)
    lin("heads." + std::to_string(j), l.heads, c.head_gears[j], l.D, l.head_first[j]);
  norm("critic_ln", l.critic_ln);
  if (c.emb_ln) norm("emb_ln", l.emb_ln);
  if (c.final_ln) norm("final_ln", l.final_ln);
  lin("critic_q", l.critic_q, d, d, 0);
  lin("critic_k", l.critic_kv, d, d, 0);
  lin("critic_v", l.critic_kv, d, d, d);
  lin("critic_out", l.critic_out, d, d, 0);
  lin("critic_mlp.0", l.critic_m0, l.D, d + l.D, 0);
  lin("critic_mlp.2", l.critic_m1, l.D, l.D, 0);
  lin("critic_mlp.4", l.critic_m2, l.bins, l.D, 0);
  return s;
}

// Regrouped q|k|v: group g holds [q rows of its heads | k rows | v rows], 3*G*dh rows per group.
std::vector<CopySlot> make_copy_slots(const bsrl_config& c, const Layout& l, const std::vector<ParamSlot>& params) {
  std::vector<CopySlot> out;
  auto find = [&](const std::string& name) {
    for (size_t i = 0; i < params.size(); ++i)
      if (params[i].name == name) return (int)i;
    return -1;
  };
  if (l.attn_G == 0) return out;
  const int d = l.d, gd = l.attn_G * (d / l.H), n_groups = d / gd;
  auto regroup = [&](const Mat& m, const std::string names[3]) {
    for (int sct = 0; sct < 3; ++sct) {
      const int pw = find(names[sct] + ".weight"), pb = find(names[sct] + ".bias");
      for (int g = 0; g < n_groups; ++g) {
        const int64_t row = (int64_t)g * 3 * gd + sct * gd;
        out.push_back({pw, (int64_t)g * gd, gd, d, m.w + row * m.pitch * 2, m.pitch, true});
        out.push_back({pb, (int64_t)g * gd, gd, 1, m.b + row * 4, 0, false});
      }
    }
  };
  for (int i = 0; i < l.L; ++i) {
    const std::string p = "blocks." + std::to_string(i);
    const std::string names[3] = {p + ".q_proj", p + ".k_proj", p + ".v_proj"};
    regroup(l.blocks[i].qkv_g, names);
  }
  const std::string cn[3] = {"critic_q", "critic_k", "critic_v"};
  regroup(l.critic_qkv_g, cn);
  return out;
}

// ------------------------------------------------------------------ workspace
Paths plan_paths(const Layout& l, int engine) {
  Paths p;
  const bool widths = engine == 0 && l.d % 64 == 0 && l.d >= 64 && l.d <= 256;
  p.attn_fused = engine == 0 && l.attn_G > 0;
  p.tail_fused = widths && l.F % 256 == 0 && l.F >= 256 && l.F <= 1024;
  p.enc_fused = widths && !l.emb_ln.width && l.note_k == 64;
  return p;
}

Workspace make_workspace(const Layout& l, int64_t B, const Paths& paths) {
  Workspace w;
  Carver cv;
  const int64_t R = B * kT, Rl = B * kLead;
  const int d = l.d;
  w.key_bias = cv.take(R * 4);
  // encoder input rows, all 64 wide, as ONE (29 B, 64) matrix: saber | torso | leg | note
  static_assert(kSaberK == 64 && kTorsoK == 64 && kLegK == 64, "the feature matrix has one row width");
  w.f_saber = cv.take(B * kT * 64 * 2);
  w.f_torso = w.f_saber + B * 2 * 64 * 2;
  w.f_leg = w.f_torso + B * 64 * 2;
  w.f_note = w.f_leg + B * 2 * 64 * 2;
  w.enc_hid = cv.take(R * d * 2);
  w.x = cv.take(R * d * 4);
  w.h = cv.take(R * d * 2);
  w.qkv = paths.attn_fused ? -1 : cv.take(R * 3 * d * 2);
  w.att = cv.take(R * d * 2);
  w.hid = paths.tail_fused ? -1 : cv.take(R * (int64_t)l.F * 2);
  w.x_lead = cv.take(Rl * d * 4);
  w.h_lead = cv.take(Rl * d * 2);
  w.lead16 = cv.take(Rl * d * 2);
  w.xt = cv.take(B * l.D * 4);
  w.u = cv.take(B * l.D * 2);
  w.r = cv.take(B * l.Hh * 2);
  w.z = cv.take(B * (d + l.D) * 2);
  w.m1 = cv.take(B * l.D * 2);
  w.m2 = cv.take(B * l.D * 2);
  w.raw = cv.take(B * l.head_cols_pad * 4);
  w.vraw = cv.take(B * l.bins_pad * 4);
  w.att_c = cv.take(B * d * 2);
  w.v0 = cv.take(l.value_residual ? R * d * 2 : 0);
  w.t32 = cv.take(l.trunk_v2 ? B * (int64_t)(l.D > l.Hh ? l.D : l.Hh) * 4 : 0);
  w.bytes = cv.off;
  return w;
}

}  // namespace bsrl
