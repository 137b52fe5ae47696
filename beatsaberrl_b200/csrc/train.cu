// Training entry points: the grad-mode forward of the PPO recompute call and its backward.
//
//   bsrl_forward_train  = NotePolicy.get_action_and_value(obs, action) in grad mode
//                         (python/policy.py:1467-1516 over :1198-1403): the SAME kernels as the rollout
//                         forward -- so rollout and recompute log-probs agree bit for bit -- but the
//                         residual stream entering every block, the tokenizer's feature rows, the readout
//                         and the head outputs are kept in a caller-owned save buffer;
//   bsrl_backward       = what autograd does for the reference (python/fp16_linear.py:461-767, :931-1064,
//                         :1197-1251; python/fused_ln.py:58-107): gradients of every parameter from the
//                         upstream gradients of log-prob, entropy, value and value-bin logits.
//
// The backward recomputes each block's intermediates (LayerNorm rows, q|k|v, attention output, hidden) from
// the saved block input with the unfused kernels, then walks the block in reverse.  Every matrix product
// runs on the tcgen05 GEMM: input gradients against a transposed copy of the weight, weight gradients as
// split-K products of the transposed gradient and activation matrices (the reduction runs over token
// rows), bias gradients as column sums.  Activation gradients are fp16 GEMM operands scaled by the
// caller's loss scale; the residual-stream gradient, LayerNorm arithmetic and parameter gradients are fp32.
#include <string.h>

#include <initializer_list>
#include <map>
#include <string>

#include "api_internal.cuh"

namespace bsrl {
int layernorm_bwd(const float* x, int64_t ldx, RowMap xmap, const float* gamma, float eps, const void* gy, int gy_f32,
                  int64_t ldgy, const float* gres, float* gx_out, int64_t ldg, RowMap gmap, float* ggamma, float* gbeta,
                  int64_t rows, int d, cudaStream_t stream, __half* gx16 = nullptr, int64_t ldg16 = 0);
int colsum16(const __half* in, int64_t ld, int64_t rows, int n, float* out, cudaStream_t stream);
int relu_mask16(__half* g, int64_t ldg, const __half* act, int64_t lda, int64_t rows, int n, cudaStream_t stream);
int cast_rows16(const float* in, int64_t ldi, RowMap imap, float scale, __half* out, int64_t ldo, int64_t rows, int n,
                cudaStream_t stream);
int add_rows32(const float* src, int64_t lds, float* dst, int64_t ldd, RowMap dmap, int64_t rows, int n, int accumulate,
               cudaStream_t stream);
int transpose16(const __half* in, int64_t ldi, RowMap imap, int64_t rows, int cols, __half* out, int64_t ldo,
                int64_t rows_pad, cudaStream_t stream, float* colsum = nullptr);
int head_tail_bwd(const HeadTailArgs& a, const float* g_logprob, const float* g_entropy, const float* g_value,
                  const float* g_vlogits, const float* g_logits, float scale, __half* g_raw, int ldg_raw, __half* g_vraw,
                  int ldg_v, cudaStream_t stream);
int attention29_bwd(const __half* qkv, int ld_qkv, const float* key_bias, int64_t n_envs, int d, int n_heads, int q_first,
                    int n_q, const __half* g_out, int ldgo, __half* gq, int ldq, __half* gk, int ldk, __half* gv, int ldv,
                    cudaStream_t stream);

int vres_mix(__half* v, int ld, int64_t rows, int d, __half* v_out, const __half* v0, const float* vres, cudaStream_t stream);
int vres_bwd(__half* g, int64_t ldg, const __half* v_own, const __half* v0, const float* ab, float* g_v0, float* g_a, float* g_b,
             int64_t rows, int d, cudaStream_t stream);
int add_f32_into_f16(__half* g, int64_t ldg, const float* acc, int64_t rows, int d, cudaStream_t stream);
int simba2_rows(int mode, const float* in, float* x, const float* vec, float c_alpha, int64_t rows, int d, __half* out16, int64_t ld16,
                cudaStream_t stream);
int scale_relu_rows(const float* in, const float* s, int64_t rows, int n, __half* out16, cudaStream_t stream);
int simba2_out_bwd(const float* x0, const float* t2, const float* alpha, float c_alpha, const float* g_h, float* g_x0, __half* g_t2,
                   float* g_alpha, int64_t rows, int d, cudaStream_t stream);
int simba2_in_bwd(const float* t0, const float* s, const float* g_a, const float* g_b, __half* g_t0, float* g_s, int64_t rows, int d,
                  cudaStream_t stream);
int scale_relu_bwd(__half* g, const float* t, const float* s, float* g_s, int64_t rows, int n, cudaStream_t stream);

namespace {
using namespace fwd;

struct Carve {
  int64_t off = 0;
  int64_t take(int64_t bytes) {
    const int64_t at = off;
    off += round_up(bytes, 256);
    return at;
  }
};

// ---- what the grad-mode forward keeps
struct SaveLayout {
  int64_t feat, key_bias, x[kMaxBlocks], lead16, raw, vraw, bytes;
};
SaveLayout make_save(const Layout& l, int64_t B) {
  SaveLayout s;
  Carve cv;
  s.feat = cv.take(B * kT * 64 * 2);
  s.key_bias = cv.take(B * kT * 4);
  for (int i = 0; i < l.L; ++i) s.x[i] = cv.take(B * kT * (int64_t)l.d * 4);
  s.lead16 = cv.take(B * kLead * (int64_t)l.d * 2);
  s.raw = cv.take(B * (int64_t)l.head_cols_pad * 4);
  s.vraw = cv.take(B * (int64_t)l.bins_pad * 4);
  s.bytes = cv.off;
  return s;
}
TrainPtrs save_ptrs(const SaveLayout& s, const Layout& l, void* save) {
  TrainPtrs t;
  memset(&t, 0, sizeof(t));
  t.feat = at<__half>(save, s.feat);
  t.key_bias = at<float>(save, s.key_bias);
  for (int i = 0; i < l.L; ++i) t.x[i] = at<float>(save, s.x[i]);
  t.lead16 = at<__half>(save, s.lead16);
  t.raw = at<float>(save, s.raw);
  t.vraw = at<float>(save, s.vraw);
  return t;
}

int train_supported(const bsrl_config* cfg, const Layout& l) {
  if (l.L > kMaxBlocks) {
    set_error("training entry points: at most %d blocks", kMaxBlocks);
    return BSRL_ERR_UNSUPPORTED;
  }
  if (l.d % 64 != 0 || l.D % 64 != 0 || l.Hh % 64 != 0 || l.F % 64 != 0) {
    set_error("training entry points: embed, trunk widths and the FFN hidden must be multiples of 64");
    return BSRL_ERR_UNSUPPORTED;
  }
  return BSRL_OK;
}

inline int64_t pad64(int64_t n) { return round_up(n, 64); }

// ---- scratch of the backward
struct BwdLayout {
  int64_t h16, qkv16, att16, x1, h2, hid, gx, gx16, g32, gA, gB, tA, tX, wT;
  // readout-side rows (B of them)
  int64_t xt, u16, r16, xt2, z16, hv16, attc16, m1, m2, gz32, graw16, gvraw16, gsmall32, gsmall16, scratch_w;
  int64_t bias_scratch, heads_scratch;
  int64_t v0, vown, gv0;        // value residual: block 0's values, a block's own values, fp32 gradient of block 0's values
  int64_t t1_32, t2_32;         // SimBaV2 trunk: fc1 and fc2 outputs (fp32)
  int64_t bytes;
  int64_t Rpad;
  int wmax, ld_graw, ld_gv;
};
BwdLayout make_bwd(const Layout& l, int64_t B) {
  BwdLayout w;
  Carve cv;
  const int64_t R = B * kT;
  const int d = l.d, F = l.F, D = l.D;
  w.Rpad = pad64(R);
  w.ld_graw = (int)pad64(l.head_cols_pad);
  w.ld_gv = (int)pad64(l.bins_pad);
  int wide = F > 3 * d ? F : 3 * d;                    // widest activation-gradient row
  if (D + d > wide) wide = D + d;
  if (kLead * d > wide) wide = kLead * d;
  if (w.ld_graw > wide) wide = w.ld_graw;
  w.h16 = cv.take(R * d * 2);
  w.qkv16 = cv.take(R * 3 * d * 2);
  w.att16 = cv.take(R * d * 2);
  w.x1 = cv.take(R * d * 4);
  w.h2 = cv.take(R * d * 2);
  w.hid = cv.take(R * (int64_t)F * 2);
  w.gx = cv.take(R * d * 4);
  w.gx16 = cv.take(R * d * 2);     // fp16 copy of the stream gradient, written by the LayerNorm backward that produces it
  w.g32 = cv.take(R * d * 4);
  w.gA = cv.take(R * (int64_t)wide * 2);
  w.gB = cv.take(R * 3 * d * 2);
  w.tA = cv.take((int64_t)wide * w.Rpad * 2);
  w.tX = cv.take((int64_t)wide * w.Rpad * 2);
  int64_t wmax = (int64_t)F * d;                       // largest weight, in elements, with its padded row count
  const int64_t cands[] = {(int64_t)3 * d * d, (int64_t)D * kLead * d, (int64_t)D * l.Hh, (int64_t)D * (d + D), (int64_t)D * D,
                           (int64_t)w.ld_graw * D, (int64_t)w.ld_gv * D};
  for (int64_t cnd : cands)
    if (cnd > wmax) wmax = cnd;
  w.wmax = (int)wmax;
  w.wT = cv.take(wmax * 2);
  w.xt = cv.take(B * D * 4);
  w.u16 = cv.take(B * D * 2);
  w.r16 = cv.take(B * (int64_t)l.Hh * 2);
  w.xt2 = cv.take(B * D * 4);
  w.z16 = cv.take(B * (int64_t)(d + D) * 2);
  w.hv16 = cv.take(R * d * 2);
  w.attc16 = cv.take(B * d * 2);
  w.m1 = cv.take(B * D * 2);
  w.m2 = cv.take(B * D * 2);
  w.gz32 = cv.take(B * (int64_t)(d + D) * 4);
  w.graw16 = cv.take(B * (int64_t)w.ld_graw * 2);
  w.gvraw16 = cv.take(B * (int64_t)w.ld_gv * 2);
  w.gsmall32 = cv.take(B * (int64_t)wide * 4);
  w.gsmall16 = cv.take(B * (int64_t)wide * 2);
  w.scratch_w = cv.take((int64_t)d * 64 * 4);
  w.bias_scratch = cv.take((int64_t)wide * 4);
  w.heads_scratch = cv.take((int64_t)l.head_cols_pad * D * 4);
  w.v0 = w.vown = w.gv0 = w.t1_32 = w.t2_32 = -1;
  if (l.value_residual && l.L > 1) {
    w.v0 = cv.take(R * d * 2);
    w.vown = cv.take(R * d * 2);
    w.gv0 = cv.take(R * d * 4);
  }
  if (l.trunk_v2) {
    w.t1_32 = cv.take(B * (int64_t)l.Hh * 4);
    w.t2_32 = cv.take(B * D * 4);
  }
  w.bytes = cv.off;
  return w;
}

struct Bwd {
  const Ctx& c;
  const Layout& l;
  const TrainPtrs& sv;
  const BwdLayout& w;
  void* ws;
  float* grads;                         // flat, parameter-table order
  std::map<std::string, int64_t> goff;  // parameter name -> offset in floats
  float scale;
  cudaStream_t st;
  int64_t B, R, Rl;
  int d, F, D;

  float* G(const std::string& name) const {
    auto it = goff.find(name);
    return it == goff.end() ? nullptr : grads + it->second;
  }
  template <typename T>
  T* S(int64_t off) const { return at<T>(ws, off); }

  // out (M, K) = g (M, N) . W, W = rows [0, N) of a (N, K) fp16 matrix with pitch ldw; g has pad64(N) columns.
  // The contraction runs over W's ROWS: the tensor cores take W as it lies (an MN-major operand); only shapes
  // that mode does not cover go through a transposed copy.
  // With relu_of (the fp16 output of the ReLU this gradient flows back through, same shape as out), entries
  // whose activation was not positive come out as zero.
  int dgrad(const __half* g, int64_t ldg, int64_t M, const __half* W, int ldw, int N, int K, void* out, int64_t ldo, bool out_f32,
            const __half* relu_of = nullptr, int64_t ld_relu = 0) {
    LinearArgs r = linear_args(g, (int)ldg, W, ldw, nullptr, out, (int)ldo, out_f32 ? 1 : 0, 0, M, K, N);
    r.w_mn = 1;
    r.mask = relu_of;
    r.ldm = (int)ld_relu;
    if (linear_rows_ok(r)) return linear(r, st);
    const int Np = (int)pad64(N);
    __half* wT = S<__half>(w.wT);
    BSRL_TRY(transpose16(W, ldw, identity_map(), N, K, wT, Np, Np, st));
    LinearArgs a = linear_args(g, (int)ldg, wT, Np, nullptr, out, (int)ldo, out_f32 ? 1 : 0, 0, M, K, Np);
    BSRL_TRY(linear(a, st));
    if (relu_of) {
      if (out_f32) {
        set_error("backward: the ReLU mask applies to fp16 gradients");
        return BSRL_ERR_UNSUPPORTED;
      }
      return relu_mask16(static_cast<__half*>(out), ldo, relu_of, ld_relu, M, K, st);
    }
    return BSRL_OK;
  }
  // Operands of the weight-gradient products gW = g^T x (the contraction runs over the M token rows).  to_tA /
  // to_tX only NAME the two matrices (and take the bias gradient, the column sums of g); wgrad_t hands them
  // to the tensor cores as they lie (MN-major operands) where the shape allows, and otherwise makes the
  // transposed copies (tA, tX: rows of the matrix become columns, M padded to 64) on first use.
  struct Operand { const __half* m = nullptr; int64_t ld = 0; RowMap map{0x7fffffff, 0, 0}; int64_t M = 0; int n = 0; bool copied = false; };
  Operand opA, opX;
  static bool is_identity(const RowMap& m) { return m.group == 0x7fffffff && m.stride == 0 && m.first == 0; }
  int to_tA(const __half* m, int64_t ld, RowMap map, int64_t M, int N, float* colsum = nullptr) {   // colsum: bias gradient on the way
    opA = Operand{m, ld, map, M, N, false};
    if (colsum && is_identity(map)) return colsum16(m, ld, M, N, colsum, st);
    if (colsum) return copy_tA(colsum);
    return BSRL_OK;
  }
  int copy_tA(float* colsum = nullptr) {
    opA.copied = true;
    return transpose16(opA.m, opA.ld, opA.map, opA.M, opA.n, S<__half>(w.tA), pad64(opA.M), pad64(opA.M), st, colsum);
  }
  // gradient matrix whose column ranges are the bias gradients of several parameters (stacked q|k|v, the packed
  // heads): the sums land in a scratch vector and are copied out slice by slice
  struct BiasSlice { float* dst; int col0, n; };
  int to_tA_slices(const __half* g, int64_t ld, int64_t M, int N, std::initializer_list<BiasSlice> slices) {
    float* scratch = S<float>(w.bias_scratch);
    BSRL_CUDA_OK(cudaMemsetAsync(scratch, 0, (size_t)N * 4, st));
    BSRL_TRY(to_tA(g, ld, identity_map(), M, N, scratch));
    for (const BiasSlice& b : slices)
      if (b.dst) BSRL_CUDA_OK(cudaMemcpyAsync(b.dst, scratch + b.col0, (size_t)b.n * 4, cudaMemcpyDeviceToDevice, st));
    return BSRL_OK;
  }
  int to_tX(const __half* m, int64_t ld, RowMap map, int64_t M, int K) {
    opX = Operand{m, ld, map, M, K, false};
    return BSRL_OK;
  }
  // gW (n, K) f32 (+)= g[:, row0 : row0 + n]^T . x; gW must be zero on entry
  int wgrad_t(int row0, int n, int K, int64_t M, float* gW, int ldgw) {
    if (!gW) return BSRL_OK;
    const int64_t Mp = pad64(M);
    if (Mp > 0x7fffffff) {
      set_error("backward: too many rows for one weight-gradient product");
      return BSRL_ERR_SHAPE;
    }
    int64_t tiles = ((n + 127) / 128) * ((K + 255) / 256);
    int splits = (int)(sm_count() / (tiles > 0 ? tiles : 1));
    if (is_identity(opA.map) && is_identity(opX.map) && !opA.copied && !opX.copied) {
      LinearArgs r = linear_args(opA.m + row0, (int)opA.ld, opX.m, (int)opX.ld, nullptr, gW, ldgw, 1, 0, n, K, (int)M);
      r.a_mn = r.w_mn = 1;
      r.k_splits = splits < 1 ? 1 : splits;
      if (linear_rows_ok(r)) return linear(r, st);
    }
    if (!opA.copied) BSRL_TRY(copy_tA());
    if (!opX.copied) {
      opX.copied = true;
      BSRL_TRY(transpose16(opX.m, opX.ld, opX.map, opX.M, opX.n, S<__half>(w.tX), Mp, Mp, st));
    }
    LinearArgs a = linear_args(S<__half>(w.tA) + (int64_t)row0 * Mp, (int)Mp, S<__half>(w.tX), (int)Mp, nullptr, gW, ldgw, 1, 0, n, K, (int)Mp);
    a.k_splits = splits < 1 ? 1 : splits;
    return linear(a, st);
  }
  // one Linear: gW += g^T x, gb += colsum(g); x through xmap
  int wgrad(const __half* g, int64_t ldg, int64_t M, int N, const __half* x, int64_t ldx, RowMap xmap, int K, const std::string& name) {
    BSRL_TRY(to_tA(g, ldg, identity_map(), M, N, G(name + ".bias")));
    BSRL_TRY(to_tX(x, ldx, xmap, M, K));
    return wgrad_t(0, N, K, M, G(name + ".weight"), K);
  }
  int cast16(const float* in, int64_t ldi, RowMap map, __half* out, int64_t ldo, int64_t rows, int n) {
    return cast_rows16(in, ldi, map, 1.f, out, ldo, rows, n, st);
  }
  int ln_bwd(const float* x, int64_t ldx, RowMap xmap, const Norm& n, const std::string& name, const void* gy, bool gy_f32,
             int64_t ldgy, const float* gres, float* gx_out, int64_t ldg, RowMap gmap, int64_t rows, int width,
             __half* gx16 = nullptr) {
    return layernorm_bwd(x, ldx, xmap, c.G(n), c.cfg->eps, gy, gy_f32 ? 1 : 0, ldgy, gres, gx_out, ldg, gmap, G(name + ".weight"),
                         G(name + ".bias"), rows, width, st, gx16, width);
  }

  // FFN + out-projection half of a block on M rows, given the gradient g_out (fp32) of the block's output:
  // leaves the gradient of x1 (the stream after the attention residual) in g_x1 and the fp16 gradient of the
  // attention output in gatt16.  x1 / h2 / hid / att are the recomputed activations of those M rows.
  // g_out16: the same gradient already as fp16 (M, d) rows, or nullptr.
  int tail_bwd(int i, int64_t M, const float* g_out, float* g_x1, const float* x1, const __half* h2, const __half* hid,
               const __half* att, __half* gatt16, const __half* g_out16 = nullptr) {
    const BlockW& b = l.blocks[i];
    const std::string p = "blocks." + std::to_string(i);
    __half* gA = S<__half>(w.gA);
    __half* gB = S<__half>(w.gB);
    float* g32 = S<float>(w.g32);
    if (!g_out16) {                                                                             // g_out as a GEMM operand
      BSRL_TRY(cast16(g_out, d, identity_map(), gB, d, M, d));
      g_out16 = gB;
    }
    BSRL_TRY(wgrad(g_out16, d, M, d, hid, F, identity_map(), F, p + ".ffn.2"));
    BSRL_TRY(dgrad(g_out16, d, M, c.W(b.down), b.down.pitch, d, F, gA, F, false, hid, F));      // g_hid, through the ReLU
    BSRL_TRY(wgrad(gA, F, M, F, h2, d, identity_map(), d, p + ".ffn.0"));
    BSRL_TRY(dgrad(gA, F, M, c.W(b.up), b.up.pitch, F, d, g32, d, true));                        // g_h2
    BSRL_TRY(ln_bwd(x1, d, identity_map(), b.ln_ffn, p + ".ln_ffn", g32, true, d, g_out, g_x1, d, identity_map(), M, d, gB));
    BSRL_TRY(wgrad(gB, d, M, d, att, d, identity_map(), d, p + ".out_proj"));
    BSRL_TRY(dgrad(gB, d, M, c.W(b.out), b.out.pitch, d, d, gatt16, d, false));
    return BSRL_OK;
  }

  // recompute x1 = x[rows] + att Wo^T + bo, h2 = LN_ffn(x1), hid = relu(h2 W0^T + b0) on M rows
  int tail_fwd(int i, int64_t M, const float* x_in, RowMap xrows, const __half* att, float* x1, __half* h2, __half* hid) {
    const BlockW& b = l.blocks[i];
    LinearArgs po = linear_args(att, d, c.W(b.out), d, c.Bv(b.out), x1, d, 1, 0, M, d, d);
    po.R = x_in; po.ldr = d; po.rmap = xrows;
    BSRL_TRY(linear(po, st));
    BSRL_TRY(layernorm(x1, d, identity_map(), c.G(b.ln_ffn), c.Be(b.ln_ffn), c.cfg->eps, M, d, h2, d, st));
    return linear(linear_args(h2, d, c.W(b.up), d, c.Bv(b.up), hid, F, 0, 1, M, F, d), st);
  }

  int run(const HeadTailArgs& tail, const float* g_logprob, const float* g_entropy, const float* g_value,
          const float* g_vlogits, const float* g_logits) {
    const float eps = c.cfg->eps;
    const RowMap ident = identity_map(), lead_rows{kLead, kT, 0}, torso_rows{1, kT, 2};
    const int ldz = d + D, Hh = l.Hh;
    __half* h16 = S<__half>(w.h16);
    __half* qkv = S<__half>(w.qkv16);
    __half* att = S<__half>(w.att16);
    float* x1 = S<float>(w.x1);
    __half* h2 = S<__half>(w.h2);
    __half* hid = S<__half>(w.hid);
    float* gx = S<float>(w.gx);
    float* g32 = S<float>(w.g32);
    __half* gA = S<__half>(w.gA);
    __half* gB = S<__half>(w.gB);
    float* xt = S<float>(w.xt);
    __half* u16 = S<__half>(w.u16);
    __half* r16 = S<__half>(w.r16);
    float* xt2 = S<float>(w.xt2);
    __half* z16 = S<__half>(w.z16);
    __half* hv = S<__half>(w.hv16);
    __half* attc = S<__half>(w.attc16);
    __half* m1 = S<__half>(w.m1);
    __half* m2 = S<__half>(w.m2);
    float* gz32 = S<float>(w.gz32);
    __half* graw = S<__half>(w.graw16);
    __half* gvraw = S<__half>(w.gvraw16);
    float* gs32 = S<float>(w.gsmall32);
    __half* gs16 = S<__half>(w.gsmall16);
    const float* x_last = sv.x[l.L - 1];            // the stream entering the last block = the critic's input

    // ---- head tail
    BSRL_TRY(head_tail_bwd(tail, g_logprob, g_entropy, g_value, g_vlogits, g_logits, scale, graw, w.ld_graw, gvraw, w.ld_gv, st));

    // ---- recompute the readout side: trunk and critic activations
    BSRL_TRY(linear(linear_args(sv.lead16, kLead * d, c.W(l.trunk_proj), kLead * d, c.Bv(l.trunk_proj), xt, D, 1, 0, B, D, kLead * d), st));
    const float c_alpha = 0.5f * sqrtf((float)D);      // SimBaV2: alpha = trunk_alpha * c_alpha
    float* t1_32 = l.trunk_v2 ? S<float>(w.t1_32) : nullptr;
    float* t2_32 = l.trunk_v2 ? S<float>(w.t2_32) : nullptr;
    if (l.trunk_v2) {
      // xt = t0 = W_in z; xt2 = x0 = l2n(t0 s_in); t1 = W1 x0; r = relu(t1 s_1); t2 = W2 r; h = sqrt(D) l2n(x0 + a (l2n(t2) - x0))
      BSRL_TRY(simba2_rows(0, xt, xt2, at<float>(c.arena, l.v2_s_in), 0.f, B, D, u16, D, st));
      BSRL_TRY(linear(linear_args(u16, D, c.W(l.trunk_fc1), D, c.Bv(l.trunk_fc1), t1_32, Hh, 1, 0, B, Hh, D), st));
      BSRL_TRY(scale_relu_rows(t1_32, at<float>(c.arena, l.v2_s_1), B, Hh, r16, st));
      BSRL_TRY(linear(linear_args(r16, Hh, c.W(l.trunk_fc2), Hh, c.Bv(l.trunk_fc2), t2_32, D, 1, 0, B, D, Hh), st));
      BSRL_TRY(simba2_rows(1, t2_32, xt2, at<float>(c.arena, l.v2_alpha), c_alpha, B, D, z16 + d, ldz, st));
    } else {
      BSRL_TRY(layernorm(xt, D, ident, c.G(l.trunk_ln1), c.Be(l.trunk_ln1), eps, B, D, u16, D, st));
      BSRL_TRY(linear(linear_args(u16, D, c.W(l.trunk_fc1), D, c.Bv(l.trunk_fc1), r16, Hh, 0, 1, B, Hh, D), st));
      LinearArgs p2 = linear_args(r16, Hh, c.W(l.trunk_fc2), Hh, c.Bv(l.trunk_fc2), xt2, D, 1, 0, B, D, Hh);
      p2.R = xt; p2.ldr = D;
      BSRL_TRY(linear(p2, st));
      BSRL_TRY(layernorm(xt2, D, ident, c.G(l.trunk_ln2), c.Be(l.trunk_ln2), eps, B, D, z16 + d, ldz, st));
    }
    BSRL_TRY(layernorm(x_last, d, ident, c.G(l.critic_ln), c.Be(l.critic_ln), eps, R, d, hv, d, st));
    BSRL_TRY(linear(linear_args(hv, d, c.W(l.critic_kv), d, c.Bv(l.critic_kv), qkv + d, 3 * d, 0, 0, R, 2 * d, d), st));
    {
      LinearArgs pq = linear_args(hv, d, c.W(l.critic_q), d, c.Bv(l.critic_q), qkv, 3 * d, 0, 0, B, d, d);
      pq.amap = torso_rows; pq.cmap = torso_rows;
      BSRL_TRY(linear(pq, st));
    }
    BSRL_TRY(attention(qkv, 3 * d, sv.key_bias, B, d, l.H, 2, 1, attc, d, st));
    BSRL_TRY(linear(linear_args(attc, d, c.W(l.critic_out), d, c.Bv(l.critic_out), z16, ldz, 0, 0, B, d, d), st));
    BSRL_TRY(linear(linear_args(z16, ldz, c.W(l.critic_m0), ldz, c.Bv(l.critic_m0), m1, D, 0, 1, B, D, ldz), st));
    BSRL_TRY(linear(linear_args(m1, D, c.W(l.critic_m1), D, c.Bv(l.critic_m1), m2, D, 0, 1, B, D, D), st));

    // ---- critic MLP
    BSRL_TRY(to_tA_slices(gvraw, w.ld_gv, B, l.bins_pad, {{G("critic_mlp.4.bias"), 0, l.bins}}));
    BSRL_TRY(to_tX(m2, D, ident, B, D));
    BSRL_TRY(wgrad_t(0, l.bins, D, B, G("critic_mlp.4.weight"), D));
    BSRL_TRY(dgrad(gvraw, w.ld_gv, B, c.W(l.critic_m2), l.critic_m2.pitch, l.bins, D, gs16, D, false));
    BSRL_TRY(relu_mask16(gs16, D, m2, D, B, D, st));
    BSRL_TRY(wgrad(gs16, D, B, D, m1, D, ident, D, "critic_mlp.2"));
    BSRL_TRY(dgrad(gs16, D, B, c.W(l.critic_m1), l.critic_m1.pitch, D, D, gA, D, false));
    BSRL_TRY(relu_mask16(gA, D, m1, D, B, D, st));
    BSRL_TRY(wgrad(gA, D, B, D, z16, ldz, ident, ldz, "critic_mlp.0"));
    BSRL_TRY(dgrad(gA, D, B, c.W(l.critic_m0), l.critic_m0.pitch, D, ldz, gz32, ldz, true));     // g_z = [g_a | g_h from the critic]
    // critic attention pool
    BSRL_TRY(cast16(gz32, ldz, ident, gs16, d, B, d));                                           // g_a
    BSRL_TRY(wgrad(gs16, d, B, d, attc, d, ident, d, "critic_out"));
    BSRL_TRY(dgrad(gs16, d, B, c.W(l.critic_out), l.critic_out.pitch, d, d, gA, d, false));       // g_attc (B, d)
    __half* gq_c = gs16;                                                                          // (B, d)
    BSRL_TRY(attention29_bwd(qkv, 3 * d, sv.key_bias, B, d, l.H, 2, 1, gA, d, gq_c, d, gB, 2 * d, gB + d, 2 * d, st));
    BSRL_TRY(to_tX(hv, d, ident, R, d));
    BSRL_TRY(to_tA_slices(gB, 2 * d, R, 2 * d, {{G("critic_k.bias"), 0, d}, {G("critic_v.bias"), d, d}}));
    BSRL_TRY(wgrad_t(0, d, d, R, G("critic_k.weight"), d));
    BSRL_TRY(wgrad_t(d, d, d, R, G("critic_v.weight"), d));
    BSRL_TRY(wgrad(gq_c, d, B, d, hv, d, torso_rows, d, "critic_q"));
    BSRL_TRY(dgrad(gB, 2 * d, R, c.W(l.critic_kv), l.critic_kv.pitch, 2 * d, d, g32, d, true));    // g_hv from k, v
    BSRL_TRY(dgrad(gq_c, d, B, c.W(l.critic_q), l.critic_q.pitch, d, d, gs32, d, true));           // ... and from q, torso rows
    BSRL_TRY(add_rows32(gs32, d, g32, d, torso_rows, B, d, 1, st));
    BSRL_TRY(ln_bwd(x_last, d, ident, l.critic_ln, "critic_ln", g32, true, d, nullptr, gx, d, ident, R, d));   // gx = critic's share

    // ---- action heads and trunk
    {   // all 29 heads as ONE stacked product into a scratch matrix, then row slices to each head's gradient
      float* hw = S<float>(w.heads_scratch);
      float* hb = S<float>(w.bias_scratch);
      BSRL_CUDA_OK(cudaMemsetAsync(hw, 0, (size_t)l.head_cols_pad * D * 4, st));
      BSRL_CUDA_OK(cudaMemsetAsync(hb, 0, (size_t)l.head_cols_pad * 4, st));
      BSRL_TRY(to_tA(graw, w.ld_graw, ident, B, l.head_cols_pad, hb));
      BSRL_TRY(to_tX(z16 + d, ldz, ident, B, D));
      BSRL_TRY(wgrad_t(0, l.head_cols_pad, D, B, hw, D));
      for (int j = 0; j < kActHeads; ++j) {
        const std::string hn = "heads." + std::to_string(j);
        const int k = c.cfg->head_gears[j];
        if (float* gw = G(hn + ".weight"))
          BSRL_CUDA_OK(cudaMemcpyAsync(gw, hw + (int64_t)l.head_first[j] * D, (size_t)k * D * 4, cudaMemcpyDeviceToDevice, st));
        if (float* gb = G(hn + ".bias"))
          BSRL_CUDA_OK(cudaMemcpyAsync(gb, hb + l.head_first[j], (size_t)k * 4, cudaMemcpyDeviceToDevice, st));
      }
    }
    BSRL_TRY(dgrad(graw, w.ld_graw, B, c.W(l.heads), l.heads.pitch, l.n_head_cols, D, gs32, D, true));   // g_h from the heads
    BSRL_TRY(add_rows32(gz32 + d, ldz, gs32, D, ident, B, D, 1, st));                                     // + the critic's
    float* g_xt2 = gz32;                               // (B, D) f32, reuses the head of g_z (g_a was consumed above)
    if (l.trunk_v2) {
      // out side: g_x0 (its direct share) -> g_xt2, g_t2 -> gs16, g_alpha; then W2, the scaled ReLU, W1; in side
      BSRL_TRY(simba2_out_bwd(xt2, t2_32, at<float>(c.arena, l.v2_alpha), c_alpha, gs32, g_xt2, gs16, G("trunk_alpha"), B, D, st));
      BSRL_TRY(wgrad(gs16, D, B, D, r16, Hh, ident, Hh, "trunk_w2"));
      BSRL_TRY(dgrad(gs16, D, B, c.W(l.trunk_fc2), l.trunk_fc2.pitch, D, Hh, gA, Hh, false));
      BSRL_TRY(scale_relu_bwd(gA, t1_32, at<float>(c.arena, l.v2_s_1), G("trunk_s_1"), B, Hh, st));
      BSRL_TRY(wgrad(gA, Hh, B, Hh, u16, D, ident, D, "trunk_w1"));
      BSRL_TRY(dgrad(gA, Hh, B, c.W(l.trunk_fc1), l.trunk_fc1.pitch, Hh, D, gs32, D, true));       // g_x0 through W1
      BSRL_TRY(simba2_in_bwd(xt, at<float>(c.arena, l.v2_s_in), g_xt2, gs32, gs16, G("trunk_s_in"), B, D, st));
      BSRL_TRY(wgrad(gs16, D, B, D, sv.lead16, kLead * d, ident, kLead * d, "trunk_in"));
    } else {
      BSRL_TRY(ln_bwd(xt2, D, ident, l.trunk_ln2, "trunk_ln2", gs32, true, D, nullptr, g_xt2, D, ident, B, D));
      BSRL_TRY(cast16(g_xt2, D, ident, gs16, D, B, D));
      BSRL_TRY(wgrad(gs16, D, B, D, r16, Hh, ident, Hh, "trunk_fc2"));
      BSRL_TRY(dgrad(gs16, D, B, c.W(l.trunk_fc2), l.trunk_fc2.pitch, D, Hh, gA, Hh, false));
      BSRL_TRY(relu_mask16(gA, Hh, r16, Hh, B, Hh, st));
      BSRL_TRY(wgrad(gA, Hh, B, Hh, u16, D, ident, D, "trunk_fc1"));
      BSRL_TRY(dgrad(gA, Hh, B, c.W(l.trunk_fc1), l.trunk_fc1.pitch, Hh, D, gs32, D, true));
      BSRL_TRY(ln_bwd(xt, D, ident, l.trunk_ln1, "trunk_ln1", gs32, true, D, g_xt2, g_xt2, D, ident, B, D));   // g_xt
      BSRL_TRY(cast16(g_xt2, D, ident, gs16, D, B, D));
      BSRL_TRY(wgrad(gs16, D, B, D, sv.lead16, kLead * d, ident, kLead * d, "trunk_proj"));
    }
    float* g_lead = gs32;                              // (B, 5 d) = (5 B, d) lead rows
    BSRL_TRY(dgrad(gs16, D, B, c.W(l.trunk_proj), l.trunk_proj.pitch, D, kLead * d, g_lead, kLead * d, true));

    // ---- value residual: block 0's values (every later block mixes them in) and the fp32 gradient that flows back to them
    const bool vres = l.value_residual && l.L > 1;
    __half* v0 = vres ? S<__half>(w.v0) : nullptr;
    __half* vown = vres ? S<__half>(w.vown) : nullptr;
    float* gv0 = vres ? S<float>(w.gv0) : nullptr;
    if (vres) {
      const BlockW& b0 = l.blocks[0];
      BSRL_TRY(layernorm(sv.x[0], d, ident, c.G(b0.ln_attn), c.Be(b0.ln_attn), eps, R, d, h16, d, st));
      BSRL_TRY(linear(linear_args(h16, d, c.W(b0.qkv, 2 * d), d, c.Bv(b0.qkv, 2 * d), v0, d, 0, 0, R, d, d), st));
      BSRL_CUDA_OK(cudaMemsetAsync(gv0, 0, (size_t)R * d * 4, st));
    }
    // after the projection of block i > 0: keep the block's own values, mix block 0's in (the forward's arithmetic)
    auto mix_values = [&](int i, __half* vcols, int ld) -> int {
      if (!vres || i == 0) return BSRL_OK;
      return vres_mix(vcols, ld, R, d, vown, v0, at<float>(c.arena, l.blocks[i].vres), st);
    };
    // after the attention backward of block i: the gradient of the mixed values becomes that of the block's own values
    // (i > 0; block 0's share collects in gv0), or block 0's own gradient takes the collected share in
    auto unmix_grads = [&](int i, __half* gvcols, int64_t ld) -> int {
      if (!vres) return BSRL_OK;
      if (i == 0) return add_f32_into_f16(gvcols, ld, gv0, R, d, st);
      const std::string pn = "blocks." + std::to_string(i);
      return vres_bwd(gvcols, ld, vown, v0, at<float>(c.arena, l.blocks[i].vres), gv0, G(pn + ".vres_a"), G(pn + ".vres_b"), R, d, st);
    };

    // ---- last block, on the lead rows
    {
      const int i = l.L - 1;
      const BlockW& b = l.blocks[i];
      const std::string p = "blocks." + std::to_string(i);
      BSRL_TRY(layernorm(x_last, d, ident, c.G(b.ln_attn), c.Be(b.ln_attn), eps, R, d, h16, d, st));
      BSRL_TRY(linear(linear_args(h16, d, c.W(b.qkv, d), d, c.Bv(b.qkv, d), qkv + d, 3 * d, 0, 0, R, 2 * d, d), st));
      {
        LinearArgs pq = linear_args(h16, d, c.W(b.qkv), d, c.Bv(b.qkv), qkv, 3 * d, 0, 0, Rl, d, d);
        pq.amap = lead_rows; pq.cmap = lead_rows;
        BSRL_TRY(linear(pq, st));
      }
      BSRL_TRY(mix_values(i, qkv + 2 * d, 3 * d));
      BSRL_TRY(attention(qkv, 3 * d, sv.key_bias, B, d, l.H, 0, kLead, att, d, st));
      BSRL_TRY(tail_fwd(i, Rl, x_last, lead_rows, att, x1, h2, hid));
      float* g_x1 = x1 + Rl * d;                       // (Rl, d) f32: the unused upper part of the x1 buffer
      if (c.cfg->final_ln) {
        // the readout is final_ln of the block's output rows: recompute them (x2 = x1 + hid W2^T + b2) and take the
        // readout gradient back through the LayerNorm, in place
        float* x2 = x1 + 3 * Rl * d;
        LinearArgs pd = linear_args(hid, F, c.W(b.down), F, c.Bv(b.down), x2, d, 1, 0, Rl, d, F);
        pd.R = x1; pd.ldr = d;
        BSRL_TRY(linear(pd, st));
        BSRL_TRY(ln_bwd(x2, d, ident, l.final_ln, "final_ln", g_lead, true, d, nullptr, g_lead, d, ident, Rl, d));
      }
      BSRL_TRY(tail_bwd(i, Rl, g_lead, g_x1, x1, h2, hid, att, gA));       // gA: fp16 gradient of the attention output
      __half* gq = gs16;                               // (Rl, d)
      BSRL_TRY(attention29_bwd(qkv, 3 * d, sv.key_bias, B, d, l.H, 0, kLead, gA, d, gq, d, gB, 2 * d, gB + d, 2 * d, st));
      BSRL_TRY(unmix_grads(i, gB + d, 2 * d));
      BSRL_TRY(to_tX(h16, d, ident, R, d));
      BSRL_TRY(to_tA_slices(gB, 2 * d, R, 2 * d, {{G(p + ".k_proj.bias"), 0, d}, {G(p + ".v_proj.bias"), d, d}}));
      BSRL_TRY(wgrad_t(0, d, d, R, G(p + ".k_proj.weight"), d));
      BSRL_TRY(wgrad_t(d, d, d, R, G(p + ".v_proj.weight"), d));
      BSRL_TRY(wgrad(gq, d, Rl, d, h16, d, lead_rows, d, p + ".q_proj"));
      BSRL_TRY(dgrad(gB, 2 * d, R, c.W(b.qkv, d), b.qkv.pitch, 2 * d, d, g32, d, true));           // g_h from k, v
      float* gq32 = S<float>(w.x1) + 2 * Rl * d;        // (Rl, d) f32
      BSRL_TRY(dgrad(gq, d, Rl, c.W(b.qkv), b.qkv.pitch, d, d, gq32, d, true));                     // ... and from q, lead rows
      BSRL_TRY(add_rows32(gq32, d, g32, d, lead_rows, Rl, d, 1, st));
      BSRL_TRY(ln_bwd(x_last, d, ident, b.ln_attn, p + ".ln_attn", g32, true, d, gx, gx, d, ident, R, d));
      BSRL_TRY(add_rows32(g_x1, d, gx, d, lead_rows, Rl, d, 1, st));                               // the residual path of the lead rows
    }

    // ---- blocks L-2 .. 0, all rows
    __half* gx16 = S<__half>(w.gx16);
    const __half* gx16_live = nullptr;     // fp16 copy of gx, once a LayerNorm backward of this loop has written it
    for (int i = l.L - 2; i >= 0; --i) {
      const BlockW& b = l.blocks[i];
      const std::string p = "blocks." + std::to_string(i);
      const float* x_in = sv.x[i];
      BSRL_TRY(layernorm(x_in, d, ident, c.G(b.ln_attn), c.Be(b.ln_attn), eps, R, d, h16, d, st));
      BSRL_TRY(linear(linear_args(h16, d, c.W(b.qkv), d, c.Bv(b.qkv), qkv, 3 * d, 0, 0, R, 3 * d, d), st));
      BSRL_TRY(mix_values(i, qkv + 2 * d, 3 * d));
      BSRL_TRY(attention(qkv, 3 * d, sv.key_bias, B, d, l.H, 0, kT, att, d, st));
      BSRL_TRY(tail_fwd(i, R, x_in, ident, att, x1, h2, hid));
      BSRL_TRY(tail_bwd(i, R, gx, gx, x1, h2, hid, att, gA, gx16_live));                            // gx: g(x_{i+1}) -> g(x1)
      BSRL_TRY(attention29_bwd(qkv, 3 * d, sv.key_bias, B, d, l.H, 0, kT, gA, d, gB, 3 * d, gB + d, 3 * d, gB + 2 * d, 3 * d, st));
      BSRL_TRY(unmix_grads(i, gB + 2 * d, 3 * d));
      BSRL_TRY(to_tX(h16, d, ident, R, d));
      BSRL_TRY(to_tA_slices(gB, 3 * d, R, 3 * d, {{G(p + ".q_proj.bias"), 0, d}, {G(p + ".k_proj.bias"), d, d},
                                                 {G(p + ".v_proj.bias"), 2 * d, d}}));
      const char* names[3] = {".q_proj", ".k_proj", ".v_proj"};
      for (int s = 0; s < 3; ++s) BSRL_TRY(wgrad_t(s * d, d, d, R, G(p + names[s] + ".weight"), d));
      BSRL_TRY(dgrad(gB, 3 * d, R, c.W(b.qkv), b.qkv.pitch, 3 * d, d, g32, d, true));
      BSRL_TRY(ln_bwd(x_in, d, ident, b.ln_attn, p + ".ln_attn", g32, true, d, gx, gx, d, ident, R, d, gx16));   // gx: g(x_i)
      gx16_live = gx16;
    }

    // ---- token encoders (no gradient flows to the observation)
    struct Enc { const Encoder* e; const char* name; int64_t rows, row0; int group, first, in; };
    const Enc encs[4] = {{&l.saber, "saber_mlp", 2 * B, 0, 2, 0, kSaberFeat + 2},
                         {&l.torso, "torso_mlp", B, 2 * B, 1, 2, kTorsoFeat},
                         {&l.leg, "leg_mlp", 2 * B, 3 * B, 2, 3, kLegFeat + 2},
                         {&l.note, "note_mlp", (int64_t)kSlots * B, 5 * B, kSlots, kLead, l.note_in}};
    for (const Enc& e : encs) {
      const __half* feat = sv.feat + e.row0 * 64;
      const RowMap rows{e.group, kT, e.first};
      BSRL_TRY(linear(linear_args(feat, 64, c.W(e.e->l0), e.e->l0.pitch, c.Bv(e.e->l0), hid, d, 0, 1, e.rows, d, 64), st));   // hidden
      BSRL_TRY(cast16(gx, d, rows, gB, d, e.rows, d));                                               // g of this encoder's tokens
      if (c.cfg->emb_ln) {
        // tokens = emb_ln(encoder output): recompute the encoder's output rows (fp32) and take g back through the
        // LayerNorm; the fp16 copy of the result lands in gB again
        float* pre = x1;                                  // (e.rows, d) f32: the block scratch is free by now
        BSRL_TRY(linear(linear_args(hid, d, c.W(e.e->l1), e.e->l1.pitch, c.Bv(e.e->l1), pre, d, 1, 0, e.rows, d, d), st));
        BSRL_TRY(ln_bwd(pre, d, ident, l.emb_ln, "emb_ln", gB, false, d, nullptr, g32, d, ident, e.rows, d, gB));
      }
      BSRL_TRY(wgrad(gB, d, e.rows, d, hid, d, ident, d, std::string(e.name) + ".2"));
      BSRL_TRY(dgrad(gB, d, e.rows, c.W(e.e->l1), e.e->l1.pitch, d, d, gA, d, false, hid, d));       // through the hidden ReLU
      // first layer: the K-padded (d, 64) product goes to a scratch matrix, its first `in` columns are the gradient
      float* sw = S<float>(w.scratch_w);
      BSRL_CUDA_OK(cudaMemsetAsync(sw, 0, (size_t)d * 64 * 4, st));
      BSRL_TRY(to_tA(gA, d, ident, e.rows, d, G(std::string(e.name) + ".0.bias")));
      BSRL_TRY(to_tX(feat, 64, ident, e.rows, 64));
      BSRL_TRY(wgrad_t(0, d, 64, e.rows, sw, 64));
      if (float* gw = G(std::string(e.name) + ".0.weight"))
        BSRL_CUDA_OK(cudaMemcpy2DAsync(gw, (size_t)e.in * 4, sw, 64 * 4, (size_t)e.in * 4, d, cudaMemcpyDeviceToDevice, st));
    }
    return BSRL_OK;
  }
};

// Flat gradient buffer: one slot per parameter in parameter-table order, each starting on a 16-byte boundary
int64_t grad_floats(const bsrl_config& cfg, const Layout& l, std::map<std::string, int64_t>* offsets,
                    int64_t* by_index = nullptr) {
  int64_t off = 0;
  int i = 0;
  for (const ParamSlot& p : make_param_slots(cfg, l)) {
    if (offsets) (*offsets)[p.name] = off;
    if (by_index) by_index[i] = off;
    ++i;
    off += round_up(p.rows * p.cols, 4);
  }
  return off;
}

}  // namespace
}  // namespace bsrl

using namespace bsrl;
using namespace bsrl::fwd;

extern "C" {

// ---- single stages of the backward (unit tests)
int bsrl_layernorm_bwd(const float* x, const float* gamma, float eps, const float* gy, const float* g_residual,
                       int64_t rows, int32_t d, float* gx, float* g_gamma, float* g_beta, void* stream) {
  return layernorm_bwd(x, d, identity_map(), gamma, eps, gy, 1, d, g_residual, gx, d, identity_map(), g_gamma, g_beta, rows, d,
                       as_stream(stream));
}

int bsrl_attention_bwd(const void* qkv_f16, const float* key_bias, int64_t n_envs, int32_t d, int32_t n_heads,
                       int32_t q_first, int32_t n_q, const void* g_out_f16, void* gq_f16, void* gkv_f16, void* stream) {
  __half* gkv = static_cast<__half*>(gkv_f16);
  return attention29_bwd(static_cast<const __half*>(qkv_f16), 3 * d, key_bias, n_envs, d, n_heads, q_first, n_q,
                         static_cast<const __half*>(g_out_f16), d, static_cast<__half*>(gq_f16), d, gkv, 2 * d, gkv + d, 2 * d,
                         as_stream(stream));
}

int bsrl_head_tail_bwd(const bsrl_config* cfg, const float* head_out, const float* value_bin_logits, int64_t n_envs,
                       const void* actions, int32_t act_dtype, const float* g_logprob, const float* g_entropy,
                       const float* g_value, const float* g_value_logits, const float* g_logits, float scale,
                       void* g_head_out_f16, int32_t ld_g_head, void* g_value_bins_f16, int32_t ld_g_bins, void* stream) {
  BSRL_TRY(validate_config(cfg));
  Layout l = make_layout(*cfg);
  if (ld_g_head < l.head_cols_pad || ld_g_bins < l.bins_pad) {
    set_error("head_tail_bwd: output pitches %d / %d below %d / %d", ld_g_head, ld_g_bins, l.head_cols_pad, l.bins_pad);
    return BSRL_ERR_SHAPE;
  }
  HeadTailArgs h;
  memset(&h, 0, sizeof(h));
  h.raw = head_out; h.ld_raw = l.head_cols_pad;
  h.vraw = value_bin_logits; h.ld_v = l.bins_pad;
  head_shape(*cfg, l, h);
  h.actions = actions; h.act_dtype = act_dtype;
  h.n_envs = n_envs;
  return head_tail_bwd(h, g_logprob, g_entropy, g_value, g_value_logits, g_logits, scale, static_cast<__half*>(g_head_out_f16),
                       ld_g_head, static_cast<__half*>(g_value_bins_f16), ld_g_bins, as_stream(stream));
}

int64_t bsrl_linear_bwd_scratch_bytes(int64_t m, int32_t n, int32_t k) {
  const int64_t mp = pad64(m);
  return round_up((int64_t)n * mp * 2, 256) + round_up((int64_t)k * mp * 2, 256) + round_up(pad64(n) * (int64_t)k * 2, 256);
}

int bsrl_linear_bwd(const void* g_f16, const void* x_f16, const void* w_f16, int64_t m, int32_t n, int32_t k,
                    float* g_weight, float* g_bias, void* g_x, int32_t g_x_f32, void* scratch, int64_t scratch_bytes,
                    void* stream) {
  if (!g_f16 || !x_f16 || !scratch) {
    set_error("linear_bwd: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (n % 64 != 0 || k % 16 != 0 || m < 1 || pad64(m) > 0x7fffffff) {
    set_error("linear_bwd: needs n %% 64 == 0, k %% 16 == 0, m >= 1");
    return BSRL_ERR_SHAPE;
  }
  if (scratch_bytes < bsrl_linear_bwd_scratch_bytes(m, n, k) || (reinterpret_cast<uintptr_t>(scratch) & 255)) {
    set_error("linear_bwd: scratch too small or not 256-byte aligned");
    return BSRL_ERR_WORKSPACE;
  }
  cudaStream_t st = as_stream(stream);
  use_process_engine();
  const int64_t mp = pad64(m);
  __half* tA = static_cast<__half*>(scratch);
  __half* tX = at<__half>(scratch, round_up((int64_t)n * mp * 2, 256));
  __half* wT = at<__half>(scratch, round_up((int64_t)n * mp * 2, 256) + round_up((int64_t)k * mp * 2, 256));
  const __half* g = static_cast<const __half*>(g_f16);
  if (g_weight) {     // g_weight (n, k) += g^T x as a split-K product over the m rows; the caller zeroes it first
    const int64_t tiles = ((n + 127) / 128) * ((k + 255) / 256);
    const int splits = (int)(sm_count() / tiles) < 1 ? 1 : (int)(sm_count() / tiles);
    LinearArgs r = linear_args(g, n, static_cast<const __half*>(x_f16), k, nullptr, g_weight, k, 1, 0, n, k, (int)m);
    r.a_mn = r.w_mn = 1;                       // both operands as they lie: the contraction index is their row
    r.k_splits = splits;
    if (linear_rows_ok(r)) {
      if (g_bias) BSRL_TRY(colsum16(g, n, m, n, g_bias, st));
      BSRL_TRY(linear(r, st));
    } else {                                   // transposed copies, bias gradient on the way
      BSRL_TRY(transpose16(g, n, identity_map(), m, n, tA, mp, mp, st, g_bias));
      BSRL_TRY(transpose16(static_cast<const __half*>(x_f16), k, identity_map(), m, k, tX, mp, mp, st));
      LinearArgs a = linear_args(tA, (int)mp, tX, (int)mp, nullptr, g_weight, k, 1, 0, n, k, (int)mp);
      a.k_splits = splits;
      BSRL_TRY(linear(a, st));
    }
  }
  if (g_bias && !g_weight) BSRL_TRY(colsum16(g, n, m, n, g_bias, st));
  if (g_x) {          // g_x (m, k) = g w
    if (!w_f16) {
      set_error("linear_bwd: the input gradient needs the weight");
      return BSRL_ERR_NULL;
    }
    LinearArgs r = linear_args(g, n, static_cast<const __half*>(w_f16), k, nullptr, g_x, k, g_x_f32 ? 1 : 0, 0, m, k, n);
    r.w_mn = 1;
    if (linear_rows_ok(r)) {
      BSRL_TRY(linear(r, st));
    } else {
      BSRL_TRY(transpose16(static_cast<const __half*>(w_f16), k, identity_map(), n, k, wT, n, n, st));
      BSRL_TRY(linear(linear_args(g, n, wT, n, nullptr, g_x, k, g_x_f32 ? 1 : 0, 0, m, k, n), st));
    }
  }
  return BSRL_OK;
}

int64_t bsrl_train_save_bytes(const bsrl_config* cfg, int64_t n_envs) {
  if (validate_config(cfg) != BSRL_OK || n_envs < 0) return -1;
  Layout l = make_layout(*cfg);
  if (train_supported(cfg, l) != BSRL_OK) return -1;
  return make_save(l, n_envs).bytes;
}

int64_t bsrl_backward_workspace_bytes(const bsrl_config* cfg, int64_t n_envs) {
  if (validate_config(cfg) != BSRL_OK || n_envs < 0) return -1;
  Layout l = make_layout(*cfg);
  if (train_supported(cfg, l) != BSRL_OK) return -1;
  return make_bwd(l, n_envs).bytes;
}

int64_t bsrl_grad_floats(const bsrl_config* cfg, int64_t* offsets, int32_t n_offsets) {
  if (validate_config(cfg) != BSRL_OK) return -1;
  Layout l = make_layout(*cfg);
  if (offsets && n_offsets != (int32_t)make_param_slots(*cfg, l).size()) {
    set_error("grad_floats: %d offsets asked for, the model has %d parameters", n_offsets, (int)make_param_slots(*cfg, l).size());
    return -1;
  }
  return grad_floats(*cfg, l, nullptr, offsets);
}

int bsrl_forward_train(const bsrl_config* cfg, const void* arena, const void* obs, int32_t obs_dtype, int64_t n_envs,
                       const void* actions, int32_t act_dtype, float* logits, float* logprob, float* entropy,
                       float* ent_head, float* value, float* value_logits, void* save, int64_t save_bytes,
                       void* workspace, int64_t workspace_bytes, void* stream) {
  Ctx c;
  BSRL_TRY(make_ctx(c, cfg, arena, n_envs, workspace, workspace_bytes, stream));
  BSRL_TRY(train_supported(cfg, c.l));
  if (!obs || !actions || !logprob || !value || !save) {
    set_error("forward_train: NULL obs / actions / logprob / value / save");
    return BSRL_ERR_NULL;
  }
  if (act_dtype != BSRL_U8 && act_dtype != BSRL_I32 && act_dtype != BSRL_I64) {
    set_error("forward_train: actions must be u8, i32 or i64");
    return BSRL_ERR_UNSUPPORTED;
  }
  if (reinterpret_cast<uintptr_t>(save) & 255) {
    set_error("forward_train: the save buffer must be 256-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  const SaveLayout s = make_save(c.l, n_envs);
  if (save_bytes < s.bytes) {
    set_error("forward_train: save buffer %lld bytes < required %lld", (long long)save_bytes, (long long)s.bytes);
    return BSRL_ERR_WORKSPACE;
  }
  if (n_envs == 0) return BSRL_OK;
  const TrainPtrs t = save_ptrs(s, c.l, save);
  c.train = &t;
  HeadTailArgs h;
  memset(&h, 0, sizeof(h));
  h.actions = actions; h.act_dtype = act_dtype;
  h.logits = logits; h.logprob = logprob; h.entropy = entropy; h.ent_head = ent_head;
  h.value = value; h.value_logits = value_logits;
  return run_forward(c, obs, obs_dtype, h);
}

int bsrl_backward(const bsrl_config* cfg, const void* arena, int64_t n_envs, const void* actions, int32_t act_dtype,
                  const void* save, int64_t save_bytes, const float* g_logprob, const float* g_entropy,
                  const float* g_value, const float* g_value_logits, const float* g_logits, float loss_scale,
                  float* grads, int64_t grad_floats_given, void* workspace, int64_t workspace_bytes, void* stream) {
  BSRL_TRY(validate_config(cfg));
  Layout l = make_layout(*cfg);
  BSRL_TRY(train_supported(cfg, l));
  if (!arena || !save || !grads || !workspace) {
    set_error("backward: NULL arena / save / grads / workspace");
    return BSRL_ERR_NULL;
  }
  if ((g_logprob || g_entropy || g_logits) && !actions && g_logprob) {
    set_error("backward: the log-prob gradient needs the actions");
    return BSRL_ERR_NULL;
  }
  if (n_envs < 0 || n_envs > (int64_t)1 << 26) {
    set_error("backward: n_envs %lld out of range", (long long)n_envs);
    return BSRL_ERR_SHAPE;
  }
  if (!(loss_scale > 0.f)) {
    set_error("backward: loss_scale must be > 0");
    return BSRL_ERR_SHAPE;
  }
  if ((reinterpret_cast<uintptr_t>(arena) & 255) || (reinterpret_cast<uintptr_t>(save) & 255) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(grads) & 15)) {
    set_error("backward: arena, save and workspace must be 256-byte aligned, grads 16-byte aligned");
    return BSRL_ERR_ALIGN;
  }
  const SaveLayout s = make_save(l, n_envs);
  const BwdLayout w = make_bwd(l, n_envs);
  std::map<std::string, int64_t> offsets;
  const int64_t n_grad = grad_floats(*cfg, l, &offsets);
  if (save_bytes < s.bytes || workspace_bytes < w.bytes || grad_floats_given < n_grad) {
    set_error("backward: save %lld / workspace %lld bytes / grads %lld floats given, %lld / %lld / %lld needed",
              (long long)save_bytes, (long long)workspace_bytes, (long long)grad_floats_given, (long long)s.bytes,
              (long long)w.bytes, (long long)n_grad);
    return BSRL_ERR_WORKSPACE;
  }
  cudaStream_t st = as_stream(stream);
  BSRL_CUDA_OK(cudaMemsetAsync(grads, 0, (size_t)n_grad * 4, st));
  if (n_envs == 0) return BSRL_OK;
  Ctx c;
  c.cfg = cfg;
  c.l = l;
  c.paths = plan_paths(l, 1);       // the recomputation runs the separate GEMM / LayerNorm / attention kernels
  use_process_engine();
  c.arena = arena;
  c.ws = workspace;
  c.B = n_envs;
  c.st = st;
  const TrainPtrs t = save_ptrs(s, l, const_cast<void*>(save));
  Bwd b{c, c.l, t, w, workspace, grads, offsets, loss_scale, st, n_envs, n_envs * kT, n_envs * kLead, l.d, l.F, l.D};
  HeadTailArgs h;
  memset(&h, 0, sizeof(h));
  h.raw = t.raw; h.ld_raw = l.head_cols_pad;
  h.vraw = t.vraw; h.ld_v = l.bins_pad;
  head_shape(*cfg, l, h);
  h.actions = actions; h.act_dtype = act_dtype;
  h.n_envs = n_envs;
  return b.run(h, g_logprob, g_entropy, g_value, g_value_logits, g_logits);
}

}  // extern "C"
