// Weight refresh in a handful of launches, optionally fused with the optimizer step.
//
// The reference keeps fp32 masters and a flat fp16 replica that ONE cast kernel refreshes after every
// optimizer step (flat_refresh, python/fp16_linear.py:236-246; the trainer bumps the weights version
// after opt.step(), python/train_batch.py:2847-2854).  Here the replica is the packed arena, whose
// matrices are stacked, K-padded and -- for the fused attention kernel -- regrouped, so a refresh is a
// scatter: every master has a primary destination and possibly a few row ranges with a second one.
//
// multi_pack_kernel does that scatter for up to kMaxSegs masters per launch (the segment table travels
// by value in the kernel parameters: no device-side table, no host-to-device copy), and, when a master
// comes with a gradient, first applies an Adam / AdamW step to it in place:
//
//   g' = g * inv_scale;  p *= 1 - lr wd;  m = b1 m + (1 - b1) g';  v = b2 v + (1 - b2) g'^2
//   p -= (lr / (1 - b1^t)) m / (sqrt(v) / sqrt(1 - b2^t) + eps)        (torch.optim.AdamW)
//
// so the fp16 arena is produced by the optimizer kernel itself and no separate refresh pass runs.  In additive
// mode (step = 0 with gradients given) the "gradient" is a finished update and the step is p += u: the last
// stage of an optimizer whose direction is computed elsewhere (the Muon half of the reference's hybrid optimizer
// orthogonalises its momentum with a chain of small matrix products first, python/train_batch.py:818-931).
#include "kernels.cuh"
#include "layout.h"

namespace bsrl {
namespace {

constexpr int kMaxSegs = 20, kMaxCopies = 64;

struct Seg {
  float* p;                // master (rows, cols) f32
  const float* g;          // gradient, or nullptr: no update, scatter only
  float* m;                // exp_avg
  float* v;                // exp_avg_sq
  int64_t dst;             // primary destination in the arena (bytes)
  int rows, cols, pitch;   // pitch: elements per destination row (fp16 matrices); 0: dense fp32 vector
  int half;
  float lr, wd;
  int copy_first, copy_n;  // its row ranges with a second destination
};
struct Copy {
  int row0, n_rows, pitch, half;
  int64_t dst;
};
struct Table {
  Seg seg[kMaxSegs];
  Copy copy[kMaxCopies];
  int n_seg;
  float beta1, beta2, eps, bc1, rsqrt_bc2;   // bias corrections 1 - b1^t and 1 / sqrt(1 - b2^t)
  const float* inv_scale;                    // device scalar multiplying every gradient, or nullptr
  const float* found_inf;                    // device scalar: non-zero = skip every update (scatter still runs)
  int additive;                              // the gradients are finished updates: p += g
};

__device__ __forceinline__ void put(uint8_t* arena, int64_t dst, int pitch, int half, int r, int c, int cols, float val) {
  if (half) reinterpret_cast<__half*>(arena + dst)[(int64_t)r * pitch + c] = __float2half_rn(val);
  else reinterpret_cast<float*>(arena + dst)[(int64_t)r * cols + c] = val;
}

// blockIdx.y = segment; blockIdx.x strides over its elements
__global__ void __launch_bounds__(256) multi_pack_kernel(const __grid_constant__ Table t, uint8_t* __restrict__ arena) {
  const Seg& s = t.seg[blockIdx.y];
  const int64_t n = (int64_t)s.rows * s.cols;
  const bool update = s.g != nullptr && !(t.found_inf && *t.found_inf != 0.f);
  const float inv_scale = (update && t.inv_scale) ? *t.inv_scale : 1.f;
  const float step = s.lr / t.bc1, decay = 1.f - s.lr * s.wd;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float p = s.p[i];
    if (update && t.additive) {
      p += s.g[i];
      s.p[i] = p;
    } else if (update) {
      const float g = s.g[i] * inv_scale;
      const float m = t.beta1 * s.m[i] + (1.f - t.beta1) * g;
      const float v = t.beta2 * s.v[i] + (1.f - t.beta2) * g * g;
      s.m[i] = m;
      s.v[i] = v;
      p = p * decay - step * m / (sqrtf(v) * t.rsqrt_bc2 + t.eps);
      s.p[i] = p;
    }
    const int r = (int)(i / s.cols), c = (int)(i % s.cols);
    put(arena, s.dst, s.pitch, s.half, r, c, s.cols, p);
    for (int k = 0; k < s.copy_n; ++k) {
      const Copy& cp = t.copy[s.copy_first + k];
      if (r >= cp.row0 && r < cp.row0 + cp.n_rows) put(arena, cp.dst, cp.pitch, cp.half, r - cp.row0, c, s.cols, p);
    }
  }
}

}  // namespace

int multi_pack(const bsrl_config& cfg, const Layout& l, float* const* params, const float* const* grads,
               float* const* exp_avg, float* const* exp_avg_sq, const float* lr, const float* wd, float beta1,
               float beta2, float eps, int step, const float* inv_scale, const float* found_inf, void* arena,
               cudaStream_t stream) {
  const std::vector<ParamSlot> slots = make_param_slots(cfg, l);
  const std::vector<CopySlot> copies = make_copy_slots(cfg, l, slots);
  return multi_pack_slots(slots, copies, params, grads, exp_avg, exp_avg_sq, lr, wd, beta1, beta2, eps, step, inv_scale,
                          found_inf, arena, stream);
}

int multi_pack_slots(const std::vector<ParamSlot>& slots, const std::vector<CopySlot>& copies, float* const* params,
                     const float* const* grads, float* const* exp_avg, float* const* exp_avg_sq, const float* lr,
                     const float* wd, float beta1, float beta2, float eps, int step, const float* inv_scale,
                     const float* found_inf, void* arena, cudaStream_t stream) {
  Table t;
  memset(&t, 0, sizeof(t));
  t.beta1 = beta1; t.beta2 = beta2; t.eps = eps;
  t.bc1 = step > 0 ? 1.f - powf(beta1, (float)step) : 1.f;
  t.rsqrt_bc2 = step > 0 ? 1.f / sqrtf(1.f - powf(beta2, (float)step)) : 1.f;
  t.inv_scale = inv_scale;
  t.found_inf = found_inf;
  t.additive = (step == 0 && grads != nullptr) ? 1 : 0;
  int n_copy = 0;
  int64_t max_elems = 0;
  auto flush = [&]() -> int {
    if (t.n_seg == 0) return BSRL_OK;
    int64_t bx = (max_elems + 255) / 256;
    if (bx > 64) bx = 64;
    if (bx < 1) bx = 1;
    multi_pack_kernel<<<dim3((unsigned)bx, (unsigned)t.n_seg), 256, 0, stream>>>(t, static_cast<uint8_t*>(arena));
    BSRL_LAUNCH_OK("multi_pack_kernel");
    t.n_seg = 0;
    n_copy = 0;
    max_elems = 0;
    return BSRL_OK;
  };
  for (size_t i = 0; i < slots.size(); ++i) {
    const ParamSlot& ps = slots[i];
    int mine = 0;
    for (const CopySlot& cs : copies)
      if (cs.param == (int)i) ++mine;
    if (mine > kMaxCopies) {
      set_error("pack: parameter %s has %d regrouped row ranges (limit %d)", ps.name.c_str(), mine, kMaxCopies);
      return BSRL_ERR_UNSUPPORTED;
    }
    if (t.n_seg == kMaxSegs || n_copy + mine > kMaxCopies) {
      int rc = flush();
      if (rc != BSRL_OK) return rc;
    }
    Seg& s = t.seg[t.n_seg++];
    s.p = params[i];
    s.g = grads ? grads[i] : nullptr;
    s.m = (s.g && exp_avg) ? exp_avg[i] : nullptr;
    s.v = (s.g && exp_avg_sq) ? exp_avg_sq[i] : nullptr;
    if (s.g && !t.additive && (!s.m || !s.v)) {
      set_error("adam_step_pack: parameter %s has a gradient but no optimizer state", ps.name.c_str());
      return BSRL_ERR_NULL;
    }
    s.dst = ps.dst;
    s.rows = (int)ps.rows; s.cols = (int)ps.cols; s.pitch = (int)ps.dst_pitch; s.half = ps.half ? 1 : 0;
    s.lr = lr ? lr[i] : 0.f;
    s.wd = wd ? wd[i] : 0.f;
    s.copy_first = n_copy;
    s.copy_n = mine;
    for (const CopySlot& cs : copies)
      if (cs.param == (int)i) {
        Copy& c = t.copy[n_copy++];
        c.row0 = (int)cs.src_row0; c.n_rows = (int)cs.n_rows; c.pitch = (int)cs.dst_pitch; c.half = cs.half ? 1 : 0;
        c.dst = cs.dst;
      }
    if (ps.rows * ps.cols > max_elems) max_elems = ps.rows * ps.cols;
  }
  return flush();
}

}  // namespace bsrl
