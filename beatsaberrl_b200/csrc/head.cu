// Head tail of the forward, one warp per environment.
//
// Lanes 0..28 each own one action head: they scatter the packed head outputs into the
// (29, k_max) logits over a -1e9 fill, and -- on the PPO recompute call -- run the
// log-softmax, pick the log-prob of the given action and compute the head's entropy; the
// 29-head sums are warp reductions.  The whole warp then turns the value-bin logits into the
// HL-Gauss expectation softmax(bins) . linspace(-vmax, vmax, bins).
//
// With the rollout outputs set it also writes the trainer's per-tick buffer rows (uint8 actions,
// de-normalised value: python/train_batch.py:2338-2350).
// Reference: masked-lane fill python/policy.py:1337-1344, value expectation :1399-1403,
// log-softmax / gather-sum / per-head entropy :1473-1516.  HBM-bound: reads
// 4*(sum K_j + bins) bytes and writes 4*(29 k_max + ...) bytes per env.
#include "kernels.cuh"

namespace bsrl {
namespace {

__device__ __forceinline__ int load_action(const void* a, int dtype, int64_t idx) {
  switch (dtype) {
    case BSRL_U8: return static_cast<const uint8_t*>(a)[idx];
    case BSRL_I32: return static_cast<const int32_t*>(a)[idx];
    default: return static_cast<int>(static_cast<const int64_t*>(a)[idx]);
  }
}

// Philox4x32-10 counter-based generator: 4 random words for (counter, key)
__device__ __forceinline__ uint4 philox4x32(uint4 c, uint2 k) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}
__device__ __forceinline__ float uniform01(uint32_t x) {   // in (0, 1)
  return __uint2float_rn(x >> 8) * 5.9604645e-8f + 2.9802322e-8f;
}

__global__ void __launch_bounds__(256) head_tail_kernel(HeadTailArgs p) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t env = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); env < p.n_envs;
       env += warps) {
    float lp = 0.f, ent = 0.f;
    if (lane < kActHeads) {
      const int k = p.gears[lane];
      const float* src = p.raw + env * p.ld_raw + p.first[lane];
      float v[7];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 7; ++i) {
        v[i] = i < k ? src[i] : kMaskedLogit;
        if (i < k) mx = fmaxf(mx, v[i]);
      }
      if (p.logits) {
        float* dst = p.logits + (env * kActHeads + lane) * p.k_max;
#pragma unroll
        for (int i = 0; i < 7; ++i)
          if (i < p.k_max) dst[i] = v[i];
      }
      if (p.logprob || p.entropy || p.ent_head || p.rng) {
        float se = 0.f;
#pragma unroll
        for (int i = 0; i < 7; ++i)
          if (i < k) se += expf(v[i] - mx);
        const float lse = mx + logf(se);
        if (p.actions || p.rng) {
          int a = 0;
          if (p.actions) {
            a = load_action(p.actions, p.act_dtype, env * kActHeads + lane);
            a = min(max(a, 0), p.k_max - 1);
          } else {
            // Gumbel-max: argmax_i (logsm_i - log E_i), E ~ Exp(1); only the head's live lanes compete
            const unsigned long long seed = p.rng[0], off = p.rng[1];
            const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
            const unsigned long long idx = (unsigned long long)env * kActHeads + lane;
            uint32_t w[8];
            uint4 r0 = philox4x32(make_uint4((uint32_t)idx, (uint32_t)(idx >> 32), (uint32_t)off, (uint32_t)(off >> 32) << 1), key);
            uint4 r1 = philox4x32(make_uint4((uint32_t)idx, (uint32_t)(idx >> 32), (uint32_t)off, ((uint32_t)(off >> 32) << 1) | 1u), key);
            w[0] = r0.x; w[1] = r0.y; w[2] = r0.z; w[3] = r0.w; w[4] = r1.x; w[5] = r1.y; w[6] = r1.z; w[7] = r1.w;
            float best = -INFINITY;
#pragma unroll
            for (int i = 0; i < 7; ++i)
              if (i < k) {
                const float sc = (v[i] - lse) - logf(-logf(uniform01(w[i])));
                if (sc > best) { best = sc; a = i; }
              }
            if (p.action_out) p.action_out[env * kActHeads + lane] = a;
            if (p.action_u8) p.action_u8[env * kActHeads + lane] = static_cast<unsigned char>(a);
          }
          float pick = kMaskedLogit;
#pragma unroll
          for (int i = 0; i < 7; ++i)
            if (i == a) pick = v[i];
          lp = pick - lse;
        }
#pragma unroll
        for (int i = 0; i < 7; ++i)
          if (i < k) {
            float ls = v[i] - lse;
            ent -= expf(ls) * ls;
          }
        if (p.ent_head) p.ent_head[env * kActHeads + lane] = ent;
      }
    }
    if (p.logprob || p.entropy) {
      lp = warp_sum(lp);
      ent = warp_sum(ent);
      if (lane == 0) {
        if (p.logprob) p.logprob[env] = lp;
        if (p.entropy) p.entropy[env] = ent;
      }
    }
    const float* vr = p.vraw + env * p.ld_v;
    if (p.bins == 1) {       // a scalar value head: the one "bin" is the value itself
      if (lane == 0) {
        const float v = vr[0];
        p.value[env] = v;
        if (p.value_logits) p.value_logits[env] = v;
        if (p.value_buf) p.value_buf[env] = v * (p.ret_sigma ? *p.ret_sigma : 1.f) + (p.ret_mu ? *p.ret_mu : 0.f);
      }
      continue;
    }
    // value = softmax(bins) . centres
    float mx = -INFINITY;
    for (int i = lane; i < p.bins; i += 32) mx = fmaxf(mx, vr[i]);
    mx = warp_max(mx);
    const float step = 2.f * p.vmax / (p.bins - 1);
    float se = 0.f, sc = 0.f;
    for (int i = lane; i < p.bins; i += 32) {
      float l = vr[i];
      float e = expf(l - mx);
      // centres mirror torch.linspace: symmetric evaluation from both ends
      float c = i < p.bins / 2 ? -p.vmax + step * i : p.vmax - step * (p.bins - 1 - i);
      se += e;
      sc += e * c;
      if (p.value_logits) p.value_logits[env * p.bins + i] = l;
    }
    se = warp_sum(se);
    sc = warp_sum(sc);
    if (lane == 0) {
      const float v = sc / se;
      p.value[env] = v;
      // the trainer stores the de-normalised value: b_val[t] = v * ret_sig + ret_mu
      if (p.value_buf) p.value_buf[env] = v * (p.ret_sigma ? *p.ret_sigma : 1.f) + (p.ret_mu ? *p.ret_mu : 0.f);
    }
  }
}
}  // namespace

int head_tail(const HeadTailArgs& a, cudaStream_t stream) {
  if (!a.raw || !a.vraw || !a.value) {
    set_error("head_tail: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (a.k_max < 3 || a.k_max > 7 || a.bins < 1 || a.n_envs < 0) {
    set_error("head_tail: bad shape k_max=%d bins=%d", a.k_max, a.bins);
    return BSRL_ERR_SHAPE;
  }
  if (a.actions && a.act_dtype != BSRL_U8 && a.act_dtype != BSRL_I32 && a.act_dtype != BSRL_I64) {
    set_error("head_tail: actions must be u8, i32 or i64");
    return BSRL_ERR_UNSUPPORTED;
  }
  if (a.n_envs == 0) return BSRL_OK;
  int64_t blocks = (a.n_envs + 7) / 8;
  int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  head_tail_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  BSRL_LAUNCH_OK("head_tail_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
