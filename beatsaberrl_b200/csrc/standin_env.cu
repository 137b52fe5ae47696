// Stand-in for the simulator's per-tick step kernel, for graph-capture tests and tick benchmarks.
//
// The real environment step (step_kernel, python/beat_arena_env/csrc/beat_arena_cuda.cu:6188-6245) is a
// sibling of the policy forward, not part of it: per env it consumes the 29 sampled gear ids, advances
// the simulation and rewrites the env's 630-lane observation row, reward and done flag IN PLACE in
// preallocated buffers -- which is all a captured rollout graph needs from it
// (python/rollout_graph.py:45-74).  This kernel has exactly that memory behaviour and none of the
// physics: the next observation is a deterministic hash of (env state, lane) shifted by the actions,
// clipped to +-5 like the synthetic benchmark inputs, with the 24 slot-mask lanes set to 0 or 1.
#include "kernels.cuh"
#include "obs_layout.h"

namespace bsrl {
namespace {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

// one warp per env
__global__ void __launch_bounds__(256) standin_step_kernel(const long long* __restrict__ actions, int64_t n_envs,
                                                           uint32_t* __restrict__ state, float* __restrict__ obs,
                                                           float* __restrict__ reward, unsigned char* __restrict__ done) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t env = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); env < n_envs; env += warps) {
    int a = lane < kActHeads ? (int)actions[env * kActHeads + lane] : 0;
    const int a_sum = (int)warp_sum((float)a);
    const uint32_t st = state[env] * 1664525u + 1013904223u + (uint32_t)a_sum;
    float* row = obs + env * kObs;
    for (int c = lane; c < kObs; c += 32) {
      const uint32_t h = mix32(st ^ (uint32_t)(c * 0x9E3779B9u));
      float v;
      if (c >= kOffMask && c < kOffMask + kSlots) {
        v = (h & 3u) ? 1.f : 0.f;                       // three slots in four are live
      } else {
        // sum of four uniform bytes, centred and scaled to unit variance, nudged by the action it belongs to
        const float u = (float)((h & 255u) + ((h >> 8) & 255u) + ((h >> 16) & 255u) + (h >> 24)) - 510.f;
        v = u * (1.f / 147.8f) + 0.05f * (float)(__shfl_sync(0xffffffffu, a, c % kActHeads) - 2);
        v = fminf(fmaxf(v, -5.f), 5.f);
      }
      row[c] = v;
    }
    if (lane == 0) {
      state[env] = st;
      if (reward) reward[env] = (float)a_sum * (1.f / (4.f * kActHeads));
      if (done) done[env] = (st >> 26) == 0u;           // about one tick in 64
    }
  }
}
}  // namespace

int standin_env_step(const long long* actions, int64_t n_envs, uint32_t* state, float* obs, float* reward,
                     unsigned char* done, cudaStream_t stream) {
  if (!actions || !state || !obs) {
    set_error("standin_env_step: NULL actions / state / obs");
    return BSRL_ERR_NULL;
  }
  if (n_envs < 0) {
    set_error("standin_env_step: n_envs %lld is negative", (long long)n_envs);
    return BSRL_ERR_SHAPE;
  }
  if (n_envs == 0) return BSRL_OK;
  int64_t blocks = (n_envs + 7) / 8;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  standin_step_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(actions, n_envs, state, obs, reward, done);
  BSRL_LAUNCH_OK("standin_step_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
