// Tokenizer: one obs row (630 lanes) -> fp16 input rows of the four token encoders + key bias.
//
// One warp per environment.  The obs row is staged in shared memory once (coalesced), then
// scattered through a constant lane table into K-padded fp16 rows: 2 saber rows (47 lanes +
// hand one-hot), 1 torso row (29), 2 leg rows (32 + side one-hot), 24 slot rows (18 lanes, plus
// the 22 hand-relative geometry lanes when note_geo is on, computed here in fp32).  Pure
// streaming: 2,520 B read per env, ~2-4 KB written.
//
// Reference: NotePolicy._split (python/policy.py:1099-1105), the one-hot / concat code at
// :1226-1249, _note_geo (:329-404) and the key bias (:1257-1260).
#include "kernels.cuh"
#include "obs_layout.h"

namespace bsrl {
namespace {

struct LaneTable {
  int16_t v[5][64];  // >= 0 obs lane, -1 zero, -2 one
};
constexpr LaneTable make_lane_table() {
  LaneTable t{};
  for (int tok = 0; tok < 5; ++tok)
    for (int k = 0; k < 64; ++k) {
      int lane = token_lane(tok, k);
      int v = lane;
      if (lane < 0) {
        int oh = k - kTokenFeat[tok];
        v = (kTokenOneHot[tok] >= 0 && oh == kTokenOneHot[tok]) ? -2 : -1;
      }
      t.v[tok][k] = static_cast<int16_t>(v);
    }
  return t;
}
__constant__ LaneTable c_lanes = make_lane_table();
constexpr LaneTable h_lanes = make_lane_table();

constexpr int kWarps = 8;

__device__ __forceinline__ float tab(const float* o, int tok, int k) {
  int l = c_lanes.v[tok][k];
  return l >= 0 ? o[l] : (l == -2 ? 1.f : 0.f);
}
// the same through a shared-memory copy of the table, for indices that differ between the lanes of a warp
// (the constant cache serves one address per cycle: 32 lanes with 32 different k take 32 passes)
__device__ __forceinline__ float tab_s(const float* o, const int16_t (*lanes)[64], int tok, int k) {
  int l = lanes[tok][k];
  return l >= 0 ? o[l] : (l == -2 ? 1.f : 0.f);
}

// 22 geometry lanes of one slot: per hand 7, then per hand 4.  flux: a bar slot (lane 9 > 0.5) is aimed
// at lanes 12, 13, where it must be crossed (python/policy.py:357-360).
__device__ void slot_geometry(const float* o, int slot, float z_asinh, bool flux, float* out) {
  const float XN = 1.0f, YN = 0.75f, ZS = 8.0f, VN = 6.0f, HANDLE = 0.16f;
  const float* n = o + kOffNotes + slot * kNoteFeat;
  const float z_m = sinhf(n[2]) * z_asinh;
  const bool bar = flux && n[9] > 0.5f;
  const float px = (bar ? n[12] : n[0]) * XN, py = (bar ? n[13] : n[1]) * YN, pz = z_m;
  const float cx = n[6], cy = n[7];
  const float live = 1.0f - n[14];
  const float speed = fmaxf(-n[3] * ZS, 1e-3f);
  const float zrel = z_m - o[kObsHeadZ] * XN;
  const float tpl = fminf(fmaxf(zrel / speed, -0.5f), 3.0f) / 3.0f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float wx = tab(o, h, 15) * XN, wy = tab(o, h, 16) * YN, wz = tab(o, h, 17);
    const float mx = px - wx, my = py - wy, mz = pz - wz;  // metres
    const float dx = mx * 0.5f, dy = my * 0.5f, dz = mz * 0.5f;
    const float dist = sqrtf(dx * dx + dy * dy + dz * dz);
    const float vx = tab(o, h, 18) * VN, vy = tab(o, h, 19) * VN, vz = tab(o, h, 20) * VN;
    const float vn = sqrtf(vx * vx + vy * vy + vz * vz) + 0.05f;
    const float bx = tab(o, h, 21), by = tab(o, h, 22), bz = tab(o, h, 23);
    float* f = out + h * 7;
    f[0] = dx;
    f[1] = dy;
    f[2] = asinhf(dz * 2.0f / 8.0f);
    f[3] = asinhf(dist * 2.0f / 8.0f);
    f[4] = tpl;
    f[5] = ((vx / vn) * cx + (vy / vn) * cy) * live;
    f[6] = (bx * cx + by * cy) * live;
    const float ab = mx * bx + my * by + mz * bz;
    const float rx = mx - ab * bx, ry = my - ab * by, rz = mz - ab * bz;
    const float tx = tab(o, h, 44), ty = tab(o, h, 45), tz = tab(o, h, 46);
    const float ux = tx * VN, uy = ty * VN, uz = tz * VN;
    const float nx = by * uz - bz * uy, ny = bz * ux - bx * uz, nz = bx * uy - by * ux;
    const float nn = sqrtf(nx * nx + ny * ny + nz * nz) + 0.05f;
    float* s = out + 14 + h * 4;
    s[0] = asinhf((ab - HANDLE) * 0.5f);
    s[1] = asinhf(sqrtf(rx * rx + ry * ry + rz * rz) * 0.5f);
    s[2] = asinhf((mx * (nx / nn) + my * (ny / nn) + mz * (nz / nn)) * 0.5f);
    s[3] = (tx * cx + ty * cy) * live;
  }
}

template <bool OBS_F16>
__global__ void __launch_bounds__(kWarps * 32, 4) embed_gather_kernel(const void* __restrict__ obs_,
                                                                  int64_t n_envs, int note_geo,
                                                                  float z_asinh, EmbedBuffers out) {
  __shared__ float s_obs[kWarps][kObs + 2];
  __shared__ float s_geo[kWarps][kSlots * kGeoFeat];
  __shared__ int16_t s_lanes[5][64];
  static_assert(kSaberK == 64 && kTorsoK == 64 && kLegK == 64 && note_k(true) == 64 && note_k(false) == 64,
                "one lane per feature pair of a 64-wide padded row");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 5 * 64; i += blockDim.x) s_lanes[i >> 6][i & 63] = c_lanes.v[i >> 6][i & 63];
  __syncthreads();
  float* o = s_obs[warp];
  float* geo = s_geo[warp];
  for (int64_t env = (int64_t)blockIdx.x * kWarps + warp; env < n_envs;
       env += (int64_t)gridDim.x * kWarps) {
    __syncwarp();
    if (OBS_F16) {
      const __half* src = static_cast<const __half*>(obs_) + env * kObs;
      for (int i = lane; i < kObs; i += 32) o[i] = __half2float(src[i]);
    } else {
      const float* src = static_cast<const float*>(obs_) + env * kObs;
      for (int i = lane; i < kObs; i += 32) o[i] = src[i];
    }
    __syncwarp();
    if (out.obs16) {   // fp16 copy of the row (b_obs[t] of the rollout buffer, python/train_batch.py:2299)
      uint32_t* d16 = reinterpret_cast<uint32_t*>(out.obs16 + env * kObs);
      for (int i = lane; i < kObs / 2; i += 32) d16[i] = pack_half2(o[2 * i], o[2 * i + 1]);
    }
    if (note_geo && lane < kSlots) slot_geometry(o, lane, z_asinh, (note_geo & 2) != 0, geo + lane * kGeoFeat);
    // lead tokens: lane writes features 2*lane, 2*lane + 1
    {
      const int k = lane * 2;
      uint32_t* d;
      d = reinterpret_cast<uint32_t*>(out.saber + (env * 2 + 0) * kSaberK);
      d[lane] = pack_half2(tab_s(o, s_lanes, 0, k), tab_s(o, s_lanes, 0, k + 1));
      d = reinterpret_cast<uint32_t*>(out.saber + (env * 2 + 1) * kSaberK);
      d[lane] = pack_half2(tab_s(o, s_lanes, 1, k), tab_s(o, s_lanes, 1, k + 1));
      d = reinterpret_cast<uint32_t*>(out.leg + (env * 2 + 0) * kLegK);
      d[lane] = pack_half2(tab_s(o, s_lanes, 3, k), tab_s(o, s_lanes, 3, k + 1));
      d = reinterpret_cast<uint32_t*>(out.leg + (env * 2 + 1) * kLegK);
      d[lane] = pack_half2(tab_s(o, s_lanes, 4, k), tab_s(o, s_lanes, 4, k + 1));
      d = reinterpret_cast<uint32_t*>(out.torso + env * kTorsoK);
      d[lane] = pack_half2(tab_s(o, s_lanes, 2, k), tab_s(o, s_lanes, 2, k + 1));
    }
    __syncwarp();
    // slot rows
    {
      // every slot row is 64 features = one lane per pair: obs lanes, then the geometry lanes, then zeros
      // (the feature counts are even, so a pair never straddles two sources)
      static_assert(kNoteFeat % 2 == 0 && kGeoFeat % 2 == 0, "feature pairs");
      uint32_t* d = reinterpret_cast<uint32_t*>(out.note + env * kSlots * 64);
      const int k = lane * 2;
      const float* src = k < kNoteFeat ? o + kOffNotes + k
                         : (note_geo && k < kNoteFeat + kGeoFeat) ? geo + (k - kNoteFeat) : nullptr;
      const int step = k < kNoteFeat ? kNoteFeat : kGeoFeat;
#pragma unroll 8
      for (int slot = 0; slot < kSlots; ++slot)
        d[slot * 32 + lane] = src ? pack_half2(src[slot * step], src[slot * step + 1]) : 0u;
    }
    if (lane < kT)
      out.key_bias[env * kT + lane] = lane < kLead ? 0.f : (o[kOffMask + lane - kLead] - 1.0f) * kMaskBias;
  }
}
}  // namespace

int token_lane_host(int tok, int k) {
  if (tok < 0 || tok >= 5 || k < 0 || k >= kTokenFeat[tok]) return -1;
  return h_lanes.v[tok][k];
}

int embed_gather(const void* obs, int obs_dtype, int64_t n_envs, int note_geo, int flux, float z_asinh,
                 const EmbedBuffers& out, cudaStream_t stream) {
  if (!obs || !out.saber || !out.torso || !out.leg || !out.note || !out.key_bias) {
    set_error("embed: NULL operand");
    return BSRL_ERR_NULL;
  }
  if (obs_dtype != BSRL_F32 && obs_dtype != BSRL_F16) {
    set_error("embed: obs must be f32 or f16");
    return BSRL_ERR_UNSUPPORTED;
  }
  if (out.ks != kSaberK || out.kl != kLegK || out.kt != kTorsoK || out.kn != note_k(note_geo != 0)) {
    set_error("embed: feature pitches do not match the encoder layout");
    return BSRL_ERR_SHAPE;
  }
  if (n_envs <= 0) return n_envs == 0 ? BSRL_OK : BSRL_ERR_SHAPE;
  note_geo = note_geo ? (flux ? 3 : 1) : 0;   // bit 1 tells the kernel to use the Flux variant
  int64_t blocks = (n_envs + kWarps - 1) / kWarps;
  int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (obs_dtype == BSRL_F16)
    embed_gather_kernel<true><<<static_cast<unsigned>(blocks), kWarps * 32, 0, stream>>>(
        obs, n_envs, note_geo, z_asinh, out);
  else
    embed_gather_kernel<false><<<static_cast<unsigned>(blocks), kWarps * 32, 0, stream>>>(
        obs, n_envs, note_geo, z_asinh, out);
  BSRL_LAUNCH_OK("embed_gather_kernel");
  return BSRL_OK;
}

}  // namespace bsrl
