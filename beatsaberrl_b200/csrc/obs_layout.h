// Observation lane routing of the five lead tokens, as (first lane, count) runs.
//
// Facts of the reference's obs contract (python/policy.py:174-275): 630 lanes; 24 entity
// slots of 18 lanes at 102..533, their live mask at 534..557.  Each lead token reads the runs
// below in order; the saber and leg tokens then get a 2-lane hand / side one-hot.
#pragma once
#include <stdint.h>

namespace bsrl {

struct LaneRun {
  int16_t first, count;
};

constexpr int kOffNotes = 102;
constexpr int kNoteFeat = 18;
constexpr int kOffMask = 534;
constexpr int kObsHeadZ = 99;
constexpr int kGeoFeat = 22;
constexpr int kSaberFeat = 47, kTorsoFeat = 29, kLegFeat = 32;
constexpr int kMaxRuns = 9;

// token order: saber_L, saber_R, torso, leg_L, leg_R
constexpr LaneRun kTokenRuns[5][kMaxRuns] = {
    // arm q, arm qd, hand block, elbow position, elbow velocity, previous note, arm torque scales, blade tip
    {{18, 8}, {49, 7}, {75, 11}, {562, 3}, {580, 3}, {598, 5}, {611, 7}, {624, 3}, {0, 0}},
    {{26, 8}, {56, 7}, {86, 11}, {565, 3}, {583, 3}, {603, 5}, {611, 7}, {627, 3}, {0, 0}},
    // root + spine q, spine qd, head + contact bits, spine torque scales
    {{0, 18}, {46, 3}, {97, 5}, {608, 3}, {0, 0}, {0, 0}, {0, 0}, {0, 0}, {0, 0}},
    // leg q, leg qd, heel/toe contact, knee pos, foot pos, knee vel, foot vel, leg torque scales
    {{34, 6}, {63, 6}, {558, 2}, {568, 3}, {574, 3}, {586, 3}, {592, 3}, {618, 6}, {0, 0}},
    {{40, 6}, {69, 6}, {560, 2}, {571, 3}, {577, 3}, {589, 3}, {595, 3}, {618, 6}, {0, 0}},
};
constexpr int kTokenFeat[5] = {kSaberFeat, kSaberFeat, kTorsoFeat, kLegFeat, kLegFeat};
// one-hot lane appended after the obs lanes (-1 = none): hand / side id
constexpr int kTokenOneHot[5] = {0, 1, -1, 0, 1};

// obs lane of feature k of lead token tok, or -1 past the obs-fed lanes
constexpr int token_lane(int tok, int k) {
  for (int r = 0; r < kMaxRuns; ++r) {
    if (k < kTokenRuns[tok][r].count) return kTokenRuns[tok][r].first + k;
    k -= kTokenRuns[tok][r].count;
  }
  return -1;
}

// K-padded widths of the first encoder layers: one 64-wide k-block each, so that all of them run on
// the tcgen05 GEMM (the warp-MMA kernel it would otherwise fall back to is several times slower here)
constexpr int kSaberK = 64, kTorsoK = 64, kLegK = 64;
constexpr int note_k(bool) { return 64; }

}  // namespace bsrl
