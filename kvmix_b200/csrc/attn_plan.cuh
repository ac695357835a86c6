// Work plan of the tensor-core attention kernels: which tokens of which head a CTA scores.
//
// The token axis of every head (a query head, or the group of query heads that share a kv head) is cut into
// units of `unit` tokens (one key tile per warp: 256, or 352 = 4 x 88 for 3-bit keys); a head has
// uph = ceil(T / unit) units, the last one possibly short.  One CTA works one segment = a run of units of one head:
//   * the first n_whole CTAs take one whole head each (only when a head fits the score buffer); n_whole is a multiple
//     of the resident-CTA slots of the GPU, so these CTAs fill whole waves;
//   * every remaining head (n_cut of them) is cut into k segments of seg_units units (the last one shorter), launched
//     after the whole heads, first segments of all heads first.  k is chosen so that these smaller CTAs, which the
//     hardware hands to whichever slot frees up, finish as early as possible: the last wave of a grid is then made of
//     short CTAs and fills all slots, whatever the number of heads.
// A head cut into several segments is merged by the CTA that finishes last (per-head counter), in segment order, so
// results do not depend on timing.
#pragma once
#include <stdint.h>

namespace kvq {

struct AttnPlan {
    int unit;            // tokens per unit
    int uph;             // units per head
    int n_whole;         // CTAs (= heads) that take a whole head
    int n_cut;           // heads that are cut
    int k;               // segments per cut head (1: a whole head per CTA here too)
    int seg_units;       // units per segment of a cut head
    int n_scores;        // most tokens in a segment, rounded up to 32
};

constexpr int kSmCount = 148;
// One partial result of a cut head: 128 accumulators, the segment's maximum and sum, padded so that rows stay 16-byte
// aligned (the merge reads them with 128-bit loads).
constexpr int kPartStride = 128 + 4;
// What merging one more segment costs the CTA that finishes last, in tokens' worth of time.
constexpr int kMergeTokensPerSegment = 4;
// A CTA costs about this many tokens' worth of time besides the tokens it scores (launch, ring fill of two phases,
// softmax barriers, warps that get one key tile fewer than their neighbours, merge).  Measured on B200 with 2-bit
// keys and values at 4096 tokens: 256 heads take 54 us whole, 60 .. 66 us cut in 2 .. 4 (more CTAs than resident
// slots), and cutting the 272 heads beyond four full waves of a 2048-head launch costs 1 .. 9 % -- so heads are cut
// only where the score buffer forces it or where whole heads would leave most slots empty.
constexpr int kCtaOverheadTokens = 2048;
constexpr int kMaxCtaRounds = 8;       // cut heads are never spread over more CTAs than this many waves (bounds the workspace)

// heads: number of heads (or head groups); max_chunk: most tokens a segment may hold (score buffer); slots: resident
// CTAs on the whole GPU.
// units_per_pass: units the warps of a CTA work side by side (4 when a unit is one warp's key tile, 1 when a unit is
// already a tile per warp): a segment takes as long as its units rounded up to that.
inline AttnPlan make_attn_plan(int T, int unit, int max_chunk, long long heads, int slots, int units_per_pass = 1) {
    AttnPlan p;
    p.unit = unit;
    p.uph = (T + unit - 1) / unit;
    const bool whole_ok = T <= max_chunk;
    p.n_whole = (int)(whole_ok ? (heads / slots) * slots : 0);
    p.n_cut = (int)(heads - p.n_whole);
    p.k = 1;
    p.seg_units = p.uph;
    if (p.n_cut > 0) {
        // candidates: segments of su units; estimated finish = rounds of CTAs x (tokens + overhead)
        const int su_max = whole_ok ? p.uph : max_chunk / unit;
        long long best = -1;
        for (int su = su_max; su >= 1; --su) {
            const int k = (p.uph + su - 1) / su;
            if (k > 1 && su < 2 && p.uph > 2) break;                           // at least two units per segment
            const long long ctas = (long long)p.n_cut * k;
            if (ctas > (long long)kMaxCtaRounds * slots && best >= 0) break;
            const long long rounds = (ctas + slots - 1) / slots;
            const long long su_eff = (long long)(su + units_per_pass - 1) / units_per_pass * units_per_pass;
            const long long tokens = k > 1 ? su_eff * unit : ((long long)su * unit < T ? (long long)su * unit : T);
            const long long cost = rounds * (tokens + kCtaOverheadTokens) +
                                   (k > 1 ? kCtaOverheadTokens / 4 + (long long)k * kMergeTokensPerSegment : 0);
            if (best < 0 || cost < best) {
                best = cost;
                p.k = k;
                p.seg_units = su;
            }
        }
        p.seg_units = (p.uph + p.k - 1) / p.k;                                   // even the segments out
        p.k = (p.uph + p.seg_units - 1) / p.seg_units;
    }
    long long ns = (long long)(p.n_whole ? p.uph : p.seg_units) * unit;
    if (ns > T) ns = T;
    p.n_scores = (int)((ns + 31) / 32 * 32);
    return p;
}

// CTA index -> (head, segment): whole heads first, then the cut heads segment-major (all first segments, then all
// second segments, ...), so the shortest segments -- the last of each head -- come last.
__host__ __device__ inline void plan_cta(const AttnPlan &p, int T, int c, int &head, int &t0, int &t1, int &seg, int &cnt) {
    if (c < p.n_whole) {
        head = c; t0 = 0; t1 = T; seg = 0; cnt = 1;
        return;
    }
    const int cc = c - p.n_whole;
    seg = cc / p.n_cut;
    head = p.n_whole + cc - seg * p.n_cut;
    cnt = p.k;
    t0 = seg * p.seg_units * p.unit;
    const int e = t0 + p.seg_units * p.unit;
    t1 = e < T ? e : T;
}

}  // namespace kvq
