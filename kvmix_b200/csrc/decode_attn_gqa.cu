// Fused decode attention for grouped-query models, tensor-core path: one CTA (4 warps) serves up to FOUR query heads
// that share a kv head, so every packed code is fetched, unpacked and fed to the tensor core once for all of them.
//
// Same formulation as decode_attn_mma.cu (codes reach mma.sync as fp16 subnormals, q*scale carried as an exact
// fp16 pair hi + lo, per-warp cp.async rings); what changes is the meaning of the eight B columns:
//   keys    column 2h / 2h+1 = hi / lo of q_h[d] * scale[d, group] for query head h of the quad.  An MMA's 16 token
//           rows therefore have to lie in ONE scale group: 1-, 2- and 4-bit keys are all fetched with transposing
//           ldmatrix loads (a 16-byte block of a channel row = 128 / 64 / 32 tokens; needs k_group >= that), and
//           3-bit keys (group 11 = one word) put the 11 tokens of a word in the rows of an MMA, extracting field g with a
//           per-lane byte permute and mask.  The zero terms sum_d q_h[d] * zero[d, group] of all groups of a tile come
//           from one MMA per 16 channels: the zero tile in shared memory ([channel][group]) read transposed is the A
//           operand (row = group), q the B operand.
//   values  column 2h / 2h+1 = p_h[t] * scale[t, group] / p_h[t] * midpoint[t, group]; an MMA's 16 channel rows lie
//           in one channel group (a 16-byte block of a token row = 128 / 64 / 32 channels; needs v_group >= that --
//           except 1-bit values at group 64, where a block spans two groups and every code tile is multiplied by both
//           groups' operands, each lane keeping the product of the group its rows belong to).
// Scores of the four heads sit side by side in shared memory ([4][n]); warp w runs the softmax of head w.
#include "attn_mma_common.cuh"
#include "attn_plan.cuh"
#include "attn_update.cuh"

namespace kvq {

constexpr int kQH = 4;                  // query-head slots per CTA
constexpr int kGqaMaxChunk = 2048;      // tokens per segment: 4 x 2048 fp32 scores (3072 fit too but measured 10 % slower)
constexpr int kGqaTailOff = 2048;       // per-warp region: [value ring | operand tiles (2 KB) | fp16-tail partial (2 KB)]

struct GqaSmem {
    float *scores;          // [kQH][n_scores]
    unsigned char *ring;    // this warp's region
    __half *q;              // [kQH][kHeadDim]
    float *misc;            // [64]
    int n_scores;
};

// Scale/zero tiles of a key warp tile are double-buffered (the operands are formed k-step by k-step, so a tile's
// scales stay in use until its last stage).  3-bit keys: 8 groups per tile, a [128][16 B] scale tile followed by the
// zero tile; other widths (<= 4 groups per tile): one [128][16 B] tile whose rows hold 4 scales then 4 zeros.
template <int KB> constexpr int gqa_sz_bytes() { return KB == 3 ? 4096 : 2048; }
template <int KB> constexpr int gqa_zero_off() { return KB == 3 ? 2048 : 8; }

template <int KB, int VB> constexpr int gqa_region_bytes() {
    constexpr int k = KGeom<KB>::NS * KGeom<KB>::STAGE_BYTES + 2 * gqa_sz_bytes<KB>();
    constexpr int v = VGeom<VB>::NS * VGeom<VB>::STAGE_BYTES + kGqaTailOff + kQH * kHeadDim * 4;
    return k > v ? k : v;
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// hi / lo part of the exact product q * s for a pair of channels: even columns carry hi = rn(q * s), odd columns
// lo = q * s - hi (exact in fp16).  neg_mask is 0 in even-column lanes and all ones in odd-column lanes:
// fma(q, s, +0) = hi, fma(q, s, -hi) = lo.
__device__ __forceinline__ uint32_t hilo(__half2 q, __half2 s, uint32_t neg_mask) {
    const uint32_t hi = as_u32(__hmul2(q, s));
    return as_u32(__hfma2(q, s, as_h2((hi ^ 0x80008000u) & neg_mask)));
}

// ---------------------------------------------------------------------------------------------
// fp16 key tail for tokens [lo, t1): 16-token tiles straight from global memory; B column n = query head n.
__device__ __forceinline__ void gqa_qk_tail(const kvq_attn_args &a, const __half *kf, int b, int hk, const GqaSmem &sm,
                                            int t0, int lo, int t1) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    uint4 qf[4];
#pragma unroll
    for (int S = 0; S < 4; ++S)
        qf[S] = g < kQH ? *reinterpret_cast<const uint4 *>(sm.q + g * kHeadDim + 32 * S + 8 * tig) : make_uint4(0u, 0u, 0u, 0u);
    const int n_tiles = (t1 - lo + 15) / 16;
    for (int tile = warp; tile < n_tiles; tile += kMmaWarps) {
        const int ta = lo + 16 * tile + g, tb = ta + 8;
        const __half *pa = k_tail_row(a, kf, b, hk, min(ta, t1 - 1)) + 8 * tig;
        const __half *pb = k_tail_row(a, kf, b, hk, min(tb, t1 - 1)) + 8 * tig;
        uint4 ra[4], rb[4];
#pragma unroll
        for (int S = 0; S < 4; ++S) {
            ra[S] = __ldg(reinterpret_cast<const uint4 *>(pa + 32 * S));
            rb[S] = __ldg(reinterpret_cast<const uint4 *>(pb + 32 * S));
        }
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int S = 0; S < 4; ++S) {
            mma16816(c, ra[S].x, rb[S].x, ra[S].y, rb[S].y, qf[S].x, qf[S].y);
            mma16816(c, ra[S].z, rb[S].z, ra[S].w, rb[S].w, qf[S].z, qf[S].w);
        }
        if (tig < 2) {                                         // columns 2 tig, 2 tig + 1 = heads 2 tig, 2 tig + 1
            if (a.round_scores) {
                const float2 r0 = __half22float2(__floats2half2_rn(c[0], c[1])), r1 = __half22float2(__floats2half2_rn(c[2], c[3]));
                c[0] = r0.x; c[1] = r0.y; c[2] = r1.x; c[3] = r1.y;
            }
            float *d0 = sm.scores + (2 * tig) * sm.n_scores, *d1 = d0 + sm.n_scores;
            if (ta < t1) { d0[ta - t0] = c[0] * a.softmax_scale; d1[ta - t0] = c[1] * a.softmax_scale; }
            if (tb < t1) { d0[tb - t0] = c[2] * a.softmax_scale; d1[tb - t0] = c[3] * a.softmax_scale; }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// q . K^T over packed keys, tokens [t0, hi), for the four heads of the quad.  Same ring and stage geometry as the
// single-head kernel (KGeom); scores[h][t - t0] receive the scaled scores.
template <int KB>
__device__ __forceinline__ void gqa_qk_packed(const kvq_attn_args &a, const int32_t *kc, const __half *ks,
                                              const __half *kz, const GqaSmem &sm, int t0, int hi, const __half *kf,
                                              int tail_lo, int t1, int b, int hk) {
    using G = KGeom<KB>;
    using F = Fields<KB>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const int Gk = a.k_group;
    const int n_words = a.Tkq / G::FPI;
    const int n_tiles = (hi - t0 + G::WT - 1) / G::WT;
    const int my_tiles = (n_tiles - warp + kMmaWarps - 1) / kMmaWarps;
    if (my_tiles <= 0) {
        __syncthreads();                                       // q is in shared memory
        if (tail_lo < t1) gqa_qk_tail(a, kf, b, hk, sm, t0, tail_lo, t1);
        return;
    }
    const int kc_sD = (int)a.kc_sD, ks_sD = (int)a.ks_sD;
    const uint32_t ring_s = smem_u32(sm.ring);
    const uint32_t sz_s = ring_s + G::NS * G::STAGE_BYTES;                    // two scale/zero tile buffers
    constexpr int SZB = gqa_sz_bytes<KB>(), ZOFF = gqa_zero_off<KB>();
    const int gr = lane % G::GPR, row0 = lane / G::GPR;
    const uint32_t cp_dst = ring_s + row0 * G::RS + gr * 16;
    constexpr int FH = (KB == 3) ? 2 : 16 / KB;                                // fields per half-word: 4 / 8 / 16
    constexpr int NBK = G::RB / 16;                                            // 16-byte blocks per channel row: 8 / 4 / 2
    constexpr int MPB = FH / 2;                                                // MMAs per block and k-step: 2 / 4 / 8
    constexpr int NACC = (KB == 3) ? 8 : NBK * MPB;                            // accumulators per tile: 8 words / 16 token pairs
    const uint32_t ldk_s = ring_s + ((lane & 7) + 8 * ((lane >> 3) & 1)) * G::RS + (lane >> 4) * 16;
    const uint32_t w3_s = ring_s + (2 * tig) * G::RS;                          // 3-bit: word rows 2 tig, +1, +8, +9
    const uint32_t szrow_s = sz_s + (2 * tig) * 16;                            // + buffer + 256 ksx [+16 | +128 | +144] [+ZOFF zero]
    const uint32_t q_s = smem_u32(sm.q) + (g >> 1) * (kHeadDim * 2) + (2 * tig) * 2;   // this column's head; + 32 ksx [+16]
    const uint32_t neg_mask = (g & 1) ? 0xffffffffu : 0u;
    const int ngw = (G::WT + Gk - 1) / Gk;                                     // groups per warp tile: 8 (3-bit) / 4 / 2
    const bool wide = Gk >= 128;                                               // 128-token groups (else 64)
    const uint32_t szcp_dst = sz_s + lane * 16;
    const int tile_words = kMmaWarps * G::WT / G::FPI;
    const int tile_groups = kMmaWarps * G::WT / Gk;
    // 3-bit keys: field g of a word sits at bits 3g..3g+2; one byte permute brings the two bytes that hold it (of both
    // channel words) into the 16-bit halves, a mask isolates it in place at bit p0 = 3g mod 8 (<= 7: linear fp16 range).
    // Fields 8..10 (rows g + 8, g < 3) sit in byte 3 at bits 0, 3, 6 (the last one 2 bits wide).
    const int byte0 = (3 * g) >> 3, p0 = 3 * g - 8 * byte0;
    const uint32_t sel0 = (uint32_t)(byte0 | ((byte0 + 1) << 4) | ((4 + byte0) << 8) | ((5 + byte0) << 12));
    const uint32_t msk0 = 0x00070007u << p0;
    const uint32_t sel1 = 0x7733u;
    const uint32_t msk1 = g == 0 ? 0x00070007u : g == 1 ? 0x00380038u : g == 2 ? 0x00c000c0u : 0u;
    const int p1 = 3 * (g < 3 ? g : 0);
    const float sc0 = __int_as_float((151 - p0) << 23), sc1 = __int_as_float((151 - p1) << 23);   // 2^(24 - position)

    const int32_t *tb_cur = kc + (int64_t)row0 * kc_sD + (t0 + warp * G::WT) / G::FPI + 4 * gr;
    const __half *ks_cur = ks + (int64_t)lane * ks_sD + (t0 + warp * G::WT) / Gk;
    const __half *kz_cur = kz + (int64_t)lane * ks_sD + (t0 + warp * G::WT) / Gk;
    int wcol_cur = (t0 + warp * G::WT) / G::FPI + 4 * gr;
    bool ok_cur = wcol_cur < n_words;

    auto issue_stage = [&](const int32_t *tb, bool ok, int sst) {
        if (ok) {
            const uint32_t dst = cp_dst + (sst % G::NS) * G::STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < G::GPL; ++i)
                cp_async<16>(dst + i * G::RPI * G::RS, tb + (sst * G::ROWS + i * G::RPI) * kc_sD);
        }
    };
    auto issue_sz = [&](const __half *ps, const __half *pz, uint32_t buf) {    // channel rows lane, lane + 32, ...
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int off = 32 * i * ks_sD;
            const uint32_t d = szcp_dst + buf + i * 512;
            if (KB == 3) { cp_async<16>(d, ps + off); cp_async<16>(d + ZOFF, pz + off); }
            else if (ngw == 4) { cp_async<8>(d, ps + off); cp_async<8>(d + ZOFF, pz + off); }
            else { cp_async<4>(d, ps + off); cp_async<4>(d + ZOFF, pz + off); }
        }
    };

    issue_sz(ks_cur, kz_cur, 0u);
    issue_stage(tb_cur, ok_cur, 0);
    cp_async_commit();
    issue_stage(tb_cur, ok_cur, 1);
    cp_async_commit();
    issue_stage(tb_cur, ok_cur, 2);
    cp_async_commit();
    __syncthreads();                                           // q is in shared memory (stored by the caller without a barrier)
    if (tail_lo < t1) gqa_qk_tail(a, kf, b, hk, sm, t0, tail_lo, t1);

    for (int j = 0; j < my_tiles; ++j) {
        const int tile0 = t0 + (j * kMmaWarps + warp) * G::WT;
        const bool have_next = j + 1 < my_tiles;
        const int32_t *tb_nxt = tb_cur + tile_words;
        const bool ok_nxt = have_next && (wcol_cur + tile_words < n_words);

        const uint32_t szbuf = (j & 1) ? SZB : 0u;
        // groups of this tile that hold tokens below hi: operands of the others are never formed (their scale/zero
        // words lie beyond the packed prefix and may hold anything, and 0 * NaN would poison a shared accumulator)
        const int nvg = min(ngw, (hi - tile0 + Gk - 1) / Gk);
        // the zero-term MMAs (one per k-step) rotate over four accumulators so that consecutive ones do not wait for each other
        float acc[NACC][4], accz[4][4];
#pragma unroll
        for (int m = 0; m < NACC; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
#pragma unroll
        for (int m = 0; m < 4; ++m) accz[m][0] = accz[m][1] = accz[m][2] = accz[m][3] = 0.f;

#pragma unroll
        for (int st = 0; st < G::NSTAGE; ++st) {
            if (st + G::P < G::NSTAGE) {
                issue_stage(tb_cur, ok_cur, st + G::P);
            } else {
                issue_stage(tb_nxt, ok_nxt, st + G::P - G::NSTAGE);
            }
            // the next tile's scale/zero tile goes to the other buffer (last read one tile ago)
            if (st == 0 && have_next) issue_sz(ks_cur + tile_groups, kz_cur + tile_groups, szbuf ^ SZB);
            cp_async_commit();
            cp_async_wait<G::P>();                             // stage st has landed (this tile's scale/zero tile long before)
            __syncwarp();
            const uint32_t stage_s = (st % G::NS) * G::STAGE_BYTES;
#pragma unroll
            for (int k = 0; k < G::KSPS; ++k) {
                const int ksx = st * G::KSPS + k;
                const uint32_t q01u = lds32(q_s + 32 * ksx), q89u = lds32(q_s + 32 * ksx + 16);
                const __half2 q01 = as_h2(q01u), q89 = as_h2(q89u);
                const uint32_t zrow = szrow_s + szbuf + 256 * ksx;   // scale rows 16 ksx + 2 tig (+1, +8, +9); zeros + ZOFF
                if constexpr (KB == 3) {
                    // every word is its own group: per word j one B operand and one code MMA (rows = its 11 tokens); words
                    // are taken in pairs so that scales arrive as 32-bit loads.  The zero terms sum_d q[d] * zero[d, j] of
                    // all eight words come from ONE MMA per k-step: the zero tile ([channel][word], 16 bytes per channel)
                    // read transposed is an A operand with row = word and k = channel, B = q in the even columns
                    // (fp16 x fp16 products are exact in the tensor core, so no hi / lo split is needed here); a word
                    // beyond the packed prefix only spoils its own row, which nothing reads
                    {
                        uint32_t za0, za2;
                        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                                     : "=r"(za0), "=r"(za2) : "r"(sz_s + szbuf + ZOFF + (16 * ksx + (lane & 15)) * 16));
                        mma16816(accz[ksx & 3], za0, 0u, za2, 0u, q01u & ~neg_mask, q89u & ~neg_mask);
                    }
#pragma unroll
                    for (int jp = 0; jp < 4; ++jp) {
                        uint32_t sA = lds32(zrow + 4 * jp), sB = lds32(zrow + 16 + 4 * jp);
                        uint32_t sC = lds32(zrow + 128 + 4 * jp), sD = lds32(zrow + 144 + 4 * jp);
                        const uint32_t src = w3_s + stage_s + (k * 16) * G::RS + 8 * jp;
                        const uint2 wA = lds64(src), wB = lds64(src + G::RS), wC = lds64(src + 8 * G::RS), wD = lds64(src + 9 * G::RS);
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int jw = 2 * jp + u;
                            if (jw >= nvg) continue;
                            const uint32_t psel = u ? 0x7632u : 0x5410u;
                            const __half2 s01 = as_h2(prmt(sA, sB, psel)), s89 = as_h2(prmt(sC, sD, psel));
                            const uint32_t a_lo = u ? wA.y : wA.x, b_lo = u ? wB.y : wB.x, a_hi = u ? wC.y : wC.x, b_hi = u ? wD.y : wD.x;
                            mma16816(acc[jw], prmt(a_lo, b_lo, sel0) & msk0, prmt(a_lo, b_lo, sel1) & msk1,
                                     prmt(a_hi, b_hi, sel0) & msk0, prmt(a_hi, b_hi, sel1) & msk1,
                                     hilo(q01, s01, neg_mask), hilo(q89, s89, neg_mask));
                        }
                    }
                } else {
                    // The zero terms sum_d q[d] * zero[d, j] of the tile's groups: one MMA per k-step whose A operand is the
                    // scale/zero tile read transposed (a channel's 16-byte row holds 4 scales then 4 zeros, so rows 4..7
                    // of the product are the zero terms of groups 0..3; rows 0..3 are not used) and whose B operand is
                    // q in the even columns (fp16 x fp16 is exact in the tensor core).  A group beyond the packed prefix
                    // only spoils its own row, which nothing reads.
                    {
                        uint32_t za0, za2;
                        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                                     : "=r"(za0), "=r"(za2) : "r"(sz_s + szbuf + (16 * ksx + (lane & 15)) * 16));
                        mma16816(accz[ksx & 3], za0, 0u, za2, 0u, q01u & ~neg_mask, q89u & ~neg_mask);
                    }
                    // B operands of the tile's groups (<= 4: k_group >= 64)
                    const uint2 sA = lds64(zrow), sB = lds64(zrow + 16), sC = lds64(zrow + 128), sD = lds64(zrow + 144);
                    uint32_t b[4][2];
#pragma unroll
                    for (int jk = 0; jk < 4; ++jk) {
                        if (jk < nvg) {
                            const uint32_t psel = (jk & 1) ? 0x7632u : 0x5410u;
                            const uint32_t a0 = (jk & 2) ? sA.y : sA.x, a1 = (jk & 2) ? sB.y : sB.x, a2 = (jk & 2) ? sC.y : sC.x, a3 = (jk & 2) ? sD.y : sD.x;
                            b[jk][0] = hilo(q01, as_h2(prmt(a0, a1, psel)), neg_mask);
                            b[jk][1] = hilo(q89, as_h2(prmt(a2, a3, psel)), neg_mask);
                        } else {
                            b[jk][0] = b[jk][1] = 0u;
                        }
                    }
                    using H = KHalf<KB>;
                    const uint32_t lsrc = ldk_s + stage_s + (k * 16) * G::RS;
#pragma unroll
                    for (int pb2 = 0; pb2 < NBK / 2; ++pb2) {
                        uint32_t x[2][2];
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                                     : "=r"(x[0][0]), "=r"(x[0][1]), "=r"(x[1][0]), "=r"(x[1][1]) : "r"(lsrc + pb2 * 32));
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int bb = 2 * pb2 + u;
                            uint32_t rlo[H::N], rhi[H::N];
                            H::unpack(x[u][0], rlo);
                            H::unpack(x[u][1], rhi);
                            // the block's group inside the tile: k_group is 64 or 128 here
                            const int j64 = (bb * 8 * FH) / 64, j128 = (bb * 8 * FH) / 128;
                            const uint32_t bx = wide ? b[j128][0] : b[j64][0], by = wide ? b[j128][1] : b[j64][1];
#pragma unroll
                            for (int i = 0; i < H::N; i += 2)
                                mma16816(acc[bb * MPB + i / 2], rlo[i], rlo[i + 1], rhi[i], rhi[i + 1], bx, by);
                        }
                    }
                }
            }
            __syncwarp();                                      // slot st % NS may be refilled
        }

        // ---- epilogue: lane (g, tig) holds, per accumulator, row g / g + 8 of head tig as (hi, lo) ------------
        // row g = group g of the tile: its zero term for head tig (hi + lo columns, summed over the rotating accumulators)
        const float zsum = ((accz[0][0] + accz[0][1]) + (accz[1][0] + accz[1][1])) + ((accz[2][0] + accz[2][1]) + (accz[3][0] + accz[3][1]));
        float *dst_h = sm.scores + tig * sm.n_scores - t0;
        if constexpr (KB == 3) {
#pragma unroll
            for (int jw = 0; jw < 8; ++jw) {
                const float corr = __shfl_sync(0xffffffffu, zsum, 4 * jw + tig);
                const int ta = tile0 + 11 * jw + g, tb = ta + 8;
                float s0 = fmaf(acc[jw][0] + acc[jw][1], sc0, corr);
                float s1 = fmaf(acc[jw][2] + acc[jw][3], sc1, corr);
                if (a.round_scores) {
                    const float2 r = __half22float2(__floats2half2_rn(s0, s1));
                    s0 = r.x;
                    s1 = r.y;
                }
                if (11 * jw + tile0 < hi) {                    // words are whole or absent (hi is a group multiple)
                    dst_h[ta] = s0 * a.softmax_scale;
                    if (g < 3) dst_h[tb] = s1 * a.softmax_scale;
                }
            }
        } else {
            float zj[4];
#pragma unroll
            for (int jk = 0; jk < 4; ++jk) zj[jk] = __shfl_sync(0xffffffffu, zsum, 4 * (4 + jk) + tig);   // rows 4..7
#pragma unroll
            for (int bb = 0; bb < NBK; ++bb) {
                const float corr = wide ? zj[(bb * 8 * FH) / 128] : zj[(bb * 8 * FH) / 64];
                const int tok0 = tile0 + bb * 8 * FH + g * FH;
                if (tok0 < hi) {                               // FH-token chunks are whole or absent (hi is a group multiple)
                    float *dst = dst_h + tok0;
#pragma unroll
                    for (int ip = 0; ip < MPB; ++ip) {
                        const int m = bb * MPB + ip;
                        float s0 = fmaf(acc[m][0] + acc[m][1], (float)(1 << (24 - F::pos(2 * ip))), corr);
                        float s1 = fmaf(acc[m][2] + acc[m][3], (float)(1 << (24 - F::pos(2 * ip + 1))), corr);
                        if (a.round_scores) {
                            const float2 r = __half22float2(__floats2half2_rn(s0, s1));
                            s0 = r.x;
                            s1 = r.y;
                        }
                        *reinterpret_cast<float2 *>(dst + 2 * ip) = make_float2(s0 * a.softmax_scale, s1 * a.softmax_scale);
                    }
                }
            }
        }
        tb_cur = tb_nxt;
        ok_cur = ok_nxt;
        wcol_cur += tile_words;
        ks_cur += tile_groups;
        kz_cur += tile_groups;
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// p . V over packed values for tokens [t0, hi), (hi - t0) % 32 == 0, for the four heads.  scores[h] hold p_h.  Leaves
// this warp's partial sums float[kQH][128] at the base of its region.  MODE as in the single-head kernel.
template <int VB, int MODE>
__device__ __forceinline__ void gqa_pv_packed(const kvq_attn_args &a, const int32_t *vc, const __half *vs,
                                              const __half *vz, const GqaSmem &sm, int t0, int hi) {
    using G = VGeom<VB>;
    using F = VHalf<VB>;
    constexpr int NB = G::GPT;                                // 16-byte blocks per token row: 1 / 2 / 4
    constexpr int CPB = kHeadDim / NB;                        // channels per block: 128 / 64 / 32
    constexpr int MPB = F::N / 2;                             // MMAs per block: 8 / 4 / 2
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const int Gv = a.v_group;
    const int ngv = kHeadDim / Gv;                            // channel groups: 4 / 2 / 1
    const int n_blocks = (hi - t0 + G::TPS - 1) / G::TPS;
    const int my_blocks = (n_blocks - warp + kMmaWarps - 1) / kMmaWarps;
    float *my_red = reinterpret_cast<float *>(sm.ring);
    if (my_blocks <= 0) {
        if (MODE != 1)
            for (int i = lane; i < kQH * kHeadDim; i += 32) my_red[i] = 0.f;
        return;
    }
    const uint32_t ring_s = smem_u32(sm.ring);
    const uint32_t pb_s = ring_s + G::NS * G::STAGE_BYTES;                               // operand tiles [ngv][16 pairs][8 cols]
    const int cp_tl0 = lane / G::GPT, cp_gr = lane % G::GPT;
    auto swz = [](int tl) { return (VB == 4) ? ((tl >> 1) & 3) : (VB == 2) ? ((tl >> 2) & 1) : 0; };
    const int cp_grs = cp_gr ^ swz(cp_tl0);
    const uint32_t cp_dst = ring_s + cp_tl0 * G::RBV + cp_grs * 16;
    const int ldm_tl = 8 * ((lane >> 3) & 1) + (lane & 7);
    const int ldm_b = (lane >> 4) & (NB - 1);
    const uint32_t ldm_s0 = ring_s + ldm_tl * G::RBV + ((ldm_b ^ swz(ldm_tl)) * 16);
    const uint32_t ldm_s1 = ring_s + ldm_tl * G::RBV + (((ldm_b + 2) & (NB - 1)) ^ swz(ldm_tl)) * 16;
    const uint32_t pb_rd = pb_s + (tig * 8 + g) * 4;                                     // + jv * 512 + (8 h2 + 4 b) * 32
    // operand build: lane -> token pair pi = lane & 15 and head pair hh = lane >> 4 (heads 2 hh, 2 hh + 1)
    const int pi = lane & 15, hh = lane >> 4;
    const int bt0 = 16 * (pi >> 3) + 8 * ((pi >> 2) & 1) + 2 * (pi & 3);                 // the pair's first token in the stage
    const uint32_t sz_rd = ring_s + G::SZ_OFF + (bt0 * ngv) * 2;                         // scale row of token bt0; + ngv * 2 next token
    const uint32_t pb_wr = pb_s + (pi * 8 + 4 * hh) * 4;
    const float *pa = sm.scores + (2 * hh) * sm.n_scores + warp * G::TPS + bt0, *pb = pa + sm.n_scores;

    const int block_stride = kMmaWarps * G::TPS;
    const char *src_codes = reinterpret_cast<const char *>(vc + (int64_t)(t0 + warp * G::TPS) * a.vc_sT) + lane * 16;
    const int ngran = 4 * ngv;
    const int sz_arr = lane >= ngran ? 1 : 0;
    const int sz_off = (lane - sz_arr * ngran) * 16;
    const bool sz_on = lane < 2 * ngran;
    const char *src_sz = reinterpret_cast<const char *>((sz_arr ? vz : vs) + (int64_t)(t0 + warp * G::TPS) * a.vs_sT) + sz_off;
    const uint32_t sz_dst = ring_s + G::SZ_OFF + sz_arr * (G::TPS * 4 * 2) + sz_off;
    const int64_t codes_step = (int64_t)block_stride * G::RBV, sz_step = (int64_t)block_stride * ngv * 2;

    int to_issue = my_blocks;
    auto issue_stage = [&](uint32_t slot_off) {
        if (to_issue > 0) {
#pragma unroll
            for (int i = 0; i < G::GPL; ++i)
                if (G::TPS * G::GPT % 32 == 0 || lane + 32 * i < G::TPS * G::GPT)
                    cp_async<16>(cp_dst + slot_off + i * (32 / G::GPT) * G::RBV, src_codes + i * 512);
            if (sz_on) cp_async<16>(sz_dst + slot_off, src_sz);
        }
        --to_issue;
        src_codes += codes_step;
        src_sz += sz_step;
    };

    float acc[8][4], accz[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};    // ones-MMAs alternate between two accumulators
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
    // 1-bit values in groups of 64 channels: a 16-byte block (128 channels) then spans two groups, and the rows of an
    // MMA (lane octet g = channels 16 g .. 16 g + 15) lie in group g / 4.  Every code tile is multiplied twice, by the
    // operands of group 0 and of group 1, and a lane keeps the product of its own group.
    const bool split = VB == 1 && Gv == 64;
    float acc2[VB == 1 ? 8 : 1][4];
#pragma unroll
    for (int m = 0; m < (VB == 1 ? 8 : 1); ++m) acc2[m][0] = acc2[m][1] = acc2[m][2] = acc2[m][3] = 0.f;
    const uint32_t ones = 0x3c003c00u;
    constexpr int kFlush = 16;                                 // short accumulation chains (see the single-head kernel)
    float sum[8][2], sumz[2] = {0.f, 0.f};
#pragma unroll
    for (int m = 0; m < 8; ++m) sum[m][0] = sum[m][1] = 0.f;
    auto flush = [&]() {
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            if constexpr (VB == 1) {
                const bool second = split && g >= 4;
                sum[m][0] += second ? acc2[m][0] : acc[m][0];
                sum[m][1] += second ? acc2[m][2] : acc[m][2];
                acc2[m][0] = acc2[m][1] = acc2[m][2] = acc2[m][3] = 0.f;
            } else {
                sum[m][0] += acc[m][0];
                sum[m][1] += acc[m][2];
            }
            acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
        }
        sumz[0] += accz[0][0] + accz[1][0];
        sumz[1] += accz[0][1] + accz[1][1];
#pragma unroll
        for (int u = 0; u < 2; ++u) accz[u][0] = accz[u][1] = accz[u][2] = accz[u][3] = 0.f;
    };

    if (MODE != 2) {
#pragma unroll
        for (int q = 0; q < G::P; ++q) { issue_stage(q * G::STAGE_BYTES); cp_async_commit(); }
        if (MODE == 1) return;
    } else {
        to_issue -= G::P;
        src_codes += G::P * codes_step;
        src_sz += G::P * sz_step;
    }

    uint32_t st = 0, issue_st = G::P * G::STAGE_BYTES;
    for (int q = 0; q < my_blocks; ++q) {
        issue_stage(issue_st);
        cp_async_commit();
        cp_async_wait<G::P>();
        __syncwarp();
        // ---- B operands for the stage: per channel group 16 token pairs x 8 columns (head x {p*scale, p*midpoint}) ----
        {
            const float2 fa = *reinterpret_cast<const float2 *>(pa), fb = *reinterpret_cast<const float2 *>(pb);
            const float a0 = fa.x * 256.f, a1 = fa.y * 256.f, b0 = fb.x * 256.f, b1 = fb.y * 256.f;   // p carries 2^8
#pragma unroll
            for (int jv = 0; jv < 4; ++jv) {
                if (jv < ngv) {
                    const float s0 = __half2float(__ushort_as_half((unsigned short)lds16(sz_rd + st + 2 * jv)));
                    const float s1 = __half2float(__ushort_as_half((unsigned short)lds16(sz_rd + st + 2 * (ngv + jv))));
                    const float z0 = __half2float(__ushort_as_half((unsigned short)lds16(sz_rd + st + 256 + 2 * jv)));
                    const float z1 = __half2float(__ushort_as_half((unsigned short)lds16(sz_rd + st + 256 + 2 * (ngv + jv))));
                    const float m0 = fmaf(G::MID, s0, z0), m1 = fmaf(G::MID, s1, z1);
                    const uint32_t c0 = pack_h2_sat(a0 * s0, a1 * s1), c1 = pack_h2_sat(a0 * m0, a1 * m1);
                    const uint32_t c2 = pack_h2_sat(b0 * s0, b1 * s1), c3 = pack_h2_sat(b0 * m0, b1 * m1);
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(pb_wr + jv * 512), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
                }
            }
        }
        __syncwarp();
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            uint32_t b[4][2];
#pragma unroll
            for (int jv = 0; jv < 4; ++jv) {
                if (jv < ngv) {
                    b[jv][0] = lds32(pb_rd + jv * 512 + (8 * h2) * 32);
                    b[jv][1] = lds32(pb_rd + jv * 512 + (8 * h2 + 4) * 32);
                    const uint32_t row1 = (g == jv) ? ones : 0u;    // sums of group jv land in row jv
                    mma16816(accz[jv & 1], row1, 0u, row1, 0u, b[jv][0], b[jv][1]);
                } else {
                    b[jv][0] = b[jv][1] = 0u;
                }
            }
            uint32_t x[NB][2];
            const uint32_t ad = st + (16 * h2) * G::RBV;
            if constexpr (VB == 1) {
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                             : "=r"(x[0][0]), "=r"(x[0][1]) : "r"(ldm_s0 + ad));
            } else {
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(x[0][0]), "=r"(x[0][1]), "=r"(x[1][0]), "=r"(x[1][1]) : "r"(ldm_s0 + ad));
                if constexpr (VB == 4)
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(x[NB - 2][0]), "=r"(x[NB - 2][1]), "=r"(x[NB - 1][0]), "=r"(x[NB - 1][1])
                                 : "r"(ldm_s1 + ad));
            }
#pragma unroll
            for (int bb = 0; bb < NB; ++bb) {
                uint32_t rlo[F::N], rhi[F::N];
                F::unpack(x[bb][0], rlo);
                F::unpack(x[bb][1], rhi);
                // the block's channel group: v_group is 32 (4-bit values only), 64 or 128
                const int j32 = (bb * CPB) / 32 < 4 ? (bb * CPB) / 32 : 3, j64 = (bb * CPB) / 64;
                const uint32_t bx = Gv == 32 ? b[j32][0] : Gv == 64 ? b[j64][0] : b[0][0];
                const uint32_t by = Gv == 32 ? b[j32][1] : Gv == 64 ? b[j64][1] : b[0][1];
#pragma unroll
                for (int i = 0; i < F::N; i += 2)
                    mma16816(acc[bb * MPB + i / 2], rlo[i], rlo[i + 1], rhi[i], rhi[i + 1], bx, by);
                if constexpr (VB == 1) {
                    if (split) {
#pragma unroll
                        for (int i = 0; i < F::N; i += 2)
                            mma16816(acc2[i / 2], rlo[i], rlo[i + 1], rhi[i], rhi[i + 1], b[1][0], b[1][1]);
                    }
                }
            }
        }
        __syncwarp();
        st = (st + G::STAGE_BYTES == G::NS * G::STAGE_BYTES) ? 0u : st + G::STAGE_BYTES;
        issue_st = (issue_st + G::STAGE_BYTES == G::NS * G::STAGE_BYTES) ? 0u : issue_st + G::STAGE_BYTES;
        pa += block_stride;
        pb += block_stride;
        if ((q % kFlush) == kFlush - 1) flush();
    }
    flush();
    cp_async_wait<0>();
    __syncwarp();
    // epilogue: lane (g, tig) holds channels of rows g / g + 8 for head tig (column 2 tig); row jv of the ones-MMAs holds
    // (sum p*scale, sum p*mid) of channel group jv for head tig
    const float corr_mine = (sumz[1] - G::MID * sumz[0]) * (1.f / 256.f);
    float cj[4];
#pragma unroll
    for (int jv = 0; jv < 4; ++jv) cj[jv] = __shfl_sync(0xffffffffu, corr_mine, 4 * jv + tig);
#pragma unroll
    for (int bb = 0; bb < NB; ++bb) {
        const int c0 = bb * CPB + g * F::N;
        const float corr = Gv == 32 ? cj[(bb * CPB) / 32 < 4 ? (bb * CPB) / 32 : 3]
                         : Gv == 64 ? (VB == 1 ? (g >= 4 ? cj[1] : cj[0]) : cj[(bb * CPB) / 64]) : cj[0];
#pragma unroll
        for (int ip = 0; ip < MPB; ++ip) {
            my_red[tig * kHeadDim + c0 + 2 * ip] = fmaf(sum[bb * MPB + ip][0], (float)(1 << (16 - F::pos(2 * ip))), corr);
            my_red[tig * kHeadDim + c0 + 2 * ip + 1] = fmaf(sum[bb * MPB + ip][1], (float)(1 << (16 - F::pos(2 * ip + 1))), corr);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// One segment: tokens [t0, t1) of head group s (sequence b, kv head hk, quad of query heads); segment `seg` of `cnt`.
template <int KB, int VB>
__device__ __forceinline__ void gqa_segment(const kvq_attn_args &a, const kvq_attn_args &ac, int n_scores, int qhv, int s, int t0, int t1, int seg,
                                            int cnt, int n_whole, float *__restrict__ parts,
                                            unsigned int *__restrict__ counters) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int kRegion = gqa_region_bytes<KB, VB>();
    GqaSmem sm;
    sm.n_scores = n_scores;
    sm.scores = reinterpret_cast<float *>(smem_raw);
    unsigned char *after_scores = smem_raw + (size_t)kQH * n_scores * 4;
    sm.ring = after_scores + warp * kRegion;
    sm.q = reinterpret_cast<__half *>(after_scores + kMmaWarps * kRegion);
    sm.misc = reinterpret_cast<float *>(sm.q + kQH * kHeadDim);
    float *tail_part = reinterpret_cast<float *>(sm.ring + VGeom<VB>::NS * VGeom<VB>::STAGE_BYTES + kGqaTailOff);

    const int n_rep = a.nh / a.nh_kv, nq = n_rep / qhv;                // quads per kv head
    const int b = s / (a.nh_kv * nq), hk = (s / nq) % a.nh_kv, h_first = hk * n_rep + (s % nq) * qhv;

    fused_cache_update<KB, VB>(a, b, hk, t0, t1, tid);        // the step's own cache update, when the caller fused it in
    // q of the quad (head slots beyond qhv repeat the last head: their columns are computed and dropped)
    {
        const int hs = min(tid >> 5, qhv - 1);                          // warp w stores head slot w
        const __half *q = static_cast<const __half *>(a.q) + (int64_t)b * a.q_sB + (int64_t)(h_first + hs) * a.q_sH;
        *reinterpret_cast<uint2 *>(sm.q + warp * kHeadDim + 4 * lane) = *reinterpret_cast<const uint2 *>(q + 4 * lane);
    }

    // ---- 1. scores ------------------------------------------------------------------------------
    const __half *kf = static_cast<const __half *>(a.kfull) + (int64_t)b * a.kf_sB + (int64_t)hk * a.kf_sH;
    {
        const int hi = min(t1, a.Tkq);
        if (t0 < hi) {
            const int32_t *kc = a.kcode + (int64_t)b * a.kc_sB + (int64_t)hk * a.kc_sH;
            const __half *ks = static_cast<const __half *>(a.kscale) + (int64_t)b * a.ks_sB + (int64_t)hk * a.ks_sH;
            const __half *kz = static_cast<const __half *>(a.kmn) + (int64_t)b * a.ks_sB + (int64_t)hk * a.ks_sH;
            gqa_qk_packed<KB>(a, kc, ks, kz, sm, t0, hi, kf, max(t0, a.Tkq), t1, b, hk);
        } else {
            __syncthreads();
            if (t0 < t1) gqa_qk_tail(a, kf, b, hk, sm, t0, t0, t1);
        }
    }
    const int32_t *vc = a.vcode + (int64_t)b * a.vc_sB + (int64_t)hk * a.vc_sH;
    const __half *vs = static_cast<const __half *>(a.vscale) + (int64_t)b * a.vs_sB + (int64_t)hk * a.vs_sH;
    const __half *vz = static_cast<const __half *>(a.vmn) + (int64_t)b * a.vs_sB + (int64_t)hk * a.vs_sH;
    const int v_hi = min(t1, a.Tvq);
    if (t0 < v_hi) gqa_pv_packed<VB, 1>(a, vc, vs, vz, sm, t0, v_hi);   // start filling this warp's value ring now
    __syncthreads();

    // ---- 2. softmax numerators: warp w owns head slot w -------------------------------------------
    // The fp16 value tail of this segment is fetched into registers first (its latency is spent under the softmax).
    const int n = t1 - t0;
    const int v_lo = max(t0, a.Tvq);
    const __half *vf = static_cast<const __half *>(a.vfull) + (int64_t)b * a.vf_sB + (int64_t)hk * a.vf_sH;
    const int co = tid & 15, tl = tid >> 4;
    uint4 vt[16];
    auto load_tail_round = [&](int base) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = base + tl + 8 * j;
            vt[j] = (t < t1) ? __ldg(reinterpret_cast<const uint4 *>(v_tail_row(a, vf, b, hk, t)) + co) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    if (v_lo < t1) load_tail_round(v_lo);

    const int h_mine = h_first + min(warp, qhv - 1);
    float m = kMaskFloor;
    const int n4 = (n + 3) >> 2;
    float4 *sc4 = reinterpret_cast<float4 *>(sm.scores + warp * n_scores);
#pragma unroll 4
    for (int i = lane; i < n4; i += 32) {
        float4 v = sc4[i];
        if (a.mask) {
            const int t = t0 + 4 * i;
            v.x = fmaxf(v.x + attn_mask_at(a, b, h_mine, min(t, a.T - 1)), kMaskFloor);
            v.y = fmaxf(v.y + attn_mask_at(a, b, h_mine, min(t + 1, a.T - 1)), kMaskFloor);
            v.z = fmaxf(v.z + attn_mask_at(a, b, h_mine, min(t + 2, a.T - 1)), kMaskFloor);
            v.w = fmaxf(v.w + attn_mask_at(a, b, h_mine, min(t + 3, a.T - 1)), kMaskFloor);
            sc4[i] = v;
        }
        if (4 * i + 3 >= n) {
            if (4 * i + 1 >= n) v.y = -INFINITY;
            if (4 * i + 2 >= n) v.z = -INFINITY;
            v.w = -INFINITY;
            sc4[i] = v;
        }
        m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
    m = warp_max(m);
    __syncwarp();
    float l = 0.f;
#pragma unroll 4
    for (int i = lane; i < n4; i += 32) {
        float4 v = sc4[i];
        v.x = __expf(v.x - m);
        v.y = __expf(v.y - m);
        v.z = __expf(v.z - m);
        v.w = __expf(v.w - m);
        sc4[i] = v;
        l += (v.x + v.y) + (v.z + v.w);
    }
    l = warp_sum(l);
    if (lane == 0) { sm.misc[warp] = m; sm.misc[4 + warp] = l; }
    __syncthreads();

    // ---- 3. p . V -----------------------------------------------------------------------------------
    if (v_lo < t1) {
#pragma unroll 1
        for (int hs = 0; hs < kQH; ++hs) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const float *ph = sm.scores + hs * n_scores - t0;
            for (int base = v_lo; base < t1; base += 128) {
                if (base > v_lo || hs > 0) { if (t1 - v_lo > 128) load_tail_round(base); }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int t = base + tl + 8 * j;
                    const float p = (t < t1) ? ph[t] : 0.f;
                    const __half2 *h = reinterpret_cast<const __half2 *>(&vt[j]);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = __half22float2(h[k]);
                        acc[2 * k] = fmaf(p, f.x, acc[2 * k]);
                        acc[2 * k + 1] = fmaf(p, f.y, acc[2 * k + 1]);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 16);
            if (lane < 16) {
                float4 *dst = reinterpret_cast<float4 *>(tail_part + hs * kHeadDim + 8 * co);
                dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
                dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
        }
    } else {
        for (int i = lane; i < kQH * kHeadDim; i += 32) tail_part[i] = 0.f;
    }
    if (t0 < v_hi) gqa_pv_packed<VB, 2>(a, vc, vs, vz, sm, t0, v_hi);
    else for (int i = lane; i < kQH * kHeadDim; i += 32) reinterpret_cast<float *>(sm.ring)[i] = 0.f;
    __syncthreads();

    // ---- 4. finish / merge: thread tid owns channel tid of every head ----------------------------------
    constexpr int kPart = kPartStride;
    float o[kQH];
#pragma unroll
    for (int hs = 0; hs < kQH; ++hs) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) {
            const unsigned char *reg = after_scores + w * kRegion;
            v += reinterpret_cast<const float *>(reg)[hs * kHeadDim + tid] +
                 reinterpret_cast<const float *>(reg + VGeom<VB>::NS * VGeom<VB>::STAGE_BYTES + kGqaTailOff)[hs * kHeadDim + tid];
        }
        o[hs] = v;
    }
    __half res[kQH];
    if (cnt == 1) {
#pragma unroll
        for (int hs = 0; hs < kQH; ++hs) {
            if (hs < qhv) {
                __half *out = static_cast<__half *>(a.out) + (int64_t)b * a.o_sB + (int64_t)(h_first + hs) * a.o_sH;
                res[hs] = __float2half_rn(o[hs] / sm.misc[4 + hs]);
                out[tid] = res[hs];
            }
        }
        peer_publish(ac, b, h_first, qhv, res, tid);
        return;
    }
    float *part = parts + ((int64_t)(s - n_whole) * cnt + seg) * qhv * kPart;    // partials of the cut head groups only
#pragma unroll
    for (int hs = 0; hs < kQH; ++hs) {
        if (hs < qhv) {
            part[hs * kPart + tid] = o[hs];
            if (tid == 0) { part[hs * kPart + kHeadDim] = sm.misc[hs]; part[hs * kPart + kHeadDim + 1] = sm.misc[4 + hs]; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        sm.misc[8] = (atomicAdd(&counters[s], 1u) == (unsigned)(cnt - 1)) ? 1.f : 0.f;
        __threadfence();
    }
    __syncthreads();
    if (sm.misc[8] == 0.f) return;
    // The last CTA merges the cnt segments of its head group.  A long context over few heads means a hundred or more
    // segments, and a merge that walks them one dependent round trip at a time becomes the kernel, so many 128-bit loads
    // are kept in flight: warp w merges head slot w, lane l owning channels 4l .. 4l + 3; the maximum over the segments
    // first (lanes over segments), then the weighted sums, sixteen segments' loads issued before the first is used.  The
    // order is fixed, so results are run-to-run identical.
    __half *stage = reinterpret_cast<__half *>(after_scores);             // [kQH][128] results, regions are idle by now
    if (warp < qhv) {
        const float *bh = parts + (int64_t)(s - n_whole) * cnt * qhv * kPart + warp * kPart;
        const int stride = qhv * kPart;
        float M = kMaskFloor;
        for (int i = lane; i < cnt; i += 32) M = fmaxf(M, __ldcg(bh + (int64_t)i * stride + kHeadDim));
        M = warp_max(M);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
#pragma unroll 16
        for (int i = 0; i < cnt; ++i) {
            const float *pi = bh + (int64_t)i * stride;
            const float2 ml = __ldcg(reinterpret_cast<const float2 *>(pi + kHeadDim));
            const float4 p = __ldcg(reinterpret_cast<const float4 *>(pi) + lane);
            const float w = __expf(ml.x - M);
            L = fmaf(ml.y, w, L);
            acc.x = fmaf(p.x, w, acc.x); acc.y = fmaf(p.y, w, acc.y);
            acc.z = fmaf(p.z, w, acc.z); acc.w = fmaf(p.w, w, acc.w);
        }
        const float inv = 1.f / L;
        __half2 *dst = reinterpret_cast<__half2 *>(stage + warp * kHeadDim + 4 * lane);
        dst[0] = __floats2half2_rn(acc.x * inv, acc.y * inv);
        dst[1] = __floats2half2_rn(acc.z * inv, acc.w * inv);
    }
    __syncthreads();
#pragma unroll
    for (int hs = 0; hs < kQH; ++hs) {
        if (hs < qhv) {
            __half *out = static_cast<__half *>(a.out) + (int64_t)b * a.o_sB + (int64_t)(h_first + hs) * a.o_sH;
            res[hs] = stage[hs * kHeadDim + tid];
            out[tid] = res[hs];
        }
    }
    if (tid == 0) counters[s] = 0u;
    peer_publish(ac, b, h_first, qhv, res, tid);
}

template <int KB, int VB, bool DEV>
__global__ void __launch_bounds__(kMmaThreads, 2) decode_attn_gqa_kernel(const __grid_constant__ kvq_attn_args a,
                                                                     const __grid_constant__ AttnPlan plan, int qhv,
                                                                     float *__restrict__ parts,
                                                                     unsigned int *__restrict__ counters) {
    int group, t0, t1, seg, cnt;
    if constexpr (DEV) {                                       // device-resident cache state: see decode_attn_mma_kernel
        kvq_attn_args b = a;
        dev_state_step(a, b);
        plan_cta(plan, b.T, blockIdx.x, group, t0, t1, seg, cnt);
        if (cnt > 1) cnt = min(cnt, (b.T + plan.seg_units * plan.unit - 1) / (plan.seg_units * plan.unit));
        if (t0 < b.T) gqa_segment<KB, VB>(b, a, plan.n_scores, qhv, group, t0, t1, seg, cnt, plan.n_whole, parts, counters);
    } else {
        plan_cta(plan, a.T, blockIdx.x, group, t0, t1, seg, cnt);
        gqa_segment<KB, VB>(a, a, plan.n_scores, qhv, group, t0, t1, seg, cnt, plan.n_whole, parts, counters);
    }
}

// ---------------------------------------------------------------------------------------------
// Query heads per CTA for this call (0: the grouped kernel does not take it and the single-head kernel runs): the
// heads of a kv head in quads (or the pair, for two heads per kv head), and group sizes that keep an MMA's rows in
// one group.
int gqa_heads_per_cta(const kvq_attn_args &a) {
    if (a.nh_kv <= 0 || a.nh % a.nh_kv != 0) return 0;
    const int n_rep = a.nh / a.nh_kv;
    if (n_rep != 2 && n_rep % 4 != 0) return 0;
    const int kmin = a.k_bits == 1 ? 128 : a.k_bits == 2 ? 64 : a.k_bits == 4 ? 64 : 11;
    const int vmin = a.v_bits == 1 ? 64 : a.v_bits == 2 ? 64 : 32;     // 1-bit values at group 64: two MMAs per code tile
    if (a.k_bits != 3 && a.k_group < kmin) return 0;
    if (a.v_group < vmin) return 0;
    return n_rep == 2 ? 2 : 4;
}

AttnPlan plan_attn_gqa(int T, int k_bits, long long head_groups) {
    const int unit = (k_bits == 3) ? 352 : 256;
    const int max_chunk = (k_bits == 3) ? 2816 : kGqaMaxChunk;     // whole units of 352 / 256 tokens
    return make_attn_plan(T, unit, max_chunk, head_groups, kSmCount * 2, k_bits == 3 ? 1 : kMmaWarps);
}

template <int KB, int VB>
static int launch_gqa(const kvq_attn_args &a, const AttnPlan &plan, int qhv, float *parts, unsigned int *counters,
                      cudaStream_t st) {
    const size_t smem = (size_t)kQH * plan.n_scores * 4 + (size_t)kMmaWarps * gqa_region_bytes<KB, VB>() +
                        kQH * kHeadDim * 2 + 64 * 4;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        e = cudaFuncSetAttribute(decode_attn_gqa_kernel<KB, VB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(decode_attn_gqa_kernel<KB, VB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const unsigned grid = (unsigned)(plan.n_whole + plan.n_cut * plan.k);
    if (a.state) decode_attn_gqa_kernel<KB, VB, true><<<grid, kMmaThreads, smem, st>>>(a, plan, qhv, parts, counters);
    else decode_attn_gqa_kernel<KB, VB, false><<<grid, kMmaThreads, smem, st>>>(a, plan, qhv, parts, counters);
    return check_launch();
}

int launch_decode_attn_gqa(const kvq_attn_args &a, const AttnPlan &plan, int qhv, float *parts, unsigned int *counters,
                           cudaStream_t st) {
#define KVQ_GQA_CASE(KB, VB) \
    if (a.k_bits == KB && a.v_bits == VB) return launch_gqa<KB, VB>(a, plan, qhv, parts, counters, st);
    KVQ_GQA_CASE(4, 4) KVQ_GQA_CASE(4, 2) KVQ_GQA_CASE(4, 1)
    KVQ_GQA_CASE(3, 4) KVQ_GQA_CASE(3, 2) KVQ_GQA_CASE(3, 1)
    KVQ_GQA_CASE(2, 4) KVQ_GQA_CASE(2, 2) KVQ_GQA_CASE(2, 1)
    KVQ_GQA_CASE(1, 4) KVQ_GQA_CASE(1, 2) KVQ_GQA_CASE(1, 1)
#undef KVQ_GQA_CASE
    return KVQ_ERR_UNSUPPORTED;
}

}  // namespace kvq
