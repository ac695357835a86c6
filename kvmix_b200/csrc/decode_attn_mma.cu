// Fused decode attention, tensor-core path: one CTA (4 warps) per query head and token split; the query heads of a
// kv head are neighbouring CTAs and share its cache through L2.
//
// Why tensor cores for a mat-vec: at the HBM rate a B200 has only ~1-3 issue slots per packed code (2.8 per 2-bit
// code at 5.6 TB/s and 1.9 GHz).  Shift-mask-convert-FMA per code does not fit; one logic op per *pair* of codes
// plus one mma.sync per 256 codes does.
//
// Codes go to the tensor core without ever being converted: a b-bit field left in place inside a 16-bit lane, with
// all other bits masked off, *is* an fp16 number with value field * 2^(pos-24) (subnormals and the first normal
// binade are linear in the bit pattern).  mma.sync multiplies such inputs exactly and accumulates in fp32, so the
// product with the fp16 operand is exact and the power of two is undone per output row in the epilogue.  Pairs
// along the contraction axis arrive ready-made from transposing ldmatrix loads (values; 1- and 2-bit keys) or are
// formed with one byte-permute of two words (3- and 4-bit keys).
//
// Keys (codes [D, T/fpi], one word = fpi tokens of one channel; scale/zero [D, T/G]):
//   A (16x16) = codes, rows = tokens, cols = 16 channels.  q[d]*scale[d,g] is carried as an exact fp16 pair hi + lo.
//   A 256-token warp tile is worked as two halves whose MMA rows touch at most four groups, so B (16x8) holds
//   {hi, lo} x 4 groups side by side and one MMA per code tile yields both parts.  3-bit keys (88-token tiles, every
//   word its own group of 11) multiply each code tile by the hi and by the lo operand instead.  The zero terms
//   sum_d q[d]*zero[d,g] of all groups of a tile come from one MMA per 16 channels whose A operand is the zero tile
//   read transposed (row = group) and whose B operand is q.
// Values (codes [T, D/fpi], one word = fpi channels of one token; scale/zero [T, D/G]):
//   A (16x16) = codes, rows = channels, cols = 16 tokens;  B (16x8): column 2j = p[t]*scale[t,j], column 2j+1 =
//   p[t]*midpoint[t,j] (codes are used centred on the group midpoint); one extra MMA with A = ones sums both columns.
// Code words and scale/zero rows stream through per-warp multi-stage cp.async rings in shared memory (128-bit
// copies, several KB in flight per warp).  The fp16 key tail is scored on the tensor cores straight from global
// memory; the softmax, the optional additive mask and the fp16 value tail run on the CUDA cores.
#include "attn_mma_common.cuh"
#include "attn_plan.cuh"
#include "attn_update.cuh"

namespace kvq {

struct MmaSmem {
    float *scores;          // [n_scores]
    unsigned char *ring;    // this warp's region
    float *tailred;         // [kMmaWarps][kHeadDim] partial sums of the fp16 value tail
    __half *q;              // [kHeadDim]
    float *misc;            // [16]
};

// ---------------------------------------------------------------------------------------------
// q . K^T over packed keys for tokens [t0, hi) (t0 is a multiple of 1024, or 352 for 3-bit keys).
// Scores (already multiplied by softmax_scale) go to sm.scores[t - t0].  Warps work independently:
// warp w takes warp tiles w, w+4, ... and streams their code words through its own ring.
__device__ __forceinline__ void qk_tail_mma(const kvq_attn_args &a, const __half *kf, int b, int hk, const MmaSmem &sm,
                                            int t0, int lo, int t1);

// If the split also holds fp16 tail keys (tail_lo < t1) they are scored right after the first code stages
// have been issued, so the tail's global-load latency overlaps the ring fill.
template <int KB>
__device__ __forceinline__ void qk_packed_mma(const kvq_attn_args &a, const int32_t *kc, const __half *ks,
                                              const __half *kz, const MmaSmem &sm, int t0, int hi,
                                              const __half *kf, int tail_lo, int t1, int b, int hk) {
    using G = KGeom<KB>;
    using F = Fields<KB>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const int Gk = a.k_group;
    const int n_words = a.Tkq / G::FPI;                       // valid code words per channel row
    const int n_tiles = (hi - t0 + G::WT - 1) / G::WT;
    const int my_tiles = (n_tiles - warp + kMmaWarps - 1) / kMmaWarps;   // tiles warp, warp+4, ...
    if (my_tiles <= 0) {
        __syncthreads();                                       // q is in shared memory (see below)
        if (tail_lo < t1) qk_tail_mma(a, kf, b, hk, sm, t0, tail_lo, t1);
        return;
    }

    const int kc_sD = (int)a.kc_sD, ks_sD = (int)a.ks_sD;
    // ---- per-lane constants --------------------------------------------------------------------
    const uint32_t ring_s = smem_u32(sm.ring);
    const uint32_t sz_s = ring_s + G::NS * G::STAGE_BYTES;                    // [2][128][8] halfs
    const int gr = lane % G::GPR, row0 = lane / G::GPR;
    const uint32_t cp_dst = ring_s + row0 * G::RS + gr * 16;                   // + slot*STAGE + i*RPI*RS
    // 3-bit: octet g owns the word of group g (11 tokens), fetched with plain 32-bit loads.
    // Other widths: code fragments come from transposing ldmatrix loads.  A channel row of the tile is NBK blocks of
    // 16 bytes; one x4 load covers channel rows 16 ksx + (0..7 | 8..15) x two neighbouring blocks and hands lane
    // (g, tig) the half-word g of each block for the channel pair (2 tig, 2 tig + 1) [+8]: an A-fragment register pair
    // along k without a byte permute.  Octet g of block bb therefore owns tokens bb * 8 FH + g * FH .. + FH - 1
    // (FH = 16 / bits fields per half-word).  The first NBK / 2 blocks are the first 128 tokens: their MMA rows touch
    // at most four groups, so the eight B columns carry {hi, lo} of q*scale for those four side by side (b0); the
    // other blocks use b1.
    constexpr int FH = (KB == 3) ? 2 : 16 / KB;                                // fields per half-word: 4 / 8 / 16
    constexpr int NBK = G::RB / 16;                                            // 16-byte blocks per channel row: 8 / 4 / 2
    constexpr int MPB = FH / 2;                                                // MMAs per block and k-step: 2 / 4 / 8
    constexpr int HW = 2;                                                      // 4-bit: code words per octet per half
    const uint32_t frag_s = ring_s + (2 * tig) * G::RS + ((KB == 4) ? 8 * g : 4 * g);   // 3-bit and 4-bit (plain loads)
    const uint32_t ldk_s = ring_s + ((lane & 7) + 8 * ((lane >> 3) & 1)) * G::RS + (lane >> 4) * 16;   // + k*16*RS + 32*pair
    // ldmatrix.x4 row addresses: lanes 0-7 scale rows 16ksx+0..7, 8-15 scale rows +8..15, 16-31 the same of the zero tile
    const uint32_t ldm_s = sz_s + (((lane >> 3) & 1) * 8 + (lane & 7)) * 16 + (lane >> 4) * 2048;
    const uint32_t q_s = smem_u32(sm.q) + (2 * tig) * 2;                       // + 32 ksx [+16]
    const int ngw = (G::WT + Gk - 1) / Gk;                                     // groups per warp tile: 8 / 4 / 2
    const uint32_t szcp_dst = sz_s + lane * 16;                                // + i*512
    const int tile_words = kMmaWarps * G::WT / G::FPI;                         // word-column distance between my tiles
    const int tile_groups = kMmaWarps * G::WT / Gk;

    const int32_t *tb_cur = kc + (int64_t)row0 * kc_sD + (t0 + warp * G::WT) / G::FPI + 4 * gr;
    const __half *ks_cur = ks + (int64_t)lane * ks_sD + (t0 + warp * G::WT) / Gk;
    const __half *kz_cur = kz + (int64_t)lane * ks_sD + (t0 + warp * G::WT) / Gk;
    int wcol_cur = (t0 + warp * G::WT) / G::FPI + 4 * gr;                      // this lane's granule word column
    bool ok_cur = wcol_cur < n_words;

    auto issue_stage = [&](const int32_t *tb, bool ok, int sst) {              // sst: compile-time stage of the tile
        if (ok) {
            const uint32_t dst = cp_dst + (sst % G::NS) * G::STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < G::GPL; ++i)
                cp_async<16>(dst + i * G::RPI * G::RS, tb + (sst * G::ROWS + i * G::RPI) * kc_sD);
        }
    };
    auto issue_sz = [&](const __half *ps, const __half *pz) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int off = 32 * i * ks_sD;
            if (ngw == 8) { cp_async<16>(szcp_dst + i * 512, ps + off); cp_async<16>(szcp_dst + 2048 + i * 512, pz + off); }
            else if (ngw == 4) { cp_async<8>(szcp_dst + i * 512, ps + off); cp_async<8>(szcp_dst + 2048 + i * 512, pz + off); }
            else { cp_async<4>(szcp_dst + i * 512, ps + off); cp_async<4>(szcp_dst + 2048 + i * 512, pz + off); }
        }
    };

    issue_sz(ks_cur, kz_cur);
    issue_stage(tb_cur, ok_cur, 0);
    cp_async_commit();
    issue_stage(tb_cur, ok_cur, 1);
    cp_async_commit();
    issue_stage(tb_cur, ok_cur, 2);
    cp_async_commit();
    // The caller stored q to shared memory just before this call without a barrier, so that the first code stages
    // are in flight while q arrives; every warp passes exactly one barrier here before anything reads q.
    __syncthreads();
    if (tail_lo < t1) qk_tail_mma(a, kf, b, hk, sm, t0, tail_lo, t1);

    for (int j = 0; j < my_tiles; ++j) {
        const int tile0 = t0 + (j * kMmaWarps + warp) * G::WT;
        const bool have_next = j + 1 < my_tiles;
        const int32_t *tb_nxt = tb_cur + tile_words;
        const bool ok_nxt = have_next && (wcol_cur + tile_words < n_words);

        // the scale/zero tile of this warp tile was committed at least 3 groups ago
        cp_async_wait<2>();
        __syncwarp();
        // ---- B fragments q*scale and the zero term sum_d q[d]*zero[d,g] ----------------------------------
        // q*scale needs 22 bits; it is carried as an fp16 pair hi + lo (lo = fma(q, s, -hi) is exact), so the key
        // side adds no rounding beyond the fp32 accumulation.
        // 3-bit keys: b0 = hi and b1 = lo of the eight groups of the tile, every code tile is multiplied by both.
        // Other widths: b0 / b1 serve the first / second half of the tile; column n carries group (n / 2) of that
        // half, hi in even and lo in odd columns, so one MMA per code tile yields both parts.
        uint32_t b0[8][2], b1[8][2];
        float accz[4] = {0.f, 0.f, 0.f, 0.f}, accy[4] = {0.f, 0.f, 0.f, 0.f};
        const int gph = ngw > 1 ? ngw / 2 : 1;                 // groups per half tile: 4 / 2 / 1
        const int src0 = 4 * ((g >> 1) % gph) + tig;           // lane holding group (n / 2) of the first half
        const int src1 = src0 + 4 * (ngw / 2);
        const bool odd = g & 1;
#pragma unroll
        for (int ksx = 0; ksx < 8; ++ksx) {
            const uint32_t q01u = lds32(q_s + 32 * ksx), q89u = lds32(q_s + 32 * ksx + 16);
            const __half2 q01 = as_h2(q01u), q89 = as_h2(q89u);
            // the tile rows are 8 groups x fp16 = one 8x8 matrix per 8 channels: a transposing ldmatrix hands
            // lane (g, tig) exactly {row 2tig, row 2tig+1} x column g, i.e. its B-fragment pairs of group g, in one go
            // (with fewer than 8 groups per tile the columns past the last group are stale and feed unused columns)
            uint32_t r0, r1, r2, r3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(ldm_s + ksx * 256));
            // The zero terms: the same two registers are also the A fragment of the transposed zero tile (row = group g,
            // k = channels 2tig, 2tig+1 / +8), so ONE MMA with B = q (in every column) leaves sum_d q[d] * zero[d, g] in
            // row g; fp16 x fp16 products are exact in the tensor core, no hi / lo split is needed.  Two accumulators
            // alternate to keep the chains short.  A stale group only spoils its own row.
            if (ksx & 1) mma16816(accy, r2, 0u, r3, 0u, q01u, q89u);
            else mma16816(accz, r2, 0u, r3, 0u, q01u, q89u);
            if constexpr (KB == 3) {
                const __half2 s01 = as_h2(r0), s89 = as_h2(r1);
                const __half2 p01 = __hmul2(q01, s01), p89 = __hmul2(q89, s89);
                b0[ksx][0] = as_u32(p01);
                b0[ksx][1] = as_u32(p89);
                b1[ksx][0] = as_u32(__hfma2(q01, s01, __hneg2(p01)));
                b1[ksx][1] = as_u32(__hfma2(q89, s89, __hneg2(p89)));
            } else {
                const __half2 sa01 = as_h2(__shfl_sync(0xffffffffu, r0, src0)), sa89 = as_h2(__shfl_sync(0xffffffffu, r1, src0));
                const __half2 sb01 = as_h2(__shfl_sync(0xffffffffu, r0, src1)), sb89 = as_h2(__shfl_sync(0xffffffffu, r1, src1));
                const __half2 pa01 = __hmul2(q01, sa01), pa89 = __hmul2(q89, sa89);
                const __half2 pb01 = __hmul2(q01, sb01), pb89 = __hmul2(q89, sb89);
                b0[ksx][0] = odd ? as_u32(__hfma2(q01, sa01, __hneg2(pa01))) : as_u32(pa01);
                b0[ksx][1] = odd ? as_u32(__hfma2(q89, sa89, __hneg2(pa89))) : as_u32(pa89);
                b1[ksx][0] = odd ? as_u32(__hfma2(q01, sb01, __hneg2(pb01))) : as_u32(pb01);
                b1[ksx][1] = odd ? as_u32(__hfma2(q89, sb89, __hneg2(pb89))) : as_u32(pb89);
            }
        }
        __syncwarp();                                          // everyone has read the tile: it may be refilled
#pragma unroll
        for (int i = 0; i < 4; ++i) accz[i] += accy[i];

        float acc[G::NMMA][4];
#pragma unroll
        for (int m = 0; m < G::NMMA; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;

#pragma unroll
        for (int st = 0; st < G::NSTAGE; ++st) {
            // issue stage st+P (of this tile or the next); the next tile's scale/zero tile rides with its first stage
            if (st + G::P < G::NSTAGE) {
                issue_stage(tb_cur, ok_cur, st + G::P);
            } else {
                issue_stage(tb_nxt, ok_nxt, st + G::P - G::NSTAGE);
            }
            if (st == 0 && have_next) issue_sz(ks_cur + tile_groups, kz_cur + tile_groups);
            cp_async_commit();
            cp_async_wait<G::P>();
            __syncwarp();
            const uint32_t src = frag_s + (st % G::NS) * G::STAGE_BYTES;
#pragma unroll
            for (int k = 0; k < G::KSPS; ++k) {
                const int ksx = st * G::KSPS + k;
                if constexpr (KB == 3) {
                    uint32_t w[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) w[r] = lds32(src + (k * 16 + (r & 1) + (r >> 1) * 8) * G::RS);
                    uint32_t rlo[F::N], rhi[F::N];
                    F::unpack(w[0], w[1], rlo);
                    F::unpack(w[2], w[3], rhi);
#pragma unroll
                    for (int i = 0; i < F::N; i += 2) {
                        const uint32_t a1 = (i + 1 < F::N) ? rlo[i + 1] : 0u, a3 = (i + 1 < F::N) ? rhi[i + 1] : 0u;
                        mma16816(acc[i / 2], rlo[i], a1, rhi[i], a3, b0[ksx][0], b0[ksx][1]);
                    }
#pragma unroll
                    for (int i = 0; i < F::N; i += 2) {
                        const uint32_t a1 = (i + 1 < F::N) ? rlo[i + 1] : 0u, a3 = (i + 1 < F::N) ? rhi[i + 1] : 0u;
                        mma16816(acc[i / 2], rlo[i], a1, rhi[i], a3, b1[ksx][0], b1[ksx][1]);
                    }
                } else if constexpr (KB == 4) {
                    // 4-bit keys: two words (16 tokens) per octet and half, plain 64-bit loads + byte permutes (measured 1.5 %
                    // faster than the ldmatrix form below for this width: 4 loads of 2 blocks each per k-step)
                    constexpr int NF = F::N;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t w[4][HW];
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const uint32_t ad = src + (k * 16 + (r & 1) + (r >> 1) * 8) * G::RS + h * (G::RB / 2);
                            asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];\n" : "=r"(w[r][0]), "=r"(w[r][1]) : "r"(ad));
                        }
#pragma unroll
                        for (int x = 0; x < HW; ++x) {
                            uint32_t rlo[F::N], rhi[F::N];
                            F::unpack(w[0][x], w[1][x], rlo);
                            F::unpack(w[2][x], w[3][x], rhi);
#pragma unroll
                            for (int i = 0; i < NF; i += 2) {
                                const int m = h * 8 + (x * NF + i) / 2;
                                if (h == 0) mma16816(acc[m], rlo[i], rlo[i + 1], rhi[i], rhi[i + 1], b0[ksx][0], b0[ksx][1]);
                                else mma16816(acc[m], rlo[i], rlo[i + 1], rhi[i], rhi[i + 1], b1[ksx][0], b1[ksx][1]);
                            }
                        }
                    }
                } else {
                    using H = KHalf<KB>;
                    const uint32_t lsrc = ldk_s + (st % G::NS) * G::STAGE_BYTES + (k * 16) * G::RS;
#pragma unroll
                    for (int pb2 = 0; pb2 < NBK / 2; ++pb2) {              // two blocks per load
                        uint32_t x[2][2];
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                                     : "=r"(x[0][0]), "=r"(x[0][1]), "=r"(x[1][0]), "=r"(x[1][1]) : "r"(lsrc + pb2 * 32));
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int bb = 2 * pb2 + u;
                            uint32_t rlo[H::N], rhi[H::N];
                            H::unpack(x[u][0], rlo);                        // channels 2tig, 2tig+1  -> k cols 2tig, 2tig+1
                            H::unpack(x[u][1], rhi);                        // channels 2tig+8, +9    -> k cols 2tig+8, 2tig+9
                            const uint32_t bx = (bb >= NBK / 2) ? b1[ksx][0] : b0[ksx][0];
                            const uint32_t by = (bb >= NBK / 2) ? b1[ksx][1] : b0[ksx][1];
#pragma unroll
                            for (int i = 0; i < H::N; i += 2)
                                mma16816(acc[bb * MPB + i / 2], rlo[i], rlo[i + 1], rhi[i], rhi[i + 1], bx, by);
                        }
                    }
                }
            }
            __syncwarp();                                      // slot st % NS is free for the stage NS ahead
        }

        // ---- epilogue ----------------------------------------------------------------------------------
        if constexpr (KB == 3) {
            // the octet's column is n = g, held by the lane with tig == g/2
            const int tok0 = tile0 + g * G::TPO;               // first token of this octet's chunk
            if (tok0 < hi && tig == (g >> 1)) {                // chunks are whole or absent (hi is a group multiple)
                const bool sel = g & 1;
                const float corr = accz[0];                    // row g of the zero-term product = group g = this octet's word
                float *dst = sm.scores + (tok0 - t0);
#pragma unroll
                for (int m = 0; m < G::NMMA; ++m) {
                    const int i0 = 2 * m, i1 = 2 * m + 1;
                    float s0 = fmaf(sel ? acc[m][1] : acc[m][0], (float)(1 << (24 - F::pos(i0 % F::N))), corr);
                    float s1 = (i1 < G::TPO) ? fmaf(sel ? acc[m][3] : acc[m][2], (float)(1 << (24 - F::pos(i1 % F::N))), corr) : 0.f;
                    if (a.round_scores) {
                        const float2 r = __half22float2(__floats2half2_rn(s0, s1));
                        s0 = r.x;
                        s1 = r.y;
                    }
                    dst[i0] = s0 * a.softmax_scale;
                    if (i1 < G::TPO) dst[i1] = s1 * a.softmax_scale;
                }
            }
        } else if constexpr (KB == 4) {
            // octet g of half h is in group h*gph + cp of the tile, cp = 16 g / Gk; its hi and lo sums are the column
            // pair cp, held by the lane with tig == cp; the group's zero term sits in the lanes of octet grp
            constexpr int NF = F::N;
            const int cp = (16 * g) / Gk;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int grp = h * gph + cp;
                const float corr = __shfl_sync(0xffffffffu, accz[0], 4 * grp);    // row grp of the zero-term product
                const int tok0 = tile0 + 128 * h + 16 * g;
                if (tok0 < hi && tig == cp) {                  // 16-token chunks are whole or absent (hi is a group multiple)
                    float *dst = sm.scores + (tok0 - t0);
#pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        const int i0 = (2 * m) % NF, i1 = (2 * m + 1) % NF;
                        float s0 = fmaf(acc[h * 8 + m][0] + acc[h * 8 + m][1], (float)(1 << (24 - F::pos(i0))), corr);
                        float s1 = fmaf(acc[h * 8 + m][2] + acc[h * 8 + m][3], (float)(1 << (24 - F::pos(i1))), corr);
                        if (a.round_scores) {
                            const float2 r = __half22float2(__floats2half2_rn(s0, s1));
                            s0 = r.x;
                            s1 = r.y;
                        }
                        *reinterpret_cast<float2 *>(dst + 2 * m) = make_float2(s0 * a.softmax_scale, s1 * a.softmax_scale);
                    }
                }
            }
        } else {
            // octet g of block bb owns tokens bb*8FH + g*FH ..; in its half of the tile they are in group cp, whose hi and
            // lo sums are the column pair cp, held by the lane with tig == cp; the group's zero term sits in the lanes
            // of octet grp
            const int lgk = 31 - __clz(Gk);                    // group sizes are powers of two here
#pragma unroll
            for (int bb = 0; bb < NBK; ++bb) {
                constexpr int kHalfBlocks = NBK / 2;
                const int h = bb / kHalfBlocks;
                const int cp = (((bb % kHalfBlocks) * 8 * FH) + g * FH) >> lgk;
                const int grp = h * gph + cp;
                const float corr = __shfl_sync(0xffffffffu, accz[0], 4 * grp);    // row grp of the zero-term product
                const int tok0 = tile0 + bb * 8 * FH + g * FH;
                if (tok0 < hi && tig == cp) {                  // FH-token chunks are whole or absent (hi is a group multiple)
                    float *dst = sm.scores + (tok0 - t0);
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
// p . V over packed values for tokens [t0, hi), (hi - t0) % 32 == 0.  sm.scores holds p.  Warp w
// takes 32-token blocks w, w+4, ... through its own ring (codes + scale + zero rows per stage).  Per
// stage the warp first forms the B operands once for all its lanes (p*scale and p*midpoint for 16
// token pairs x 8 columns, half2 per pair) in a small tile, then every lane reads its two B registers
// per k-step with one 32-bit load each.  Returns this warp's 128 partial channel sums in its own
// ring region (float [128] at the region base).
// MODE 1 only issues the first stages (called before the softmax, whose latency then hides the ring fill);
// MODE 2 continues after such a call; MODE 0 does both.
template <int VB, int MODE>
__device__ __forceinline__ void pv_packed_mma(const kvq_attn_args &a, const int32_t *vc, const __half *vs,
                                              const __half *vz, const MmaSmem &sm, int t0, int hi) {
    using G = VGeom<VB>;
    using F = VHalf<VB>;
    constexpr int NB = G::GPT;                                // 16-byte blocks per token row: 1 / 2 / 4
    constexpr int CPB = kHeadDim / NB;                        // channels per block: 128 / 64 / 32
    constexpr int MPB = F::N / 2;                             // MMAs (channel pairs per octet) per block: 8 / 4 / 2
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const int Gv = a.v_group;
    const int ngv = kHeadDim / Gv;                            // channel groups: 4 / 2 / 1
    const int n_blocks = (hi - t0 + G::TPS - 1) / G::TPS;
    const int my_blocks = (n_blocks - warp + kMmaWarps - 1) / kMmaWarps;
    float *my_red = reinterpret_cast<float *>(sm.ring);
    if (my_blocks <= 0) {
        if (MODE != 1)
            for (int i = lane; i < kHeadDim; i += 32) my_red[i] = 0.f;
        return;
    }

    // ---- per-lane constants ----------------------------------------------------------------------
    const uint32_t ring_s = smem_u32(sm.ring);
    const uint32_t pb_s = ring_s + G::PB_OFF;
    // cp.async: granule x = lane + 32 i -> token row tl = x / GPT, granule gr = x % GPT (source is contiguous)
    const int cp_tl0 = lane / G::GPT, cp_gr = lane % G::GPT;
    // rows are XOR-swizzled by token so that the 8 rows x 16 bytes of every ldmatrix tile hit all 32 banks once
    auto swz = [](int tl) { return (VB == 4) ? ((tl >> 1) & 3) : (VB == 2) ? ((tl >> 2) & 1) : 0; };
    const int cp_grs = cp_gr ^ swz(cp_tl0);                                              // (tl + 8 k, 16 k keep the swizzle)
    const uint32_t cp_dst = ring_s + cp_tl0 * G::RBV + cp_grs * 16;                      // + slot*STAGE + i*(32/GPT)*RBV
    // fragment loads: one transposing ldmatrix hands lane (g, tig) the half-word g of a 16-byte block for the
    // token pair (2 tig, 2 tig + 1) in one register, i.e. an A-fragment register pair along k without a byte permute.
    // Tile j of an x4 load (lanes 8j .. 8j+7 give its row addresses): tokens 8 (j & 1) .. +7 of the k-step, block
    // b0 + (j >> 1); the x2 load of 1-bit values has tiles j = 0, 1 only.
    const int ldm_tl = 8 * ((lane >> 3) & 1) + (lane & 7);                               // + 16 h2
    const int ldm_b = (lane >> 4) & (NB - 1);                                            // + b0 (4-bit: 0 or 2)
    const uint32_t ldm_s0 = ring_s + ldm_tl * G::RBV + ((ldm_b ^ swz(ldm_tl)) * 16);
    const uint32_t ldm_s1 = ring_s + ldm_tl * G::RBV + (((ldm_b + 2) & (NB - 1)) ^ swz(ldm_tl)) * 16;   // 4-bit: blocks 2, 3
    // operand tile: pair pi = 8 h2 + 4 b + tig holds tokens (16 h2 + 8 b + 2 tig, +1); reader column g
    const uint32_t pb_rd = pb_s + (tig * 8 + g) * 4;                                     // + (8 h2 + 4 b) * 32
    // operand build: lane -> pair pi = lane & 15, column half ch = lane >> 4 (groups 2ch, 2ch+1)
    const int pi = lane & 15, ch = lane >> 4;
    const int bt0 = 16 * (pi >> 3) + 8 * ((pi >> 2) & 1) + 2 * (pi & 3), bt1 = bt0 + 1;  // the pair's tokens in the stage
    // columns beyond the last channel group repeat that group: finite values in C columns nobody reads
    const int g0 = min(2 * ch, ngv - 1), g1 = min(2 * ch + 1, ngv - 1);
    const uint32_t o00 = ring_s + G::SZ_OFF + (bt0 * ngv + g0) * 2, o01 = ring_s + G::SZ_OFF + (bt0 * ngv + g1) * 2;
    const uint32_t o10 = ring_s + G::SZ_OFF + (bt1 * ngv + g0) * 2, o11 = ring_s + G::SZ_OFF + (bt1 * ngv + g1) * 2;
    const uint32_t pb_wr = pb_s + (pi * 8 + 4 * ch) * 4;

    const int block_stride = kMmaWarps * G::TPS;
    const char *src_codes = reinterpret_cast<const char *>(vc + (int64_t)(t0 + warp * G::TPS) * a.vc_sT) + lane * 16;
    const int ngran = 4 * ngv;                                                           // 16-byte granules per array per stage
    const int sz_arr = lane >= ngran ? 1 : 0;                                            // 0: scale rows, 1: zero rows
    const int sz_off = (lane - sz_arr * ngran) * 16;
    const bool sz_on = lane < 2 * ngran;
    const char *src_sz = reinterpret_cast<const char *>((sz_arr ? vz : vs) + (int64_t)(t0 + warp * G::TPS) * a.vs_sT) + sz_off;
    const uint32_t sz_dst = ring_s + G::SZ_OFF + sz_arr * (G::TPS * 4 * 2) + sz_off;
    const int64_t codes_step = (int64_t)block_stride * G::RBV, sz_step = (int64_t)block_stride * ngv * 2;

    int to_issue = my_blocks;                                                            // blocks not yet issued
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

    float acc[8][4], accz[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
    const uint32_t ones = 0x3c003c00u;
    // The MMA accumulators hold sums of non-negative terms (codes and p are >= 0) whose centred difference is
    // the result, and the tensor core adds into its fp32 accumulator with truncation: measured on a chain of
    // 128 MMAs the sum comes out 1.7e-6 low (1e-7 after 32, exact to 2e-8 when restarted every 16), which the
    // cancellation multiplies by a few hundred at 131k diffuse tokens.  Chains are therefore kept short: every
    // kFlush stages the columns this lane owns are added to fp32 sums (round to nearest) and restart from zero.
    constexpr int kFlush = 16;
    float sum[8][2], sumz[2] = {0.f, 0.f};
#pragma unroll
    for (int m = 0; m < 8; ++m) sum[m][0] = sum[m][1] = 0.f;
    auto flush = [&]() {
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            sum[m][0] += acc[m][0];
            sum[m][1] += acc[m][2];
            acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
        }
        sumz[0] += accz[0];
        sumz[1] += accz[1];
        accz[0] = accz[1] = accz[2] = accz[3] = 0.f;
    };

    if (MODE != 2) {
#pragma unroll
        for (int q = 0; q < G::P; ++q) { issue_stage(q * G::STAGE_BYTES); cp_async_commit(); }
        if (MODE == 1) return;
    } else {                                                   // those stages are already in flight
        to_issue -= G::P;
        src_codes += G::P * codes_step;
        src_sz += G::P * sz_step;
    }

    uint32_t st = 0, issue_st = G::P * G::STAGE_BYTES;         // byte offsets of the slot being read / filled
    const float *pp = sm.scores + warp * G::TPS;               // p of this warp's current block
    for (int q = 0; q < my_blocks; ++q) {
        issue_stage(issue_st);
        cp_async_commit();
        cp_async_wait<G::P>();
        __syncwarp();
        // ---- B operands for the stage: 16 token pairs x 8 columns -----------------------------------
        {
            // p is scaled by 2^8 before the fp16 rounding so that the many small probabilities of a long, diffuse
            // context stay in the normal fp16 range (p <= 1, so this saturates only if a scale exceeds 255)
            const float p0 = pp[bt0] * 256.f, p1 = pp[bt1] * 256.f;
            const float s00 = __half2float(__ushort_as_half((unsigned short)lds16(o00 + st)));
            const float s01 = __half2float(__ushort_as_half((unsigned short)lds16(o01 + st)));
            const float s10 = __half2float(__ushort_as_half((unsigned short)lds16(o10 + st)));
            const float s11 = __half2float(__ushort_as_half((unsigned short)lds16(o11 + st)));
            const float z00 = __half2float(__ushort_as_half((unsigned short)lds16(o00 + st + 256)));
            const float z01 = __half2float(__ushort_as_half((unsigned short)lds16(o01 + st + 256)));
            const float z10 = __half2float(__ushort_as_half((unsigned short)lds16(o10 + st + 256)));
            const float z11 = __half2float(__ushort_as_half((unsigned short)lds16(o11 + st + 256)));
            // columns 4ch .. 4ch+3 = (p*scale_g0, p*mid_g0, p*scale_g1, p*mid_g1), each a half2 over the token pair;
            // mid = zero + MID*scale is the midpoint of the group: codes are used as (code - MID)
            const uint32_t c0 = pack_h2_sat(p0 * s00, p1 * s10);
            const uint32_t c1 = pack_h2_sat(p0 * fmaf(G::MID, s00, z00), p1 * fmaf(G::MID, s10, z10));
            const uint32_t c2 = pack_h2_sat(p0 * s01, p1 * s11);
            const uint32_t c3 = pack_h2_sat(p0 * fmaf(G::MID, s01, z01), p1 * fmaf(G::MID, s11, z11));
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(pb_wr), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
        }
        __syncwarp();
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const uint32_t b0 = lds32(pb_rd + (8 * h2) * 32), b1 = lds32(pb_rd + (8 * h2 + 4) * 32);
            // x[b][0] / x[b][1]: block b, tokens (2 tig, 2 tig + 1) / (2 tig + 8, 2 tig + 9) of the k-step
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
            mma16816(accz, ones, ones, ones, ones, b0, b1);
#pragma unroll
            for (int bb = 0; bb < NB; ++bb) {
                uint32_t rlo[F::N], rhi[F::N];
                F::unpack(x[bb][0], rlo);
                F::unpack(x[bb][1], rhi);
#pragma unroll
                for (int i = 0; i < F::N; i += 2)              // rows g / g+8: channels bb*CPB + g*F::N + i / + i + 1
                    mma16816(acc[bb * MPB + i / 2], rlo[i], rlo[i + 1], rhi[i], rhi[i + 1], b0, b1);
            }
        }
        __syncwarp();
        st = (st + G::STAGE_BYTES == G::NS * G::STAGE_BYTES) ? 0u : st + G::STAGE_BYTES;
        issue_st = (issue_st + G::STAGE_BYTES == G::NS * G::STAGE_BYTES) ? 0u : issue_st + G::STAGE_BYTES;
        pp += block_stride;
        if ((q % kFlush) == kFlush - 1) flush();
    }
    flush();
    cp_async_wait<0>();
    __syncwarp();
    // epilogue: accumulator m = bb * MPB + ip holds channels c = bb*CPB + g*F::N + 2 ip (+1) in rows g (g+8); the column
    // of its group grp = c / Gv (sum p*scale) and the group's correction (sum p*mid, sum p*scale) sit in the lane with
    // tig == grp
    const float corr = (sumz[1] - G::MID * sumz[0]) * (1.f / 256.f);              // undo the 2^8 carried by the B operands
#pragma unroll
    for (int bb = 0; bb < NB; ++bb) {
        const int c0 = bb * CPB + g * F::N;
        if (tig == c0 / Gv) {                                                       // F::N <= 16 <= Gv: one group per octet block
#pragma unroll
            for (int ip = 0; ip < MPB; ++ip) {
                my_red[c0 + 2 * ip] = fmaf(sum[bb * MPB + ip][0], (float)(1 << (16 - F::pos(2 * ip))), corr);
                my_red[c0 + 2 * ip + 1] = fmaf(sum[bb * MPB + ip][1], (float)(1 << (16 - F::pos(2 * ip + 1))), corr);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// q . K^T over the fp16 tail for tokens [lo, t1): 16-token tiles on the tensor core, straight from
// global memory (row g and g+8 of a tile per lane-octet, 16-byte loads of 8 channels; the k axis is
// permuted identically in the q fragments).  Every B column carries q, so each lane sees its rows' sums.
__device__ __forceinline__ void qk_tail_mma(const kvq_attn_args &a, const __half *kf, int b, int hk, const MmaSmem &sm,
                                            int t0, int lo, int t1) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    uint4 qf[4];
#pragma unroll
    for (int S = 0; S < 4; ++S) qf[S] = *reinterpret_cast<const uint4 *>(sm.q + 32 * S + 8 * tig);
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
        if (tig == 0) {
            float s0 = c[0], s1 = c[2];
            if (a.round_scores) {
                const float2 r = __half22float2(__floats2half2_rn(s0, s1));
                s0 = r.x;
                s1 = r.y;
            }
            if (ta < t1) sm.scores[ta - t0] = s0 * a.softmax_scale;
            if (tb < t1) sm.scores[tb - t0] = s1 * a.softmax_scale;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// One segment: tokens [t0, t1) of query head (b, h); segment `seg` of the `cnt` the head is cut into.
template <int KB, int VB>
__device__ __forceinline__ void attn_segment(const kvq_attn_args &a, const kvq_attn_args &ac, int n_scores, int s, int t0, int t1, int seg,
                                             int cnt, int n_whole, float *__restrict__ parts,
                                             unsigned int *__restrict__ counters) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    MmaSmem sm;
    sm.scores = reinterpret_cast<float *>(smem_raw);
    unsigned char *after_scores = smem_raw + (size_t)n_scores * 4;
    sm.ring = after_scores + warp * warp_region_bytes<KB, VB>();
    sm.tailred = reinterpret_cast<float *>(after_scores + kMmaWarps * warp_region_bytes<KB, VB>());
    sm.q = reinterpret_cast<__half *>(sm.tailred + kMmaWarps * kHeadDim);
    sm.misc = reinterpret_cast<float *>(sm.q + kHeadDim);
    const int b = s / a.nh, h = s % a.nh;
    // grouped queries: each query head is its own segment and reads kv head hk; the heads of one kv head are
    // neighbouring units of work, so the cache is fetched from HBM once and re-read from L2
    const int hk = h / (a.nh / a.nh_kv);

    fused_cache_update<KB, VB>(a, b, hk, t0, t1, tid);        // the step's own cache update, when the caller fused it in
    const __half *q = static_cast<const __half *>(a.q) + (int64_t)b * a.q_sB + (int64_t)h * a.q_sH;
    if (tid < kHeadDim) sm.q[tid] = q[tid];
    for (int i = tid; i < kMmaWarps * kHeadDim; i += kMmaThreads) sm.tailred[i] = 0.f;

    // ---- 1. scores ------------------------------------------------------------------------------
    {
        const int hi = min(t1, a.Tkq);
        if (t0 < hi) {
            const int32_t *kc = a.kcode + (int64_t)b * a.kc_sB + (int64_t)hk * a.kc_sH;
            const __half *ks = static_cast<const __half *>(a.kscale) + (int64_t)b * a.ks_sB + (int64_t)hk * a.ks_sH;
            const __half *kz = static_cast<const __half *>(a.kmn) + (int64_t)b * a.ks_sB + (int64_t)hk * a.ks_sH;
            const __half *kf = static_cast<const __half *>(a.kfull) + (int64_t)b * a.kf_sB + (int64_t)hk * a.kf_sH;
            qk_packed_mma<KB>(a, kc, ks, kz, sm, t0, hi, kf, max(t0, a.Tkq), t1, b, hk);
        } else {
            __syncthreads();                                   // q is in shared memory
            const __half *kf = static_cast<const __half *>(a.kfull) + (int64_t)b * a.kf_sB + (int64_t)hk * a.kf_sH;
            if (t0 < t1) qk_tail_mma(a, kf, b, hk, sm, t0, t0, t1);
        }
    }
    const int32_t *vc = a.vcode + (int64_t)b * a.vc_sB + (int64_t)hk * a.vc_sH;
    const __half *vs = static_cast<const __half *>(a.vscale) + (int64_t)b * a.vs_sB + (int64_t)hk * a.vs_sH;
    const __half *vz = static_cast<const __half *>(a.vmn) + (int64_t)b * a.vs_sB + (int64_t)hk * a.vs_sH;
    const int v_hi = min(t1, a.Tvq);
    if (t0 < v_hi) pv_packed_mma<VB, 1>(a, vc, vs, vz, sm, t0, v_hi);   // start filling this warp's value ring now
    __syncthreads();

    // ---- 2. softmax numerators ------------------------------------------------------------------
    // The fp16 value tail of this split (the window: usually <= 128 tokens) is fetched into registers first, so its
    // global-load latency is spent under the two softmax passes.  Thread (co, tl) owns 8 channels and tokens
    // v_lo + tl + 8 j; rounds of 128 tokens, the first one preloaded.
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

    float m = kMaskFloor;                                      // a fully masked range then weighs uniformly, as upstream's does
    const int n4 = (n + 3) >> 2;
    float4 *sc4 = reinterpret_cast<float4 *>(sm.scores);
#pragma unroll 4
    for (int i = tid; i < n4; i += kMmaThreads) {
        float4 v = sc4[i];
        if (a.mask) {                                          // weights + mask, clamped at the fp32 floor
            const int t = t0 + 4 * i;
            v.x = fmaxf(v.x + attn_mask_at(a, b, h, min(t, a.T - 1)), kMaskFloor);
            v.y = fmaxf(v.y + attn_mask_at(a, b, h, min(t + 1, a.T - 1)), kMaskFloor);
            v.z = fmaxf(v.z + attn_mask_at(a, b, h, min(t + 2, a.T - 1)), kMaskFloor);
            v.w = fmaxf(v.w + attn_mask_at(a, b, h, min(t + 3, a.T - 1)), kMaskFloor);
            sc4[i] = v;
        }
        if (4 * i + 3 >= n) {                                  // the last, partial quad: neutral padding
            if (4 * i + 1 >= n) v.y = -INFINITY;
            if (4 * i + 2 >= n) v.z = -INFINITY;
            v.w = -INFINITY;
            sc4[i] = v;
        }
        m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
    m = warp_max(m);
    if (lane == 0) sm.misc[warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(sm.misc[0], sm.misc[1]), fmaxf(sm.misc[2], sm.misc[3]));
    float l = 0.f;
#pragma unroll 4
    for (int i = tid; i < n4; i += kMmaThreads) {
        float4 v = sc4[i];
        v.x = __expf(v.x - m);
        v.y = __expf(v.y - m);
        v.z = __expf(v.z - m);
        v.w = __expf(v.w - m);
        sc4[i] = v;
        l += (v.x + v.y) + (v.z + v.w);
    }
    l = warp_sum(l);
    if (lane == 0) sm.misc[4 + warp] = l;
    __syncthreads();
    l = (sm.misc[4] + sm.misc[5]) + (sm.misc[6] + sm.misc[7]);

    // ---- 3. p.V -----------------------------------------------------------------------------------
    if (v_lo < t1) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int base = v_lo; base < t1; base += 128) {
            if (base > v_lo) load_tail_round(base);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int t = base + tl + 8 * j;
                const float p = (t < t1) ? sm.scores[t - t0] : 0.f;
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
        for (int k = 0; k < 8; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 16);   // the warp's two token lanes
        if (lane < 16) {
            float4 *dst = reinterpret_cast<float4 *>(sm.tailred + warp * kHeadDim + 8 * co);
            dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
    }
    if (t0 < v_hi) pv_packed_mma<VB, 2>(a, vc, vs, vz, sm, t0, v_hi);
    __syncthreads();

    // ---- 4. finish / merge --------------------------------------------------------------------------
    float o = (sm.tailred[tid] + sm.tailred[kHeadDim + tid]) + (sm.tailred[2 * kHeadDim + tid] + sm.tailred[3 * kHeadDim + tid]);
    if (t0 < min(t1, a.Tvq)) {                               // each warp left its packed-value partial at its region base
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w)
            o += reinterpret_cast<const float *>(after_scores + w * warp_region_bytes<KB, VB>())[tid];
    }
    __half *out = static_cast<__half *>(a.out) + (int64_t)b * a.o_sB + (int64_t)h * a.o_sH;
    if (cnt == 1) {
        const __half r[1] = {__float2half_rn(o / l)};
        out[tid] = r[0];
        peer_publish(ac, b, h, 1, r, tid);
        return;
    }
    constexpr int kPart = kPartStride;
    float *part = parts + ((int64_t)(s - n_whole) * cnt + seg) * kPart;          // partials of the cut heads only
    part[tid] = o;
    if (tid == 0) { part[kHeadDim] = m; part[kHeadDim + 1] = l; }
    __syncthreads();
    if (tid == 0) {
        // one cumulative device-scope fence after the CTA barrier publishes every thread's partial before the count;
        // the fence after the count orders the merging CTA's reads (ld.cg, from L2) behind the other CTAs' fences
        __threadfence();
        sm.misc[8] = (atomicAdd(&counters[s], 1u) == (unsigned)(cnt - 1)) ? 1.f : 0.f;
        __threadfence();
    }
    __syncthreads();
    if (sm.misc[8] == 0.f) return;
    const float *base = parts + (int64_t)(s - n_whole) * cnt * kPart;
    float M = kMaskFloor;
    for (int i = 0; i < cnt; ++i) M = fmaxf(M, __ldcg(base + i * kPart + kHeadDim));
    float L = 0.f, acc = 0.f;
    for (int i = 0; i < cnt; ++i) {
        const float w = __expf(__ldcg(base + i * kPart + kHeadDim) - M);
        L = fmaf(__ldcg(base + i * kPart + kHeadDim + 1), w, L);
        acc = fmaf(__ldcg(base + i * kPart + tid), w, acc);
    }
    const __half r[1] = {__float2half_rn(acc / L)};
    out[tid] = r[0];
    if (tid == 0) counters[s] = 0u;                          // the head is done: its counter is ready for the next launch
    peer_publish(ac, b, h, 1, r, tid);
}

// CTA = one segment (see attn_plan.cuh): a whole head, or one of the k pieces of a head that is cut.
// DEV: lengths and ring starts come from the device-resident state (attn_update.cuh); the plan was laid out for an
// upper bound of the length, so segments beyond the real length are empty and a head counts fewer of them.
template <int KB, int VB, bool DEV>
__global__ void __launch_bounds__(kMmaThreads, 3) decode_attn_mma_kernel(const __grid_constant__ kvq_attn_args a,
                                                                     const __grid_constant__ AttnPlan plan,
                                                                     float *__restrict__ parts,
                                                                     unsigned int *__restrict__ counters) {
    int head, t0, t1, seg, cnt;
    if constexpr (DEV) {
        kvq_attn_args b = a;
        dev_state_step(a, b);
        plan_cta(plan, b.T, blockIdx.x, head, t0, t1, seg, cnt);
        if (cnt > 1) cnt = min(cnt, (b.T + plan.seg_units * plan.unit - 1) / (plan.seg_units * plan.unit));
        if (t0 < b.T) attn_segment<KB, VB>(b, a, plan.n_scores, head, t0, t1, seg, cnt, plan.n_whole, parts, counters);
    } else {
        plan_cta(plan, a.T, blockIdx.x, head, t0, t1, seg, cnt);
        attn_segment<KB, VB>(a, a, plan.n_scores, head, t0, t1, seg, cnt, plan.n_whole, parts, counters);
    }
}

// ---------------------------------------------------------------------------------------------
// The tensor-core path needs a whole number of query heads per kv head, supported group sizes, 16-byte aligned
// and row-contiguous packed tensors (cp.async granules), and a packed-value length that is a multiple of 32.
bool mma_path_eligible(const kvq_attn_args &a) {
    if (a.nh_kv <= 0 || a.nh % a.nh_kv != 0 || a.D != kHeadDim) return false;
    if (a.k_bits == 3) {
        if (a.k_group != 11) return false;
    } else if (a.k_group != 32 && a.k_group != 64 && a.k_group != 128) {
        return false;
    }
    if (a.v_bits == 3) return false;
    if (a.v_group != 32 && a.v_group != 64 && a.v_group != 128) return false;
    if (a.Tvq % 32 != 0) return false;
    auto al16 = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (a.T > a.Tkq && (!al16(a.kfull) || a.kf_sB % 8 || a.kf_sH % 8 || a.kf_sT % 8)) return false;
    if (a.T > a.Tvq && (!al16(a.vfull) || a.vf_sB % 8 || a.vf_sH % 8 || a.vf_sT % 8)) return false;
    if (a.Tkq > 0) {
        if (!al16(a.kcode) || a.kc_sB % 4 || a.kc_sH % 4 || a.kc_sD % 4) return false;
        if (!al16(a.kscale) || !al16(a.kmn) || a.ks_sB % 8 || a.ks_sH % 8 || a.ks_sD % 8) return false;
    }
    if (a.Tvq > 0) {
        const int fv = fields_per_word(a.v_bits);
        if (!al16(a.vcode) || a.vc_sB % 4 || a.vc_sH % 4 || a.vc_sT != kHeadDim / fv) return false;
        if (!al16(a.vscale) || !al16(a.vmn) || a.vs_sB % 8 || a.vs_sH % 8 || a.vs_sT != kHeadDim / a.v_group) return false;
    }
    return true;
}

template <int KB, int VB>
static int launch_mma(const kvq_attn_args &a, const AttnPlan &plan, float *parts, unsigned int *counters,
                      cudaStream_t st) {
    const size_t smem = (size_t)plan.n_scores * 4 + (size_t)kMmaWarps * warp_region_bytes<KB, VB>() +
                        kMmaWarps * kHeadDim * 4 + kHeadDim * 2 + 16 * 4;
    static bool attr_set[64] = {};                           // per device: the opt-in is sticky for the process
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        e = cudaFuncSetAttribute(decode_attn_mma_kernel<KB, VB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(decode_attn_mma_kernel<KB, VB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const unsigned grid = (unsigned)(plan.n_whole + plan.n_cut * plan.k);
    if (a.state) decode_attn_mma_kernel<KB, VB, true><<<grid, kMmaThreads, smem, st>>>(a, plan, parts, counters);
    else decode_attn_mma_kernel<KB, VB, false><<<grid, kMmaThreads, smem, st>>>(a, plan, parts, counters);
    return check_launch();
}

int launch_decode_attn_mma(const kvq_attn_args &a, const AttnPlan &plan, float *parts, unsigned int *counters,
                           cudaStream_t st) {
#define KVQ_MMA_CASE(KB, VB) \
    if (a.k_bits == KB && a.v_bits == VB) return launch_mma<KB, VB>(a, plan, parts, counters, st);
    KVQ_MMA_CASE(4, 4) KVQ_MMA_CASE(4, 2) KVQ_MMA_CASE(4, 1)
    KVQ_MMA_CASE(3, 4) KVQ_MMA_CASE(3, 2) KVQ_MMA_CASE(3, 1)
    KVQ_MMA_CASE(2, 4) KVQ_MMA_CASE(2, 2) KVQ_MMA_CASE(2, 1)
    KVQ_MMA_CASE(1, 4) KVQ_MMA_CASE(1, 2) KVQ_MMA_CASE(1, 1)
#undef KVQ_MMA_CASE
    return KVQ_ERR_UNSUPPORTED;
}

// Plan of the tensor-core kernel for B * nh query heads (one head per segment).
AttnPlan plan_attn_mma(int T, int k_bits, long long heads) {
    const int unit = (k_bits == 3) ? 352 : 256;              // one key tile per warp
    const int max_chunk = (k_bits == 3) ? 8096 : 8192;       // scores held in shared memory
    return make_attn_plan(T, unit, max_chunk, heads, kSmCount * 3, k_bits == 3 ? 1 : kMmaWarps);
}

}  // namespace kvq
