// Building blocks shared by the tensor-core attention kernels: mma.sync / cp.async / ldmatrix wrappers, the
// in-place field extraction that turns packed codes into fp16 subnormal operands, and the per-bit-width
// geometry of the per-warp cp.async rings.
#pragma once
#include "common.cuh"

namespace kvq {

constexpr int kMmaThreads = 128;
constexpr int kMmaWarps = 4;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// ---------------------------------------------------------------------------------------------
// Field extraction.  unpack(wa, wb, r): r[i] = fp16x2 { field i of wa (low), field i of wb (high) }
// left at bit position pos(i) inside each 16-bit half, i.e. the subnormal pair
// { f_a * 2^(pos-24), f_b * 2^(pos-24) }.  inv_scale(i) = 2^(24-pos(i)).
template <int BITS> struct Fields;

template <> struct Fields<4> {
    static constexpr int N = 8;
    __device__ static __forceinline__ int pos(int i) { return (i & 1) ? 4 : 0; }
    __device__ static __forceinline__ void unpack(uint32_t wa, uint32_t wb, uint32_t (&r)[8]) {
        const uint32_t lo = prmt(wa, wb, 0x5410), hi = prmt(wa, wb, 0x7632);
        const uint32_t los = lo >> 8, his = hi >> 8;
        r[0] = lo & 0x000f000fu; r[1] = lo & 0x00f000f0u; r[2] = los & 0x000f000fu; r[3] = los & 0x00f000f0u;
        r[4] = hi & 0x000f000fu; r[5] = hi & 0x00f000f0u; r[6] = his & 0x000f000fu; r[7] = his & 0x00f000f0u;
    }
};

template <> struct Fields<2> {
    static constexpr int N = 16;
    __device__ static __forceinline__ int pos(int i) { const int t = i & 7; return t < 5 ? 2 * t : 2 * (t - 5); }
    __device__ static __forceinline__ void unpack(uint32_t wa, uint32_t wb, uint32_t (&r)[16]) {
        const uint32_t lo = prmt(wa, wb, 0x5410), hi = prmt(wa, wb, 0x7632);
        const uint32_t los = lo >> 10, his = hi >> 10;
#pragma unroll
        for (int t = 0; t < 5; ++t) { r[t] = lo & (0x00030003u << (2 * t)); r[8 + t] = hi & (0x00030003u << (2 * t)); }
#pragma unroll
        for (int t = 5; t < 8; ++t) {
            r[t] = los & (0x00030003u << (2 * (t - 5)));
            r[8 + t] = his & (0x00030003u << (2 * (t - 5)));
        }
    }
};

template <> struct Fields<1> {
    static constexpr int N = 32;
    __device__ static __forceinline__ int pos(int i) { const int t = i & 15; return t < 10 ? t : t - 10; }
    __device__ static __forceinline__ void unpack(uint32_t wa, uint32_t wb, uint32_t (&r)[32]) {
        const uint32_t lo = prmt(wa, wb, 0x5410), hi = prmt(wa, wb, 0x7632);
        const uint32_t los = lo >> 10, his = hi >> 10;
#pragma unroll
        for (int t = 0; t < 10; ++t) { r[t] = lo & (0x00010001u << t); r[16 + t] = hi & (0x00010001u << t); }
#pragma unroll
        for (int t = 10; t < 16; ++t) { r[t] = los & (0x00010001u << (t - 10)); r[16 + t] = his & (0x00010001u << (t - 10)); }
    }
};

// 3-bit words: fields 0..9 at bits 3i, field 10 (2 bits) at bit 30.
template <> struct Fields<3> {
    static constexpr int N = 11;
    __device__ static __forceinline__ int pos(int i) {
        constexpr int P[11] = {0, 3, 6, 0, 3, 0, 3, 6, 0, 3, 0};
        return P[i];
    }
    __device__ static __forceinline__ void unpack(uint32_t wa, uint32_t wb, uint32_t (&r)[11]) {
        const uint32_t x0 = prmt(wa, wb, 0x5410), x1 = x0 >> 9;
        const uint32_t y = prmt(wa >> 15, wb >> 15, 0x5410), y1 = y >> 9;
        const uint32_t z1 = prmt(wa, wb, 0x7632) >> 14;
        r[0] = x0 & 0x00070007u; r[1] = x0 & 0x00380038u; r[2] = x0 & 0x01c001c0u;
        r[3] = x1 & 0x00070007u; r[4] = x1 & 0x00380038u;
        r[5] = y & 0x00070007u; r[6] = y & 0x00380038u; r[7] = y & 0x01c001c0u;
        r[8] = y1 & 0x00070007u; r[9] = y1 & 0x00380038u;
        r[10] = z1 & 0x00030003u;
    }
};

// Value-side field extraction: same contract as Fields, but every field is moved to bit position >= 4 (>= 2
// for 4-bit codes) of its 16-bit half.  The tensor core aligns the 16 products of an MMA (and the accumulator) to
// the largest operand EXPONENT and truncates what falls about 26 bits below it; a subnormal's exponent is fixed at
// -14 however small its value, so a code parked in the lowest mantissa bits loses low product bits whenever a
// neighbouring token's probability is larger.  The loss is always downwards, so over a long, diffuse softmax it
// adds up to a bias (2e-5 of the non-negative code sum for 2-bit codes at position 0, a quarter of that per two
// positions higher) which the centring of the codes amplifies.  Two more shifts per word pair keep it below the
// fp32 accumulation error.
template <int BITS> struct VFields;

template <> struct VFields<4> {
    static constexpr int N = 8;
    __device__ static __forceinline__ int pos(int i) { return (i & 1) ? 6 : 2; }
    __device__ static __forceinline__ void unpack(uint32_t wa, uint32_t wb, uint32_t (&r)[8]) {
        const uint32_t lo = prmt(wa, wb, 0x5410), hi = prmt(wa, wb, 0x7632);
        const uint32_t lou = lo << 2, lod = lo >> 6, hiu = hi << 2, hid = hi >> 6;
        r[0] = lou & 0x003c003cu; r[1] = lou & 0x03c003c0u; r[2] = lod & 0x003c003cu; r[3] = lod & 0x03c003c0u;
        r[4] = hiu & 0x003c003cu; r[5] = hiu & 0x03c003c0u; r[6] = hid & 0x003c003cu; r[7] = hid & 0x03c003c0u;
    }
};

template <> struct VFields<2> {
    static constexpr int N = 16;
    __device__ static __forceinline__ int pos(int i) { const int t = i & 7; return t < 2 ? 6 + 2 * t : t < 5 ? 2 * t : 2 * t - 6; }
    __device__ static __forceinline__ void unpack(uint32_t wa, uint32_t wb, uint32_t (&r)[16]) {
        const uint32_t lo = prmt(wa, wb, 0x5410), hi = prmt(wa, wb, 0x7632);
        const uint32_t lou = lo << 6, lod = lo >> 6, hiu = hi << 6, hid = hi >> 6;
#pragma unroll
        for (int t = 0; t < 2; ++t) { r[t] = lou & (0x00030003u << (6 + 2 * t)); r[8 + t] = hiu & (0x00030003u << (6 + 2 * t)); }
#pragma unroll
        for (int t = 2; t < 5; ++t) { r[t] = lo & (0x00030003u << (2 * t)); r[8 + t] = hi & (0x00030003u << (2 * t)); }
#pragma unroll
        for (int t = 5; t < 8; ++t) { r[t] = lod & (0x00030003u << (2 * t - 6)); r[8 + t] = hid & (0x00030003u << (2 * t - 6)); }
    }
};

template <> struct VFields<1> {
    static constexpr int N = 32;
    __device__ static __forceinline__ int pos(int i) { const int t = i & 15; return t < 4 ? t + 6 : t < 10 ? t : t - 6; }
    __device__ static __forceinline__ void unpack(uint32_t wa, uint32_t wb, uint32_t (&r)[32]) {
        const uint32_t lo = prmt(wa, wb, 0x5410), hi = prmt(wa, wb, 0x7632);
        const uint32_t lou = lo << 6, lod = lo >> 6, hiu = hi << 6, hid = hi >> 6;
#pragma unroll
        for (int t = 0; t < 4; ++t) { r[t] = lou & (0x00010001u << (t + 6)); r[16 + t] = hiu & (0x00010001u << (t + 6)); }
#pragma unroll
        for (int t = 4; t < 10; ++t) { r[t] = lo & (0x00010001u << t); r[16 + t] = hi & (0x00010001u << t); }
#pragma unroll
        for (int t = 10; t < 16; ++t) { r[t] = lod & (0x00010001u << (t - 6)); r[16 + t] = hid & (0x00010001u << (t - 6)); }
    }
};

// Key-side extraction from ONE register that already pairs the same 16-bit half-word of two channel rows (as a
// transposing ldmatrix delivers them): r[i] = fp16x2 of field i of both half-words, i < 16 / BITS, at bit position
// Fields<BITS>::pos(i).
template <int BITS> struct KHalf;
template <> struct KHalf<4> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void unpack(uint32_t x, uint32_t (&r)[4]) {
        const uint32_t xs = x >> 8;
        r[0] = x & 0x000f000fu; r[1] = x & 0x00f000f0u; r[2] = xs & 0x000f000fu; r[3] = xs & 0x00f000f0u;
    }
};
template <> struct KHalf<2> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void unpack(uint32_t x, uint32_t (&r)[8]) {
        const uint32_t xs = x >> 10;
#pragma unroll
        for (int t = 0; t < 5; ++t) r[t] = x & (0x00030003u << (2 * t));
#pragma unroll
        for (int t = 5; t < 8; ++t) r[t] = xs & (0x00030003u << (2 * (t - 5)));
    }
};
template <> struct KHalf<1> {
    static constexpr int N = 16;
    __device__ static __forceinline__ void unpack(uint32_t x, uint32_t (&r)[16]) {
        const uint32_t xs = x >> 10;
#pragma unroll
        for (int t = 0; t < 10; ++t) r[t] = x & (0x00010001u << t);
#pragma unroll
        for (int t = 10; t < 16; ++t) r[t] = xs & (0x00010001u << (t - 10));
    }
};
template <> struct KHalf<3> {                       // 3-bit keys do not use this path (11 fields do not split into half-words)
    static constexpr int N = 2;
    __device__ static __forceinline__ void unpack(uint32_t, uint32_t (&)[2]) {}
};

// Value-side extraction from ONE register that already pairs two 16-bit half-words along the contraction axis (as
// a transposing ldmatrix delivers them): r[i] = fp16x2 of field i of both half-words, i < 16 / BITS, each left at
// bit position pos(i) >= 4 (>= 2 for 4-bit codes) of its half -- the positions VFields uses, for the same reason.
template <int BITS> struct VHalf;
template <> struct VHalf<4> {
    static constexpr int N = 4;
    __device__ static __forceinline__ int pos(int i) { return (i & 1) ? 6 : 2; }
    __device__ static __forceinline__ void unpack(uint32_t x, uint32_t (&r)[4]) {
        const uint32_t xu = x << 2, xd = x >> 6;
        r[0] = xu & 0x003c003cu; r[1] = xu & 0x03c003c0u; r[2] = xd & 0x003c003cu; r[3] = xd & 0x03c003c0u;
    }
};
template <> struct VHalf<2> {
    static constexpr int N = 8;
    __device__ static __forceinline__ int pos(int i) { return i < 2 ? 6 + 2 * i : i < 5 ? 2 * i : 2 * i - 6; }
    __device__ static __forceinline__ void unpack(uint32_t x, uint32_t (&r)[8]) {
        const uint32_t xu = x << 6, xd = x >> 6;
#pragma unroll
        for (int t = 0; t < 2; ++t) r[t] = xu & (0x00030003u << (6 + 2 * t));
#pragma unroll
        for (int t = 2; t < 5; ++t) r[t] = x & (0x00030003u << (2 * t));
#pragma unroll
        for (int t = 5; t < 8; ++t) r[t] = xd & (0x00030003u << (2 * t - 6));
    }
};
template <> struct VHalf<1> {
    static constexpr int N = 16;
    __device__ static __forceinline__ int pos(int i) { return i < 4 ? i + 6 : i < 10 ? i : i - 6; }
    __device__ static __forceinline__ void unpack(uint32_t x, uint32_t (&r)[16]) {
        const uint32_t xu = x << 6, xd = x >> 6;
#pragma unroll
        for (int t = 0; t < 4; ++t) r[t] = xu & (0x00010001u << (t + 6));
#pragma unroll
        for (int t = 4; t < 10; ++t) r[t] = x & (0x00010001u << t);
#pragma unroll
        for (int t = 10; t < 16; ++t) r[t] = xd & (0x00010001u << (t - 6));
    }
};

// ---------------------------------------------------------------------------------------------
// Key-side geometry per bit width.  A warp tile is 8 lane-octets x TPO tokens; code words reach the
// warp through its own ring of cp.async stages in shared memory (padded rows so the fragment loads
// are bank-conflict free), three stages in flight ahead of the math.  All shared-memory offsets are
// compile-time constants relative to one per-lane base; global addresses advance by per-stage strides.
template <int KB> struct KGeom {
    static constexpr int FPI = fields_per_word(KB);
    static constexpr int WPL = (KB == 4) ? 4 : (KB == 2) ? 2 : 1;     // words per octet: 32 tokens (11 for 3-bit)
    static constexpr int TPO = WPL * FPI;                              // tokens per octet chunk
    static constexpr int WT = 8 * TPO;                                 // tokens per warp tile (256 / 88)
    static constexpr int KSPS = (KB == 4) ? 1 : 2;                     // k-steps (16 channels) per stage
    static constexpr int NSTAGE = 8 / KSPS;                            // stages per warp tile: 8 / 4
    static constexpr int NMMA = (TPO + 1) / 2;                         // MMAs (token pairs) per octet chunk
    static constexpr int RB = 32 * WPL;                                // code bytes per channel row per warp tile
    static constexpr int RS = RB + 16;                                 // padded row stride in the ring
    static constexpr int ROWS = 16 * KSPS;                             // channel rows per stage
    static constexpr int STAGE_BYTES = ROWS * RS;                      // 2304 / 2560 / 1536
    static constexpr int GPR = RB / 16;                                // 16-byte granules per row: 8 / 4 / 2
    static constexpr int GPL = ROWS * GPR / 32;                        // granules per lane per stage: 4 / 4 / 2
    static constexpr int RPI = 32 / GPR;                               // rows between a lane's granules
    static constexpr int NS = 4;                                       // ring slots (NSTAGE % NS == 0: slots are static)
    static constexpr int P = NS - 1;                                   // stages in flight
    static constexpr int SZ_BYTES = 2 * kHeadDim * 16;                 // scale + zero tile: 16 B per channel row
    static constexpr int WARP_BYTES = NS * STAGE_BYTES + SZ_BYTES;
    static constexpr float MID = (float)((1 << KB) - 1) * 0.5f;        // codes are centred on the group midpoint
};

template <int WPL> struct WordVec;
template <> struct WordVec<1> { using T = uint32_t; };
template <> struct WordVec<2> { using T = uint2; };
template <> struct WordVec<4> { using T = uint4; };

template <int VB> struct VGeom {
    static constexpr int FPI = fields_per_word(VB);
    static constexpr int RBV = kHeadDim / FPI * 4;                     // code bytes per token row: 64 / 32 / 16
    static constexpr int TPS = 32;                                     // tokens per stage (2 k-steps)
    static constexpr int GPT = RBV / 16;                               // granules per token row: 4 / 2 / 1
    static constexpr int GPL = (TPS * GPT + 31) / 32;                  // code granules per lane per stage: 4 / 2 / 1
    static constexpr int SZ_OFF = TPS * RBV;                           // scale rows, then zero rows (<= 4 groups each)
    static constexpr int STAGE_BYTES = TPS * RBV + 2 * TPS * 4 * 2;
    static constexpr int NS = (VB == 4) ? 4 : (VB == 2) ? 6 : 8;
    static constexpr int P = NS - 1;
    static constexpr int PB_OFF = NS * STAGE_BYTES;                    // operand tile p*scale / p*mid: 16 token pairs x 8 cols
    static constexpr int WARP_BYTES = NS * STAGE_BYTES + 16 * 8 * 4;
    static constexpr float MID = (float)((1 << VB) - 1) * 0.5f;
};

template <int KB, int VB> constexpr int warp_region_bytes() {
    return KGeom<KB>::WARP_BYTES > VGeom<VB>::WARP_BYTES ? KGeom<KB>::WARP_BYTES : VGeom<VB>::WARP_BYTES;
}

template <int BYTES>
__device__ __forceinline__ void cp_async(uint32_t smem_addr, const void *gmem) {
    if constexpr (BYTES == 16) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gmem));
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(smem_addr), "l"(gmem), "n"(BYTES));
    }
}
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
    return v;
}
// {lo, hi} -> fp16x2, round to nearest, saturating to the largest finite fp16 instead of overflowing to inf
__device__ __forceinline__ uint32_t pack_h2_sat(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

}  // namespace kvq
