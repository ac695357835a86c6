// The arithmetic core of the group quantizer, shared by the stand-alone quantizer kernels (quant.cu) and by the
// attention kernels' fused cache update (attn_update.cuh): bit-identical to upstream
// quant_cuda/csrc/quantization_cuda.cu:553-596 with IEEE division.
#pragma once
#include "common.cuh"

namespace kvq {

// q = clamp(roundf(n), 0, emax) for n >= 0 or NaN.  n - trunc(n) is exact for these magnitudes,
// so comparing the fraction with 0.5 is roundf's half-away-from-zero rule.
__device__ __forceinline__ int round_code(float n, int emax) {
    int k = (n == n) ? __float2int_rz(n) : 0;
    float frac = n - (float)k;
    k += (frac >= 0.5f) ? 1 : 0;
    return max(0, min(k, emax));
}

// One packed word of E = fields_per_word(BITS) consecutive elements get(0..E-1) of a group with minimum lo, scale
// sc and rinv = fl(1/sc), bit-identical to OR_i clamp(roundf((v_i - lo) / sc), 0, emax_i) << shift_i with IEEE
// division -- without a division, an int conversion or a clamp per element:
//   m  = fma(a, rinv, 1.5 * 2^23), a = v - lo     the addition rounds a*rinv to the nearest integer (low mantissa bits)
//   yr = m - 1.5 * 2^23                          that integer as a float (exact)
//   e  = fma(a, rinv, -yr)                       signed distance of a*rinv from it, in [-0.5, 0.5]
// a*rinv and the IEEE quotient differ by < 1.3e-7 relative (< 2e-6 for codes up to 15), so unless |e| is within
// 1e-5 of 0.5 both round to the same integer, whatever the tie rule; 0 <= a*rinv <= qmax (1 + 2e-7) keeps it in
// range.  The word is summed in two fp32 chunks of <= 17 bits (exact) and converted once.  If any element is near
// a tie or not finite (constant group: 0 * inf), the whole word is redone with the exact division.
template <int BITS, typename Get>
__device__ __forceinline__ uint32_t quant_word(Get get, float lo, float sc, float rinv) {
    constexpr int E = fields_per_word(BITS);
    constexpr int QMAX = (1 << BITS) - 1;
    constexpr int NLO = (BITS == 3) ? 5 : E / 2;               // fields in the low chunk
    constexpr int HI_SHIFT = (BITS == 3) ? 15 : BITS * NLO;
    constexpr float kMagic = 12582912.0f;
    float wl = 0.f, wh = 0.f;
    bool ok = true;
#pragma unroll
    for (int i = 0; i < E; ++i) {
        const float a = get(i) - lo;
        const float m = fmaf(a, rinv, kMagic);
        float yr = m - kMagic;
        const float e = fmaf(a, rinv, -yr);
        ok = ok && (fabsf(e) <= 0.49999f);
        if (BITS == 3 && i == 10) yr = fminf(yr, 3.f);          // the 11th code of a 3-bit group has two bits
        if (i < NLO) {
            wl = fmaf(yr, (float)(1 << (BITS * i)), wl);
        } else {
            const int sh = (BITS == 3) ? (i < 10 ? 3 * (i - 5) : 15) : BITS * (i - NLO);
            wh = fmaf(yr, (float)(1 << sh), wh);
        }
    }
    if (ok) return __float2uint_rz(wl) | (__float2uint_rz(wh) << HI_SHIFT);
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < E; ++i) {
        const float n = (get(i) - lo) / sc;
        if (BITS == 3) word |= (uint32_t)round_code(n, i < 10 ? 7 : 3) << (i < 10 ? 3 * i : 30);
        else word |= (uint32_t)round_code(n, QMAX) << (BITS * i);
    }
    return word;
}

template <int QMAX>
__device__ __forceinline__ float stored_scale(float range, float quotient, int by_div) {
    return by_div ? quotient : __fmul_rn(range, 1.0f / (float)QMAX);
}

}  // namespace kvq
