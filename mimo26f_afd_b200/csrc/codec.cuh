// Bit-exact FP8 E4M3 / UE8M0-K32 block codecs, integer arithmetic only.
//
// Two codecs live on the expert path and they round differently:
//   * wire codec   - the coordinator's activation quantiser: scale byte
//     clamp(ceil(log2(amax/448)) + 127, 0, 254), zero block -> byte 0, payload
//     rounded to nearest with ties to the larger magnitude, clamp +-448,
//     NaN -> 0 (crates/mimo26-coordinator/src/wire.rs:53-78,
//     crates/mimo26-load/src/e4m3.rs:50-81).
//   * quant_v1     - "e4m3fn-k32-v1", used for the FC1 -> FC2 intermediate:
//     amax floored at FP32(1e-4), smallest k with amax <= 448 * 2^k, payload
//     rounded to nearest even on the exact grid, scale bytes 105..247, faults
//     instead of clipping (crates/mimo26-expert/kernels/b1/quant_v1.cuh:32-100,
//     oracle/lattice/quant_v1.py:74-87).
// Both reduce to: split the FP32 magnitude into a 24-bit significand and an
// exponent relative to the block scale, then round the significand onto the
// E4M3 grid (4 significant bits above 2^-6, a fixed 2^-9 quantum below).
#pragma once
#include <cstdint>

namespace m26b {

constexpr uint32_t kQuantFloorBits = 0x38d1b717u;  // FP32(1e-4)

// Smallest k with |amax| <= 448 * 2^k for a normal FP32 magnitude given as bits.
// 448 = 1.75 * 2^8, so k = e - 8 when the significand is <= 1.75, else e - 7.
__device__ __forceinline__ int scale_exp_normal(uint32_t amax_bits) {
    const int e = int(amax_bits >> 23) - 127;
    return e - ((amax_bits & 0x7fffffu) <= 0x600000u ? 8 : 7);
}

// Significand (bit 23 set) and unbiased exponent of a finite nonzero magnitude.
__device__ __forceinline__ void split_f32(uint32_t mag, uint32_t& sig, int& exp) {
    const uint32_t field = mag >> 23;
    sig = mag & 0x7fffffu;
    if (field) {
        sig |= 0x800000u;
        exp = int(field) - 127;
    } else {
        const int sh = __clz(sig) - 8;  // FP32 subnormal: normalise
        sig <<= sh;
        exp = -126 - sh;
    }
}

// v >> s rounded to nearest, ties to even (EVEN) or ties up (!EVEN); 1 <= s <= 31, v < 2^24.
template <bool EVEN>
__device__ __forceinline__ uint32_t round_shift(uint32_t v, int s) {
    const uint32_t half = 1u << (s - 1);
    return EVEN ? (v + half - 1u + ((v >> s) & 1u)) >> s : (v + half) >> s;
}

// Magnitude code (7 bits) of sig * 2^(exp - 23) on the E4M3 grid.
template <bool EVEN>
__device__ __forceinline__ uint32_t e4m3_mag_code(uint32_t sig, int exp) {
    if (exp < -6) {  // below the smallest normal: fixed quantum 2^-9, code == multiple
        const int s = 14 - exp;  // >= 21
        return s > 25 ? 0u : round_shift<EVEN>(sig, s);
    }
    uint32_t r = round_shift<EVEN>(sig, 20);  // 8..16
    if (r == 16u) { r = 8u; ++exp; }
    if (exp > 8) return 0x7eu;
    const uint32_t code = uint32_t(exp + 7) * 8u + (r - 8u);
    return code > 0x7eu ? 0x7eu : code;
}

// ---- quant_v1 -----------------------------------------------------------------
__device__ __forceinline__ int quant_v1_scale_exp(uint32_t amax_bits) {
    return scale_exp_normal(amax_bits < kQuantFloorBits ? kQuantFloorBits : amax_bits);
}
// Payload byte for finite input bits under block exponent k (-22 <= k <= 120); -0 keeps its sign.
// h * 2^-k is exact (a power-of-two scaling; an underflow can only happen far below the 2^-10 rounding threshold) and
// lies within +-448 by the choice of k, so the codec's rule - round to nearest even on the E4M3 grid, quantum 2^-9
// below 2^-6, sign kept on a zero result, clamp at 448 - is exactly what the hardware conversion
// cvt.rn.satfinite.e4m3x2.f32 does. One instruction instead of eighteen; the intermediate bytes are compared bit for
// bit with the oracle's codec in the tests.
__device__ __forceinline__ uint32_t quant_v1_payload(uint32_t bits, int k) {
    const float a = __fmul_rn(__uint_as_float(bits), __uint_as_float(uint32_t(127 - k) << 23));
    uint16_t pair;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(a));
    return uint32_t(pair) & 0xffu;
}
// Whether payload * 2^k is representable in FP32.
__device__ __forceinline__ bool quant_v1_finite(uint32_t payload, int k) {
    const uint32_t field = (payload >> 3) & 15u;
    return field == 0u || int(field) - 7 + k <= 127;
}

// ---- wire codec -----------------------------------------------------------------
// Scale byte from the block's magnitude maximum (bits of a finite or infinite FP32).
__device__ __forceinline__ uint32_t wire_scale_byte(uint32_t amax_bits) {
    if (!amax_bits) return 0u;
    if (amax_bits >= 0x7f800000u) return 254u;
    uint32_t sig; int exp;
    split_f32(amax_bits, sig, exp);
    const int k = exp - ((sig & 0x7fffffu) <= 0x600000u ? 8 : 7);
    const int s = k + 127;
    return uint32_t(s < 0 ? 0 : s > 254 ? 254 : s);
}
// Integer form, valid for every scale byte.
__device__ __forceinline__ uint32_t wire_payload_exact(uint32_t bits, uint32_t scale_byte) {
    const uint32_t mag = bits & 0x7fffffffu;
    if (!mag || mag > 0x7f800000u) return 0u;          // +-0 and NaN encode to code 0, sign clear
    const uint32_t sign = (bits >> 24) & 0x80u;
    if (mag == 0x7f800000u) return sign | 0x7eu;       // infinity clamps to 448
    uint32_t sig; int exp;
    split_f32(mag, sig, exp);
    return sign | e4m3_mag_code<false>(sig, exp + 127 - int(scale_byte));
}
// The same code through the FP32 pipeline, for scale bytes 1..253 (every block with a finite nonzero maximum):
// |x| * 2^(127 - s) is a power-of-two scaling, exact unless it underflows, which only happens far below the 2^-10
// rounding threshold. At or above 2^-6 the grid keeps four significant bits: adding half of the dropped field to the
// bit pattern and truncating is round-half-away, and the carry walks into the exponent by itself. Below, the grid is the
// fixed quantum 2^-9: floor(512 a + 1/2), with the add rounded toward zero so that a sum just under an integer is not
// rounded up to it.
__device__ __forceinline__ uint32_t wire_payload(uint32_t bits, uint32_t scale_byte) {
    if (scale_byte - 1u > 252u) return wire_payload_exact(bits, scale_byte);
    const uint32_t mag = bits & 0x7fffffffu;
    if (!mag || mag > 0x7f800000u) return 0u;
    const uint32_t sign = (bits >> 24) & 0x80u;
    if (mag == 0x7f800000u) return sign | 0x7eu;
    const float a = __fmul_rn(__uint_as_float(mag), __uint_as_float((254u - scale_byte) << 23));
    const uint32_t sub = __float2uint_rz(__fadd_rz(__fmul_rn(a, 512.0f), 0.5f));      // 0..8; 8 is the smallest normal's code
    const uint32_t ab = __float_as_uint(a);
    uint32_t nrm = ((ab + 0x80000u) >> 20) - 960u;
    nrm = nrm > 0x7eu ? 0x7eu : nrm;
    return sign | (a < 0.015625f ? sub : nrm);
}

// ---- BF16 ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t bf16_rne_bits(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b + 0x7fffu + ((b >> 16) & 1u)) >> 16;
}

}  // namespace m26b
