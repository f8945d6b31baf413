// Activations as int8 digit planes for the integer tensor-core products (mma.sync.m16n8k32.s8):
//   x = scale * (d0 + d1/128 + d2/128^2 + d3/128^3),  scale = max|x| / 127,  every d an int8,
// which holds each fp32 value to 2^-22 of the largest one. int8 weights and 4-bit codes are multiplied
// as they are stored, the four planes are four of the eight B columns, and the integer sums are exact.
#pragma once

namespace b2 {

constexpr int M1_PLANES = 4;

__device__ __forceinline__ void imma16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// an integer of magnitude below 2^22 as fp32, without the conversion unit
__device__ __forceinline__ float small_int_to_float(int t) { return __int_as_float(t + 0x4B400000) - 12582912.0f; }

// four digits of q = v * inv (|q| <= 127): q = d0 + d1/128 + d2/128^2 + d3/128^3 up to 2^-22. q is rounded once to
// a multiple of 2^-21 (one conversion), then split with integer arithmetic into balanced base-128 digits: d1..d3 in
// [-64, 63], d0 = what remains (|d0| <= 127).
__device__ __forceinline__ void to_digits(float v, float inv, int (&d)[M1_PLANES]) {
    int q = __float2int_rn(v * inv * 2097152.0f);
#pragma unroll
    for (int p = M1_PLANES - 1; p > 0; p--) {
        const int r = ((q + 64) & 127) - 64;
        d[p] = r;
        q = (q - r) >> 7;
    }
    d[0] = q;
}
// eight consecutive values -> per plane the 8 digits as two words; `evenodd`: even positions first (the
// order in which the low / high nibbles of a word of eight codes come out), else natural order
__device__ __forceinline__ void digits8(const float (&v)[8], float inv, bool evenodd, uint2 (&w)[M1_PLANES]) {
    int d[8][M1_PLANES];
#pragma unroll
    for (int i = 0; i < 8; i++) to_digits(v[i], inv, d[i]);
#pragma unroll
    for (int p = 0; p < M1_PLANES; p++) {
        const uint32_t b0 = d[0][p] & 255, b1 = d[1][p] & 255, b2 = d[2][p] & 255, b3 = d[3][p] & 255;
        const uint32_t b4 = d[4][p] & 255, b5 = d[5][p] & 255, b6 = d[6][p] & 255, b7 = d[7][p] & 255;
        w[p].x = evenodd ? (b0 | (b2 << 8) | (b4 << 16) | (b6 << 24)) : (b0 | (b1 << 8) | (b2 << 16) | (b3 << 24));
        w[p].y = evenodd ? (b1 | (b3 << 8) | (b5 << 16) | (b7 << 24)) : (b4 | (b5 << 8) | (b6 << 16) | (b7 << 24));
    }
}
// weight of the planes a lane holds after an mma (columns 2 tid and 2 tid + 1 = planes 0,1 | 2,3 | none)
__device__ __forceinline__ void plane_weights(int tid, float scale, float& w0, float& w1) {
    w0 = tid == 0 ? scale : (tid == 1 ? scale * (1.0f / 16384.0f) : 0.f);
    w1 = w0 * (1.0f / 128.0f);
}

}  // namespace b2
