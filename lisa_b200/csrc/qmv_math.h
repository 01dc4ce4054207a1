// Register-level decode of packed affine codes for the CUDA-core GEMV.
//
// A b-bit code q sitting at bit position P (P+b <= 23) of a 32-bit word becomes
// the f32 value t = 1 + q * 2^(P-23) by masking it in place and OR-ing the
// exponent of 1.0f: no shift to bit 0, no int->float conversion.  With the
// activation pre-scaled to xs = x * 2^(23-P),
//     t * xs = xs + q * x,
// so a dot product accumulates sum(t*xs) and subtracts the per-chunk constant
// sum(xs) once.  Codes whose position is outside the usable window are brought
// into it with one shift/rotate of the whole word that serves several codes.
// Position windows are chosen so that xs is at most x * 2^11 (4-bit) or
// x * 2^13 (2-bit): the cancellation costs at most 8 (4-bit) / 12 (2-bit) of
// the 24 significand bits of an accumulator that only spans 16 or 32 codes.
//
// The functions are __host__ __device__ so that the same bit manipulation is
// exercised by a CPU unit test.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define LISA_HD __host__ __device__ __forceinline__
#else
#define LISA_HD inline
#endif

namespace lisa {

template <int BITS>
struct QmvCode;

// ---- 4-bit: 8 codes per word, 4 (lo,hi) pairs, positions P=12 (lo) and P=16 (hi).
template <>
struct QmvCode<4> {
    static constexpr int kCodesPerWord = 8;
    static constexpr int kPairsPerWord = 4;
    // code index within the word that pair p, element e decodes
    LISA_HD static int code_of(int p, int e) {
        // p0: w        -> j=3 @12, j=4 @16
        // p1: w << 8   -> j=1 @12, j=2 @16
        // p2: w >> 8   -> j=5 @12, j=6 @16
        // p3: rot16(w) -> j=7 @12, j=0 @16
        const int tab[4][2] = {{3, 4}, {1, 2}, {5, 6}, {7, 0}};
        return tab[p][e];
    }
    // power of two the activation paired with (p, e) is multiplied by
    LISA_HD static float xscale_of(int /*p*/, int e) { return e == 0 ? 2048.0f : 128.0f; }
    // t bit patterns for the 4 pairs of one word
    LISA_HD static void decode(uint32_t w, uint32_t (&lo)[4], uint32_t (&hi)[4]) {
        const uint32_t one = 0x3f800000u, mlo = 0x0000f000u, mhi = 0x000f0000u;
        const uint32_t s1 = w << 8, s2 = w >> 8, s3 = (w << 16) | (w >> 16);
        lo[0] = (w & mlo) | one;
        hi[0] = (w & mhi) | one;
        lo[1] = (s1 & mlo) | one;
        hi[1] = (s1 & mhi) | one;
        lo[2] = (s2 & mlo) | one;
        hi[2] = (s2 & mhi) | one;
        lo[3] = (s3 & mlo) | one;
        hi[3] = (s3 & mhi) | one;
    }
};

// ---- 2-bit: 16 codes per word, 8 pairs, positions P in {10,12,...,20}.
template <>
struct QmvCode<2> {
    static constexpr int kCodesPerWord = 16;
    static constexpr int kPairsPerWord = 8;
    LISA_HD static int code_of(int p, int e) {
        // s0 = w       : codes 5..10 at P = 10..20
        // s1 = w << 10 : codes 0..4  at P = 10..18
        // s2 = w >> 12 : codes 11..15 at P = 10..18
        const int tab[8][2] = {{5, 6}, {7, 8}, {9, 10}, {0, 1}, {2, 3}, {11, 12}, {13, 14}, {4, 15}};
        return tab[p][e];
    }
    LISA_HD static int pos_of(int p, int e) {
        const int tab[8][2] = {{10, 12}, {14, 16}, {18, 20}, {10, 12},
                               {14, 16}, {10, 12}, {14, 16}, {18, 18}};
        return tab[p][e];
    }
    LISA_HD static float xscale_of(int p, int e) {
        return static_cast<float>(1u << (23 - pos_of(p, e)));
    }
    LISA_HD static void decode(uint32_t w, uint32_t (&lo)[8], uint32_t (&hi)[8]) {
        const uint32_t one = 0x3f800000u;
        const uint32_t s1 = w << 10, s2 = w >> 12;
        lo[0] = (w & (3u << 10)) | one;
        hi[0] = (w & (3u << 12)) | one;
        lo[1] = (w & (3u << 14)) | one;
        hi[1] = (w & (3u << 16)) | one;
        lo[2] = (w & (3u << 18)) | one;
        hi[2] = (w & (3u << 20)) | one;
        lo[3] = (s1 & (3u << 10)) | one;
        hi[3] = (s1 & (3u << 12)) | one;
        lo[4] = (s1 & (3u << 14)) | one;
        hi[4] = (s1 & (3u << 16)) | one;
        lo[5] = (s2 & (3u << 10)) | one;
        hi[5] = (s2 & (3u << 12)) | one;
        lo[6] = (s2 & (3u << 14)) | one;
        hi[6] = (s2 & (3u << 16)) | one;
        lo[7] = (s1 & (3u << 18)) | one;
        hi[7] = (s2 & (3u << 18)) | one;
    }
};

}  // namespace lisa
