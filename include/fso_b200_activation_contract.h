/* The activation contract of fish_scales_ops_b200 (sm_100 family), version 1, as compilable code.
 *
 * What fso.dense.quantize_activation returns and fso.dense.linear(xq, weight, x_scale=...) accepts: for a bf16
 * activation [M, K] (K % 128 == 0), E4M3 codes [M, K] row-major and one 32-bit scale word per (row, 128-wide K
 * chunk), each word holding the four UE8M0 bytes of the chunk's four 1 x 32 blocks. A producer that wants to hand
 * this library a pre-quantized activation (a fused attention or normalisation epilogue, say) includes this header,
 * on the host or in a CUDA kernel, and follows it; it then writes the bytes the library's own quantizer writes.
 *
 * It restates, for this device family, what python/fish_scales_ops/include/fso/activation_contract.h:138-172 of the
 * reference states (scale byte from the block amax, quant scale, word packing, the sm_100 index formula). The scale
 * byte is given in the division-free integer form (the reference's own equivalent form,
 * csrc/gemm/include/blockscale_gemm/arch/sm100/mxfp8/dense_epi_math.cuh:21-28), which equals
 * q = 448.f / amax; d = 1.f / q; byte = exponent_field(d) + (mantissa(d) != 0), capped at 254, for every amax.
 *
 * C99 / C++ / CUDA. Nothing here allocates or launches.
 */
#ifndef FSO_B200_ACTIVATION_CONTRACT_H
#define FSO_B200_ACTIVATION_CONTRACT_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#include <cuda_fp8.h>
#define FSO_B200_HD __host__ __device__ static inline
#else
#define FSO_B200_HD static inline
#endif

#define FSO_B200_ACTIVATION_CONTRACT_VERSION 1
#define FSO_B200_BLOCK 32           /* elements that share one scale byte */
#define FSO_B200_CHUNK 128          /* elements that share one scale word */

FSO_B200_HD uint32_t fso_b200_bits_of(float v)
{
    uint32_t u;
    memcpy(&u, &v, sizeof(u));
    return u;
}

FSO_B200_HD float fso_b200_float_of(uint32_t u)
{
    float v;
    memcpy(&v, &u, sizeof(v));
    return v;
}

/* A block's amax is max |x| over its 32 elements in fp32, NaN elements left out (a NaN never becomes the amax),
 * then raised to this floor. */
FSO_B200_HD float fso_b200_amax_floor(void) { return 1e-10f; }

/* fmaxf semantics spelled out: a NaN operand is passed over. */
FSO_B200_HD float fso_b200_amax_step(float running, float x)
{
    float const a = x < 0.f ? -x : x;
    return a > running ? a : running;        /* false for a NaN a: the running value stays */
}

/* UE8M0 scale byte of a block from its (floored) amax, and the factor 2^(127 - byte) its elements are multiplied by
 * before conversion. With E and f the exponent and mantissa fields of amax: byte = E - (f <= 0x600000 ? 8 : 7),
 * kept inside [0, 254]; an infinite amax gives 254. */
FSO_B200_HD uint8_t fso_b200_scale_byte(float amax, float* quant_scale)
{
    uint32_t const bits = fso_b200_bits_of(amax);
    int const e = (int)((bits >> 23) & 0xFFu);
    uint32_t const f = bits & 0x7FFFFFu;
    int byte = e - (f <= 0x600000u ? 8 : 7);
    if (byte < 0) byte = 0;
    if (byte > 254 || e == 255) byte = 254;
    if (quant_scale) {
        uint32_t q = (uint32_t)(254 - byte) << 23;          /* 2^(127 - byte) */
        if (byte == 254) q = 0x00400000u;                    /* 2^-127 is a subnormal */
        if (byte == 0) q = 0x3F800000u;
        *quant_scale = fso_b200_float_of(q);
    }
    return (uint8_t)byte;
}

/* One E4M3 code of v (already multiplied by the quant scale): round to nearest even, saturate to +-448, any NaN ->
 * 0x7F (what cvt.rn.satfinite.e4m3x2.f32 gives). */
FSO_B200_HD uint8_t fso_b200_e4m3(float v)
{
#if defined(__CUDA_ARCH__)
    return (uint8_t)(__nv_cvt_float2_to_fp8x2(make_float2(v, 0.f), __NV_SATFINITE, __NV_E4M3) & 0xFFu);
#else
    uint32_t const bits = fso_b200_bits_of(v);
    uint8_t const sign = (uint8_t)((bits >> 24) & 0x80u);
    uint32_t const mag = bits & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return 0x7Fu;                              /* NaN, whatever its sign */
    if (mag >= 0x43E00000u) return (uint8_t)(sign | 0x7Eu);           /* |v| >= 448 (Inf included): saturate */
    int const e = (int)(mag >> 23) - 127;
    if (e < -10) return sign;                                         /* below half of the smallest subnormal */
    /* |v| = m * 2^(e - 23), m with the implicit bit. One unit of the code is 2^-9 below 2^-6 (subnormal codes) and
     * 2^(e - 3) from there on, so |v| is m / 2^d units with d = 14 - e or 20; round half to even. */
    uint32_t const m = (mag & 0x7FFFFFu) | 0x800000u;
    int const d = e < -6 ? 14 - e : 20;
    uint32_t q = m >> d;
    uint32_t const rem = m & ((1u << d) - 1u);
    uint32_t const half = 1u << (d - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    if (e < -6) return (uint8_t)(sign | q);                           /* q in [0, 8]; 8 is the smallest normal code */
    /* q in [8, 16]: 3 mantissa bits under the implicit one; 16 carries into the next exponent by itself */
    uint32_t const code = ((uint32_t)(e + 7) << 3) + (q - 8u);
    return (uint8_t)(sign | (code > 0x7Eu ? 0x7Eu : code));
#endif
}

/* Scale word of one 128-wide chunk: the byte of block i (elements [32 i, 32 i + 32) of the chunk) in bits 8i..8i+7. */
FSO_B200_HD uint32_t fso_b200_pack_word(uint8_t b0, uint8_t b1, uint8_t b2, uint8_t b3)
{
    return (uint32_t)b0 | ((uint32_t)b1 << 8) | ((uint32_t)b2 << 16) | ((uint32_t)b3 << 24);
}

/* Position of the word of (row m, chunk kp) in the 1-D int32 scale tensor of an [M, k] activation: 128-row groups
 * of k / 128 chunks each; inside a (group, chunk) the 128 words are ordered by (m % 32) * 4 + (m % 128) / 32, which
 * is the byte order the tensor cores' scale-factor copy expects. */
FSO_B200_HD int64_t fso_b200_sf_word_index(int64_t m, int64_t kp, int64_t k)
{
    int64_t const chunks = k / FSO_B200_CHUNK;
    int64_t const r = m % 128;
    return ((m / 128) * chunks + kp) * 128 + (r % 32) * 4 + r / 32;
}

/* Words in that tensor: rows are padded to a multiple of 128; the padded rows' words are zero. */
FSO_B200_HD int64_t fso_b200_sf_words(int64_t m, int64_t k)
{
    return (m + 127) / 128 * 128 * (k / FSO_B200_CHUNK);
}

/* One 1 x 32 block: x are the 32 values (the exact fp32 values of the bf16 elements), codes receives 32 bytes;
 * returns the block's scale byte. */
FSO_B200_HD uint8_t fso_b200_quantize_block(const float* x, uint8_t* codes)
{
    float amax = 0.f;
    for (int i = 0; i < FSO_B200_BLOCK; ++i) amax = fso_b200_amax_step(amax, x[i]);
    if (!(amax >= fso_b200_amax_floor())) amax = fso_b200_amax_floor();
    float qs;
    uint8_t const byte = fso_b200_scale_byte(amax, &qs);
    for (int i = 0; i < FSO_B200_BLOCK; ++i) codes[i] = fso_b200_e4m3(x[i] * qs);
    return byte;
}

#endif /* FSO_B200_ACTIVATION_CONTRACT_H */
