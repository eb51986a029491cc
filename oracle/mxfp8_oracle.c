/*
 * TEST INFRASTRUCTURE ONLY. CPU restatement (plain C) of the reference's MXFP8 1x32 hot path, used by the tests,
 * the smoke check and the bench's cpu_baseline leg as the parity checker. The product library never links,
 * loads or calls this file.
 *
 * Parity pin: every function that produces bytes is compared, in tests/test_oracle.py, with the reference's own
 * header python/fish_scales_ops/include/fso/activation_contract.h compiled on the host (oracle/_ref) and with the
 * golden vectors generated from it (tests/golden). The GEMM / MoE *outputs* have no golden vectors in the
 * reference (its tests are tolerance tests), so their parity is "unpinned": they are gated by tolerance against
 * the fp32 dequantize-then-matmul form built from the functions below.
 *
 * Reference locations each function follows (paths inside the reference project):
 *   orc_e8m0_from_amax      python/fish_scales_ops/include/fso/activation_contract.h:138-151
 *                           (csrc/gemm/ops/quant_kernels.cu:341-366, e8m0_from_amax<true>)
 *   orc_e8m0_from_amax_int  csrc/gemm/include/blockscale_gemm/arch/sm100/mxfp8/dense_epi_math.cuh:21-28,203-214
 *   orc_e4m3_from_float     activation_contract.h:117-122 (cvt.rn.satfinite.e4m3x2.f32)
 *   orc_sf_word_index       activation_contract.h:166-171, csrc/gemm/ops/quant_kernels.cu:420-442
 *   orc_quantize_1x32       csrc/gemm/ops/quant_kernels.cu:655-688 (wide kernel), launcher :736-820
 *   orc_requant_bs128       python/fish_scales_ops/dense/__init__.py:422-462
 *   orc_pack_ue8m0          python/fish_scales_ops/gemm/mxfp8.py:636-648, 718-768
 *   orc_route               csrc/gemm/ops/moe_glue.cu:2651-2823 (contract: tests/gemm/unit/test_moe_routing_compact.py:98-195)
 *   orc_gather_quant        csrc/gemm/ops/quant_kernels.cu:1572-2111
 *   orc_swiglu_quant        csrc/gemm/include/blockscale_gemm/arch/sm100/mxfp8/fused_swiglu_store.cuh:266-346
 *                           (exact silu here; the reference kernel uses tanh.approx, so this one is a tolerance oracle)
 *   orc_combine             csrc/gemm/ops/moe_glue.cu:304-398, 425-639
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline float bf16_to_float(uint16_t b) { return u2f((uint32_t)b << 16); }

/* fp32 -> bf16, round to nearest even (finite inputs). */
uint16_t orc_bf16_from_float(float f)
{
    uint32_t u = f2u(f);
    if ((u & 0x7F800000u) == 0x7F800000u) return (uint16_t)((u >> 16) | ((u & 0xFFFFu) ? 0x40u : 0u));
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

/* e4m3fn byte -> fp32 (0x7F / 0xFF are NaN). */
float orc_e4m3_to_float(uint8_t b)
{
    uint32_t sign = (uint32_t)(b >> 7);
    uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
    float v;
    if (e == 0xFu && m == 7u) return u2f(0x7FC00000u);
    if (e == 0) v = ldexpf((float)m, -9);            /* subnormal: m * 2^-9 */
    else v = ldexpf(1.f + (float)m / 8.f, (int)e - 7);
    return sign ? -v : v;
}

/* fp32 -> e4m3fn, round to nearest even, saturate finite (|v| > 448 -> 448); NaN -> 0x7F. */
uint8_t orc_e4m3_from_float(float v)
{
    uint32_t u = f2u(v);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return 0x7Fu;                /* NaN */
    float av = u2f(a);
    if (av >= 448.f) return (uint8_t)(sign | 0x7Eu);  /* satfinite (inf too) */
    /* the spacing of e4m3 at this magnitude: 2^(max(e,-6) - 3) */
    int e;
    (void)frexpf(av, &e);                             /* av = f * 2^e, f in [0.5,1) -> exponent e-1 */
    int ex = e - 1;
    if (av == 0.f) return sign;
    if (ex < -6) ex = -6;
    float step = ldexpf(1.f, ex - 3);
    float qf = av / step;                             /* exact: power-of-two division */
    float r = nearbyintf(qf);                         /* default rounding mode: to nearest even */
    float rv = r * step;
    if (rv > 448.f) rv = 448.f;
    /* encode rv */
    if (rv == 0.f) return sign;
    int e2;
    float f2 = frexpf(rv, &e2);                       /* rv = f2 * 2^e2 */
    int ee = e2 - 1;
    if (ee < -6) {                                    /* subnormal */
        uint32_t m = (uint32_t)(rv / ldexpf(1.f, -9));
        return (uint8_t)(sign | m);
    }
    uint32_t m = (uint32_t)((f2 * 2.f - 1.f) * 8.f);
    return (uint8_t)(sign | ((uint32_t)(ee + 7) << 3) | m);
}

/* The divide form of the scale byte. amax is already floored at 1e-10f. */
uint8_t orc_e8m0_from_amax(float amax, float* quant_scale)
{
    volatile float q_raw = 448.f / amax;
    volatile float d_raw = 1.f / q_raw;
    uint32_t bits = f2u(d_raw);
    uint32_t byte = ((bits >> 23) & 0xFFu) + ((bits & 0x7FFFFFu) != 0u ? 1u : 0u);
    if (byte > 254u) byte = 254u;
    float dq = u2f(byte << 23);
    *quant_scale = byte != 0u ? 1.f / dq : 1.f;
    return (uint8_t)byte;
}

/* The division-free form the CUDA quantizers use; equal to the divide form for every amax a bf16 block can have
 * (checked exhaustively in tests/test_oracle.py). quant scale = 2^(127 - byte). */
uint8_t orc_e8m0_from_amax_int(float amax, float* quant_scale)
{
    uint32_t bits = f2u(amax);
    int e = (int)((bits >> 23) & 0xFFu);
    uint32_t f = bits & 0x7FFFFFu;
    int byte = e - (f <= 0x600000u ? 8 : 7);
    if (byte < 0) byte = 0;
    if (byte > 254) byte = 254;
    if (e == 255) byte = 254;      /* amax = Inf: the divide form gives 448 / Inf = 0, 1 / 0 = Inf, field 255, capped */
    *quant_scale = byte == 254 ? u2f(0x00400000u) : u2f((uint32_t)(254 - byte) << 23);
    if (byte == 0) *quant_scale = 1.f;
    return (uint8_t)byte;
}

int64_t orc_sf_word_index(int64_t m, int64_t kp, int64_t k)
{
    int64_t nkp = k / 128, r = m % 128;
    return ((m / 128) * nkp + kp) * 128 + (r % 32) * 4 + r / 32;
}

int64_t orc_sf_words(int64_t m, int64_t k) { return (m + 127) / 128 * 128 * (k / 128); }

/* One 32-element block of fp32 values -> 32 codes + the scale byte. */
static uint8_t quant_block(const float* v, uint8_t* q)
{
    float amax = 0.f;
    for (int i = 0; i < 32; ++i) { float a = fabsf(v[i]); if (a > amax) amax = a; }
    if (amax < 1e-10f) amax = 1e-10f;
    float qs;
    uint8_t b = orc_e8m0_from_amax(amax, &qs);
    for (int i = 0; i < 32; ++i) { volatile float p = v[i] * qs; q[i] = orc_e4m3_from_float(p); }
    return b;
}

/* fp32 rows (already the exact values of the bf16 input) -> codes + atom-layout words; dst_row lets the caller
 * place row r of the input at another row of the output (gather / interleave); NULL = identity. */
static void quant_rows_f32(const float* x, int64_t rows_in, int64_t k, const int64_t* dst_row, uint8_t* q,
    uint32_t* sf)
{
    for (int64_t r = 0; r < rows_in; ++r) {
        int64_t d = dst_row ? dst_row[r] : r;
        if (d < 0) continue;
        for (int64_t kp = 0; kp < k / 128; ++kp) {
            uint32_t w = 0;
            for (int b = 0; b < 4; ++b) {
                uint8_t byte = quant_block(x + r * k + kp * 128 + b * 32, q + d * k + kp * 128 + b * 32);
                w |= (uint32_t)byte << (8 * b);
            }
            sf[orc_sf_word_index(d, kp, k)] = w;
        }
    }
}

/* bf16 [M, K] -> e4m3 [M, K] + int32 words [align(M,128) * K/128] (padded rows zero).
 * interleave_i > 0: the input is G stacked [2*I, K] experts in [gate; up] order and output row 2j / 2j+1 of an
 * expert takes its input row j / I + j (mxfp8.py:621-633). */
void orc_quantize_1x32(const uint16_t* x, int64_t m, int64_t k, int64_t interleave_i, uint8_t* q, uint32_t* sf)
{
    memset(sf, 0, (size_t)orc_sf_words(m, k) * 4);
    float* row = (float*)malloc((size_t)k * 4);
    for (int64_t r = 0; r < m; ++r) {
        int64_t src = r;
        if (interleave_i > 0) {
            int64_t two_i = 2 * interleave_i, g = r / two_i, o = r % two_i;
            src = g * two_i + ((o & 1) ? interleave_i + o / 2 : o / 2);
        }
        for (int64_t c = 0; c < k; ++c) row[c] = bf16_to_float(x[src * k + c]);
        int64_t d = r;
        /* quant_rows_f32 indexes the input by row 0 here */
        for (int64_t kp = 0; kp < k / 128; ++kp) {
            uint32_t w = 0;
            for (int b = 0; b < 4; ++b)
                w |= (uint32_t)quant_block(row + kp * 128 + b * 32, q + d * k + kp * 128 + b * 32) << (8 * b);
            sf[orc_sf_word_index(d, kp, k)] = w;
        }
    }
    free(row);
}

/* Block-FP8 checkpoint (e4m3 [N, K] + fp32 [N/128, K/128]) -> MXFP8: bf16_rne(float(fp8) * s) then the 1x32 rule.
 * interleave_i as in orc_quantize_1x32 (python/fish_scales_ops/moe/__init__.py:400-407 + mxfp8.py:621-633). */
void orc_requant_bs128(const uint8_t* wq, const float* scale, int64_t n, int64_t k, int64_t interleave_i, uint8_t* q,
    uint32_t* sf)
{
    memset(sf, 0, (size_t)orc_sf_words(n, k) * 4);
    float* row = (float*)malloc((size_t)k * 4);
    for (int64_t r = 0; r < n; ++r) {
        int64_t src = r;
        if (interleave_i > 0) {
            int64_t two_i = 2 * interleave_i, g = r / two_i, o = r % two_i;
            src = g * two_i + ((o & 1) ? interleave_i + o / 2 : o / 2);
        }
        for (int64_t c = 0; c < k; ++c) {
            volatile float p = orc_e4m3_to_float(wq[src * k + c]) * scale[(src / 128) * (k / 128) + c / 128];
            row[c] = bf16_to_float(orc_bf16_from_float(p));
        }
        for (int64_t kp = 0; kp < k / 128; ++kp) {
            uint32_t w = 0;
            for (int b = 0; b < 4; ++b)
                w |= (uint32_t)quant_block(row + kp * 128 + b * 32, q + r * k + kp * 128 + b * 32) << (8 * b);
            sf[orc_sf_word_index(r, kp, k)] = w;
        }
    }
    free(row);
}

/* Checkpoint UE8M0 bytes uint8 [G, N, K/32] -> int32 atom slabs [G, align(N,128) * K/128]; interleave_i as above. */
void orc_pack_ue8m0(const uint8_t* s, int64_t g, int64_t n, int64_t k, int64_t interleave_i, uint32_t* out)
{
    int64_t kb = k / 128, slab = (n + 127) / 128 * 128 * kb;
    memset(out, 0, (size_t)(g * slab) * 4);
    for (int64_t e = 0; e < g; ++e)
        for (int64_t r = 0; r < n; ++r) {
            int64_t src = r;
            if (interleave_i > 0) src = (r & 1) ? interleave_i + r / 2 : r / 2;
            for (int64_t kp = 0; kp < kb; ++kp) {
                const uint8_t* b = s + ((e * n + src) * (k / 32)) + kp * 4;
                out[e * slab + orc_sf_word_index(r, kp, k)] =
                    (uint32_t)b[0] | (uint32_t)b[1] << 8 | (uint32_t)b[2] << 16 | (uint32_t)b[3] << 24;
            }
        }
}

/* e4m3 [M, K] + atom words -> fp32 [M, K]: code * 2^(byte - 127). */
void orc_dequant(const uint8_t* q, const uint32_t* sf, int64_t m, int64_t k, float* out)
{
    for (int64_t r = 0; r < m; ++r)
        for (int64_t kp = 0; kp < k / 128; ++kp) {
            uint32_t w = sf[orc_sf_word_index(r, kp, k)];
            for (int b = 0; b < 4; ++b) {
                int byte = (int)((w >> (8 * b)) & 0xFFu);
                float s = ldexpf(1.f, byte - 127);
                for (int i = 0; i < 32; ++i) {
                    int64_t c = kp * 128 + b * 32 + i;
                    out[r * k + c] = orc_e4m3_to_float(q[r * k + c]) * s;
                }
            }
        }
}

/* Compact routing, canonical order: the pairs of an expert keep ascending flat index.
 * masked_m[E], blk0[E+1], slot_of_flat[P], blk_expert[num_blocks] (-1 past the used blocks). */
void orc_route(const int32_t* ids, int64_t pairs, int64_t num_experts, int64_t num_blocks, int32_t* masked_m,
    int32_t* blk0, int32_t* slot_of_flat, int32_t* blk_expert)
{
    memset(masked_m, 0, (size_t)num_experts * 4);
    for (int64_t i = 0; i < pairs; ++i)
        if (ids[i] >= 0 && ids[i] < num_experts) masked_m[ids[i]]++;
    int32_t acc = 0;
    for (int64_t e = 0; e < num_experts; ++e) { blk0[e] = acc; acc += (masked_m[e] + 127) / 128; }
    blk0[num_experts] = acc;
    if (blk_expert) {
        for (int64_t b = 0; b < num_blocks; ++b) blk_expert[b] = -1;
        for (int64_t e = 0; e < num_experts; ++e)
            for (int32_t b = blk0[e]; b < blk0[e + 1] && b < num_blocks; ++b) blk_expert[b] = (int32_t)e;
    }
    int32_t* fill = (int32_t*)calloc((size_t)num_experts, 4);
    for (int64_t i = 0; i < pairs; ++i) {
        int32_t e = ids[i];
        if (e < 0 || e >= num_experts) { slot_of_flat[i] = -1; continue; }
        slot_of_flat[i] = blk0[e] * 128 + fill[e]++;
    }
    free(fill);
}

/* Row gather + 1x32 quantize into the compact buffer: pair i = (token i / topk) goes to row slot_of_flat[i].
 * Rows no pair maps to are left untouched. */
void orc_gather_quant(const uint16_t* hidden, int64_t tokens, int64_t topk, int64_t h, const int32_t* slot_of_flat,
    uint8_t* hq, uint32_t* sh)
{
    float* row = (float*)malloc((size_t)h * 4);
    for (int64_t i = 0; i < tokens * topk; ++i) {
        int64_t d = slot_of_flat[i];
        if (d < 0) continue;
        int64_t t = i / topk;
        for (int64_t c = 0; c < h; ++c) row[c] = bf16_to_float(hidden[t * h + c]);
        quant_rows_f32(row, 1, h, &d, hq, sh);
    }
    free(row);
}

/* FC1 epilogue oracle: acc fp32 [rows, 2*I] with interleaved (gate, up) columns -> silu(gate) * up in fp32
 * (exact silu) -> 1x32 rule -> e4m3 [rows, I] + atom words. Only rows with live[r] != 0 are written. */
void orc_swiglu_quant(const float* acc, int64_t rows, int64_t inter, const uint8_t* live, uint8_t* dq, uint32_t* sd)
{
    float* row = (float*)malloc((size_t)inter * 4);
    for (int64_t r = 0; r < rows; ++r) {
        if (live && !live[r]) continue;
        for (int64_t j = 0; j < inter; ++j) {
            float g = acc[r * 2 * inter + 2 * j], u = acc[r * 2 * inter + 2 * j + 1];
            row[j] = (g / (1.f + expf(-g))) * u;
        }
        int64_t d = r;
        quant_rows_f32(row, 1, inter, &d, dq, sd);
    }
    free(row);
}

/* out[t] = bf16_rn( sum_{j ascending} w[t,j] * float(dn[slot_j]) + bias_scale[t] * bias[t] ), fp32 FMA chain,
 * skipped slots contribute nothing. bias / bias_scale may be NULL (bias_scale NULL with bias = factor 1). */
void orc_combine(const uint16_t* dn, const int32_t* slot_of_flat, const float* w, const uint16_t* bias,
    const float* bias_scale, int64_t tokens, int64_t topk, int64_t h, uint16_t* out)
{
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t c = 0; c < h; ++c) {
            float acc = 0.f;
            for (int64_t j = 0; j < topk; ++j) {
                int32_t s = slot_of_flat[t * topk + j];
                if (s < 0) continue;
                acc = fmaf(w[t * topk + j], bf16_to_float(dn[(int64_t)s * h + c]), acc);
            }
            if (bias) acc = fmaf(bias_scale ? bias_scale[t] : 1.f, bf16_to_float(bias[t * h + c]), acc);
            out[t * h + c] = orc_bf16_from_float(acc);
        }
}
