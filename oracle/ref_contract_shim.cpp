// TEST INFRASTRUCTURE ONLY (parity checker; never linked into or called by the product library).
//
// A thin C-ABI shim over the reference's own quantizer statement,
// python/fish_scales_ops/include/fso/activation_contract.h (host path), compiled from where that header lies
// (the build recipe passes its directory with -I; nothing of the reference is copied here).
// It drives the header's functions over a whole [M, K] bf16 activation the way the header's own comment
// prescribes (activation_contract.h:14-28): per 32-element block amax floored at fso_mx_amax_floor(), byte and
// quant scale from fso_e8m0_from_amax, codes from fso_mx_quantize4, words packed by fso_mx_pack_word and placed
// at fso_mx_sf_word_index_sm100; the padded rows' words are zero.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "fso/activation_contract.h"

static inline float bf16_to_float(uint16_t b)
{
    uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    std::memcpy(&f, &u, sizeof(f));
    return f;
}

extern "C" {

int ref_contract_version() { return kFsoActivationContractVersion; }

// x: bf16 bits [M, K]; q: e4m3 bytes [M, K]; sf: int32 words, fso_mx_sf_words_sm100(M, K) of them.
void ref_quantize_1x32_sm100(const uint16_t* x, int64_t m, int64_t k, uint8_t* q, uint32_t* sf)
{
    int64_t const words = fso_mx_sf_words_sm100(m, k);
    std::memset(sf, 0, static_cast<size_t>(words) * 4);
    for (int64_t r = 0; r < m; ++r) {
        for (int64_t kp = 0; kp < k / 128; ++kp) {
            uint8_t bytes[4];
            for (int b = 0; b < 4; ++b) {
                const uint16_t* src = x + r * k + kp * 128 + b * 32;
                float amax = 0.f;
                for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(bf16_to_float(src[i])));
                amax = std::fmax(amax, fso_mx_amax_floor());
                float qs;
                bytes[b] = fso_e8m0_from_amax(amax, &qs);
                uint32_t* dst = reinterpret_cast<uint32_t*>(q + r * k + kp * 128 + b * 32);
                for (int i = 0; i < 32; i += 4) {
                    uint32_t w = fso_mx_quantize4(bf16_to_float(src[i]), bf16_to_float(src[i + 1]),
                        bf16_to_float(src[i + 2]), bf16_to_float(src[i + 3]), qs);
                    std::memcpy(dst + i / 4, &w, 4);
                }
            }
            sf[fso_mx_sf_word_index_sm100(r, kp, k)] = fso_mx_pack_word(bytes[0], bytes[1], bytes[2], bytes[3]);
        }
    }
}

// The byte and quant-scale bits the header gives for one (already floored) amax.
uint32_t ref_e8m0_from_amax(float amax, uint32_t* quant_scale_bits)
{
    float qs;
    uint8_t const b = fso_e8m0_from_amax(amax, &qs);
    std::memcpy(quant_scale_bits, &qs, 4);
    return b;
}

// One e4m3 code of the header's conversion (cvt.rn.satfinite semantics of the CUDA host path).
uint32_t ref_e4m3_from_float(float v) { return fso_fp8x4_from_floats(v, 0.f, 0.f, 0.f) & 0xFFu; }

int64_t ref_sf_word_index_sm100(int64_t m, int64_t kp, int64_t k) { return fso_mx_sf_word_index_sm100(m, kp, k); }
int64_t ref_sf_words_sm100(int64_t m, int64_t k) { return fso_mx_sf_words_sm100(m, k); }

}  // extern "C"
