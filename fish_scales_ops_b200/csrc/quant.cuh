// HBM-bound quantizers: bf16 -> MXFP8 (1x32 blocks, UE8M0 scales), block-FP8 128x128 -> MXFP8, and the
// checkpoint scale packer. All of them write the scale words straight into the atom layout the GEMM's
// scale-factor copy reads (one contiguous 512-byte block per 128 rows x 128 K).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace fso {

// ---------------------------------------------------------------------------------------------------- the rule

// Scale byte and quant scale of a block from its amax (already floored at 1e-10f). Division-free form of
// b = exp(1 / (448 / amax)) + (mantissa != 0): with E, f the exponent and mantissa fields of amax,
// b = E - (f <= 0x600000 ? 8 : 7), clamped to [0, 254]; quant scale 2^(127 - b). Equal to the two-division form
// for every finite fp32 amax >= 1e-10f (checked exhaustively on the host). An infinite amax (a block that holds an
// Inf) gives 254 like the division form does: 448 / Inf = 0, 1 / 0 = Inf, exponent field 255, capped.
__device__ __forceinline__ uint32_t e8m0_from_amax(float amax, float& quant_scale)
{
    uint32_t const bits = __float_as_uint(amax);
    int const e = static_cast<int>((bits >> 23) & 0xFFu);
    uint32_t const f = bits & 0x7FFFFFu;
    int byte = e - (f <= 0x600000u ? 8 : 7);
    byte = max(0, min(254, byte));
    if (e == 255) byte = 254;
    uint32_t qbits = static_cast<uint32_t>(254 - byte) << 23;
    if (byte == 254) qbits = 0x00400000u;    // 2^-127, a subnormal
    if (byte == 0) qbits = 0x3F800000u;
    quant_scale = __uint_as_float(qbits);
    return static_cast<uint32_t>(byte);
}

__device__ __forceinline__ uint32_t fp8x4(float v0, float v1, float v2, float v3)
{
    uint32_t const lo = __nv_cvt_float2_to_fp8x2(make_float2(v0, v1), __NV_SATFINITE, __NV_E4M3);
    uint32_t const hi = __nv_cvt_float2_to_fp8x2(make_float2(v2, v3), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 const v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ int64_t sf_word_index(int64_t m, int64_t kp, int64_t kb)
{
    int64_t const r = m & 127;
    return ((m >> 7) * kb + kp) * 128 + (r & 31) * 4 + (r >> 5);
}

// max |.| of the two bf16 halves of each word, as 15-bit patterns (monotonic in magnitude for non-NaN values)
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t a, uint32_t b)
{
    return __vmaxu2(a & 0x7FFF7FFFu, b & 0x7FFF7FFFu);
}

// |.| patterns of the two halves with NaN halves replaced by zero. The block amax is a chain of fmaxf in the
// reference (csrc/gemm/ops/quant_kernels.cu:625-633), which passes over NaNs: a NaN never becomes the amax. On bit
// patterns a NaN (> 0x7F80) would win the integer max, so a block whose pattern max says "NaN present" is reduced
// again through this form (rare path).
__device__ __forceinline__ uint32_t abs_bf16x2_drop_nan(uint32_t a)
{
    uint32_t const m = a & 0x7FFF7FFFu;
    return m & ~__vcmpgtu2(m, 0x7F807F80u);
}

// max over the halves of n words
template <int N>
__device__ __forceinline__ uint32_t absmax_words(uint32_t const (&w)[N], bool drop_nan)
{
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) m = __vmaxu2(m, drop_nan ? abs_bf16x2_drop_nan(w[i]) : (w[i] & 0x7FFF7FFFu));
    return max(m & 0xFFFFu, m >> 16);
}

// Quantizes the 8 bf16 values of `v` (one 16-byte load) of a 32-element block shared by 4 adjacent lanes.
// Returns the 8 codes in `out` and the block's byte (same value on the 4 lanes).
__device__ __forceinline__ uint32_t quant8_shared4(uint4 const& v, uint2& out)
{
    uint32_t const w4[4] = {v.x, v.y, v.z, v.w};
    uint32_t m = absmax_words(w4, false);
    m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
    m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
    if (__any_sync(0xFFFFFFFFu, m > 0x7F80u)) {            // a NaN somewhere in the warp's blocks: leave NaNs out
        m = absmax_words(w4, true);
        m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
        m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
    }
    float const amax = fmaxf(__uint_as_float(m << 16), 1e-10f);
    float qs;
    uint32_t const byte = e8m0_from_amax(amax, qs);
    auto lo = [](uint32_t w) { return __uint_as_float(w << 16); };
    auto hi = [](uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); };
    out.x = fp8x4(__fmul_rn(lo(v.x), qs), __fmul_rn(hi(v.x), qs), __fmul_rn(lo(v.y), qs), __fmul_rn(hi(v.y), qs));
    out.y = fp8x4(__fmul_rn(lo(v.z), qs), __fmul_rn(hi(v.z), qs), __fmul_rn(lo(v.w), qs), __fmul_rn(hi(v.w), qs));
    return byte;
}

// The scale word of a 128-element chunk handled by 16 adjacent lanes (4 lanes per block): every lane passes its
// block's byte, every lane gets the word.
__device__ __forceinline__ uint32_t word_from_16lanes(uint32_t byte, int sub16)
{
    uint32_t w = byte << (8 * (sub16 >> 2));
    w |= __shfl_xor_sync(0xFFFFFFFFu, w, 4);
    w |= __shfl_xor_sync(0xFFFFFFFFu, w, 8);
    return w;
}

// ---------------------------------------------------------------------------------------------------- bf16 -> MXFP8

// One 128-element chunk (row, kp) per half-warp and step; every half-warp owns kUnroll consecutive chunks so that
// kUnroll independent 16-byte loads per thread are in flight. Rows in [m, m_pad) only get their zero words.
template <int kUnroll>
__global__ void __launch_bounds__(256) quantize_1x32_kernel(const uint4* __restrict__ x, uint2* __restrict__ q,
    uint32_t* __restrict__ sf, uint32_t m, uint32_t m_pad, uint32_t kb, uint32_t interleave_i, uint32_t early)
{
    // activation form: a GEMM launched behind this kernel may start loading its weights while this one runs, and
    // this kernel itself may have been started under its predecessor, whose output x may be
    if (early) {
        griddep_launch_dependents();
        griddep_wait();
    }
    // 32-bit index arithmetic throughout (the launcher refuses more than 2^31 chunks): one division per thread.
    uint32_t const sub = threadIdx.x & 15;
    uint32_t const half = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    uint32_t const total = m_pad * kb;
    uint32_t const c0 = half * kUnroll;
    uint32_t row0 = c0 / kb;
    uint32_t kp0 = c0 - row0 * kb;

    uint4 v[kUnroll];
    uint32_t row[kUnroll];
    uint32_t kp[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        row[u] = row0;
        kp[u] = kp0;
        if (++kp0 == kb) {
            kp0 = 0;
            ++row0;
        }
        v[u] = make_uint4(0, 0, 0, 0);
        if (c0 + u < total && row[u] < m) {
            uint32_t src = row[u];
            if (interleave_i > 0) {
                uint32_t const two_i = 2 * interleave_i;
                uint32_t const g = src / two_i, o = src - g * two_i;
                src = g * two_i + ((o & 1) ? interleave_i + (o >> 1) : (o >> 1));
            }
            v[u] = __ldg(x + (static_cast<size_t>(src) * kb + kp[u]) * 16 + sub);
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        uint2 codes;
        uint32_t const byte = quant8_shared4(v[u], codes);
        uint32_t const word = word_from_16lanes(byte, sub);
        if (c0 + u < total) {
            bool const live = row[u] < m;
            if (live) q[(static_cast<size_t>(row[u]) * kb + kp[u]) * 16 + sub] = codes;
            if (sub == 0) sf[sf_word_index(row[u], kp[u], kb)] = live ? word : 0u;
        }
    }
}

// The same rule with 16 elements per thread (one 256-bit load, one 128-bit store): 2 lanes per 1x32 block, 8 lanes
// per scale word, half the shuffles and index arithmetic per element. Needs a 32-byte aligned input.
__device__ __forceinline__ void ld_nc_256(const void* p, uint32_t (&r)[8])
{
    asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}

__device__ __forceinline__ uint32_t quant16_shared2(uint32_t const (&v)[8], uint4& out)
{
    uint32_t m = absmax_words(v, false);
    m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
    if (__any_sync(0xFFFFFFFFu, m > 0x7F80u)) {            // a NaN somewhere in the warp's blocks: leave NaNs out
        m = absmax_words(v, true);
        m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
    }
    float const amax = fmaxf(__uint_as_float(m << 16), 1e-10f);
    float qs;
    uint32_t const byte = e8m0_from_amax(amax, qs);
    auto lo = [](uint32_t w) { return __uint_as_float(w << 16); };
    auto hi = [](uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); };
    out.x = fp8x4(__fmul_rn(lo(v[0]), qs), __fmul_rn(hi(v[0]), qs), __fmul_rn(lo(v[1]), qs), __fmul_rn(hi(v[1]), qs));
    out.y = fp8x4(__fmul_rn(lo(v[2]), qs), __fmul_rn(hi(v[2]), qs), __fmul_rn(lo(v[3]), qs), __fmul_rn(hi(v[3]), qs));
    out.z = fp8x4(__fmul_rn(lo(v[4]), qs), __fmul_rn(hi(v[4]), qs), __fmul_rn(lo(v[5]), qs), __fmul_rn(hi(v[5]), qs));
    out.w = fp8x4(__fmul_rn(lo(v[6]), qs), __fmul_rn(hi(v[6]), qs), __fmul_rn(lo(v[7]), qs), __fmul_rn(hi(v[7]), qs));
    return byte;
}

__device__ __forceinline__ uint32_t word_from_8lanes(uint32_t byte, uint32_t sub8)
{
    uint32_t w = byte << (8 * (sub8 >> 1));
    w |= __shfl_xor_sync(0xFFFFFFFFu, w, 2);
    w |= __shfl_xor_sync(0xFFFFFFFFu, w, 4);
    return w;
}

template <int kUnroll>
__global__ void __launch_bounds__(256) quantize_1x32_wide_kernel(const uint8_t* __restrict__ x, uint4* __restrict__ q,
    uint32_t* __restrict__ sf, uint32_t m, uint32_t m_pad, uint32_t kb, uint32_t interleave_i, uint32_t early)
{
    if (early) {
        griddep_launch_dependents();
        griddep_wait();
    }
    uint32_t const sub = threadIdx.x & 7;
    uint32_t const oct = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;      // 8 lanes per 128-element chunk
    uint32_t const total = m_pad * kb;
    uint32_t const c0 = oct * kUnroll;
    uint32_t row0 = c0 / kb;
    uint32_t kp0 = c0 - row0 * kb;
    uint32_t v[kUnroll][8];
    uint32_t row[kUnroll];
    uint32_t kp[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        row[u] = row0;
        kp[u] = kp0;
        if (++kp0 == kb) {
            kp0 = 0;
            ++row0;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = 0;
        if (c0 + u < total && row[u] < m) {
            uint32_t src = row[u];
            if (interleave_i > 0) {
                uint32_t const two_i = 2 * interleave_i;
                uint32_t const g = src / two_i, o = src - g * two_i;
                src = g * two_i + ((o & 1) ? interleave_i + (o >> 1) : (o >> 1));
            }
            ld_nc_256(x + ((static_cast<size_t>(src) * kb + kp[u]) * 8 + sub) * 32, v[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        uint4 codes;
        uint32_t const byte = quant16_shared2(v[u], codes);
        uint32_t const word = word_from_8lanes(byte, sub);
        if (c0 + u < total) {
            bool const live = row[u] < m;
            if (live) q[(static_cast<size_t>(row[u]) * kb + kp[u]) * 8 + sub] = codes;
            if (sub == 0) sf[sf_word_index(row[u], kp[u], kb)] = live ? word : 0u;
        }
    }
}

inline bool quantizer_pdl_enabled()
{
    static int const v = [] {
        const char* e = getenv("FSO_B200_PDL");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    return v != 0;
}

// early: the activation form, which lets a decode GEMM launched behind it (programmatic dependent launch) read its
// weights while this kernel runs. Never for a call whose output the next kernel uses as a weight.
inline int launch_quantize_1x32(const void* x, void* q, void* sf, int64_t m, int64_t k, int64_t interleave_i,
    cudaStream_t stream, bool early = false)
{
    constexpr int kUnroll = 4;
    int64_t const m_pad = (m + 127) / 128 * 128;
    int const kb = static_cast<int>(k / 128);
    int64_t const halves = (m_pad * kb + kUnroll - 1) / kUnroll;
    int64_t const blocks = (halves * 16 + 255) / 256;
    if (m_pad * kb >= (1ll << 31) - 4096 || m_pad >= (1ll << 31)) {
        set_error("fso_quantize_1x32: %lld x %lld is beyond the kernel's 2^31-chunk index range; split the call by rows",
            static_cast<long long>(m), static_cast<long long>(k));
        return FSO_ERR_INVALID;
    }
    // the activation form is itself launched with the programmatic-serialization attribute (it waits at its top)
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (early && quantizer_pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    if ((reinterpret_cast<uintptr_t>(x) & 31u) == 0) {
        constexpr int kWide = 2;
        int64_t const octs = (m_pad * kb + kWide - 1) / kWide;
        int64_t const wblocks = (octs * 8 + 255) / 256;
        cfg.gridDim = dim3(static_cast<unsigned>(wblocks), 1, 1);
        FSO_CUDA(cudaLaunchKernelEx(&cfg, quantize_1x32_wide_kernel<kWide>, static_cast<const uint8_t*>(x),
            static_cast<uint4*>(q), static_cast<uint32_t*>(sf), static_cast<uint32_t>(m), static_cast<uint32_t>(m_pad),
            static_cast<uint32_t>(kb), static_cast<uint32_t>(interleave_i), early ? 1u : 0u));
        return launch_status("fso_quantize_1x32");
    }
    cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
    FSO_CUDA(cudaLaunchKernelEx(&cfg, quantize_1x32_kernel<kUnroll>, static_cast<const uint4*>(x), static_cast<uint2*>(q),
        static_cast<uint32_t*>(sf), static_cast<uint32_t>(m), static_cast<uint32_t>(m_pad), static_cast<uint32_t>(kb),
        static_cast<uint32_t>(interleave_i), early ? 1u : 0u));
    return launch_status("fso_quantize_1x32");
}

// ------------------------------------------------------------------------------------------- SiLU(gate) * up -> MXFP8

// gu bf16 [M, 2I]: columns [0, I) are the gate, [I, 2I) the up projection. h = silu(gate) * up in fp32 (hardware
// tanh approximation: silu(g) = 0.5 g (1 + tanh(0.5 g))), quantized with the 1x32 rule without h ever reaching
// memory. 16 outputs per thread (two 256-bit loads, one 128-bit store), 2 lanes per 1x32 block, 8 per scale word.
// Rows in [m, m_pad) only get their zero scale words.
__global__ void __launch_bounds__(256) silu_mul_quantize_kernel(const uint8_t* __restrict__ gu, uint4* __restrict__ q,
    uint32_t* __restrict__ sf, uint32_t m, uint32_t m_pad, uint32_t kb)
{
    griddep_launch_dependents();      // the down projection launched behind this kernel may start loading weights
    griddep_wait();                   // gu is the gate_up projection's output
    uint32_t const sub = threadIdx.x & 7;
    uint32_t const c = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;        // chunk (row, kp) of the output
    if (c >= m_pad * kb) return;                                            // whole groups of 8 lanes leave together
    uint32_t const row = c / kb;
    uint32_t const kp = c - row * kb;
    bool const live = row < m;
    uint32_t g[8], u[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = u[i] = 0;
    if (live) {
        const uint8_t* const src = gu + (static_cast<size_t>(row) * (2 * kb) + kp) * 256 + sub * 32;
        ld_nc_256(src, g);
        ld_nc_256(src + static_cast<size_t>(kb) * 256, u);
    }
    float h[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float const g0 = __uint_as_float(g[i] << 16), g1 = __uint_as_float(g[i] & 0xFFFF0000u);
        float const u0 = __uint_as_float(u[i] << 16), u1 = __uint_as_float(u[i] & 0xFFFF0000u);
        float t0, t1;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(0.5f * g0));
        asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(0.5f * g1));
        h[2 * i] = (0.5f * g0) * (1.f + t0) * u0;
        h[2 * i + 1] = (0.5f * g1) * (1.f + t1) * u1;
        amax = fmaxf(amax, fmaxf(fabsf(h[2 * i]), fabsf(h[2 * i + 1])));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, 1e-10f);
    float qs;
    uint32_t const byte = e8m0_from_amax(amax, qs);
    uint32_t const word = word_from_8lanes(byte, sub);
    if (live) {
        uint4 o;
        o.x = fp8x4(__fmul_rn(h[0], qs), __fmul_rn(h[1], qs), __fmul_rn(h[2], qs), __fmul_rn(h[3], qs));
        o.y = fp8x4(__fmul_rn(h[4], qs), __fmul_rn(h[5], qs), __fmul_rn(h[6], qs), __fmul_rn(h[7], qs));
        o.z = fp8x4(__fmul_rn(h[8], qs), __fmul_rn(h[9], qs), __fmul_rn(h[10], qs), __fmul_rn(h[11], qs));
        o.w = fp8x4(__fmul_rn(h[12], qs), __fmul_rn(h[13], qs), __fmul_rn(h[14], qs), __fmul_rn(h[15], qs));
        q[(static_cast<size_t>(row) * kb + kp) * 8 + sub] = o;
    }
    if (sub == 0) sf[sf_word_index(row, kp, kb)] = live ? word : 0u;
}

// The same step for the decode band of the MoE layer: gu is the fp32 [rows, 2I] output of the grouped FC1 over the
// compact activation (the accumulators, so that the activation sees what the fused epilogue of the prefill kernels
// sees) with its columns in the experts' interleaved order (gate_j, up_j adjacent); only the routed rows of the
// blocks in use are read and written (row r of block b is routed when r % 128 < rows of the block's expert that fall
// into this block). 16 outputs per thread from 128 contiguous input bytes.
__global__ void __launch_bounds__(256) silu_mul_quantize_rows_kernel(const uint8_t* __restrict__ gu,
    uint4* __restrict__ q, uint32_t* __restrict__ sf, const int32_t* __restrict__ masked_m,
    const int32_t* __restrict__ blk0, const int32_t* __restrict__ blk_expert, int num_experts, uint32_t rows_bound,
    uint32_t kb)
{
    griddep_launch_dependents();
    griddep_wait();
    uint32_t const sub = threadIdx.x & 7;
    uint32_t const c = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    if (c >= rows_bound * kb) return;                                       // whole groups of 8 lanes leave together
    uint32_t const row = c / kb;
    uint32_t const kp = c - row * kb;
    int const block = static_cast<int>(row >> 7);
    bool live = false;
    if (block < __ldg(blk0 + num_experts)) {
        int const e = __ldg(blk_expert + block);
        live = static_cast<int>(row & 127u) < __ldg(masked_m + e) - 128 * (block - __ldg(blk0 + e));
    }
    uint32_t v[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j][i] = 0;
    if (live) {
        const uint8_t* const src = gu + (static_cast<size_t>(row) * kb + kp) * 1024 + sub * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) ld_nc_256(src + 32 * j, v[j]);
    }
    float h[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float const g0 = __uint_as_float(v[i >> 2][2 * (i & 3)]), u0 = __uint_as_float(v[i >> 2][2 * (i & 3) + 1]);
        float t0;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(0.5f * g0));
        h[i] = (0.5f * g0) * (1.f + t0) * u0;
        amax = fmaxf(amax, fabsf(h[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, 1e-10f);
    float qs;
    uint32_t const byte = e8m0_from_amax(amax, qs);
    uint32_t const word = word_from_8lanes(byte, sub);
    if (live) {
        uint4 o;
        o.x = fp8x4(__fmul_rn(h[0], qs), __fmul_rn(h[1], qs), __fmul_rn(h[2], qs), __fmul_rn(h[3], qs));
        o.y = fp8x4(__fmul_rn(h[4], qs), __fmul_rn(h[5], qs), __fmul_rn(h[6], qs), __fmul_rn(h[7], qs));
        o.z = fp8x4(__fmul_rn(h[8], qs), __fmul_rn(h[9], qs), __fmul_rn(h[10], qs), __fmul_rn(h[11], qs));
        o.w = fp8x4(__fmul_rn(h[12], qs), __fmul_rn(h[13], qs), __fmul_rn(h[14], qs), __fmul_rn(h[15], qs));
        q[(static_cast<size_t>(row) * kb + kp) * 8 + sub] = o;
        if (sub == 0) sf[sf_word_index(row, kp, kb)] = word;
    }
}

inline int launch_silu_mul_quantize_rows(const void* gu, void* q, void* sf, const int32_t* masked_m, const int32_t* blk0,
    const int32_t* blk_expert, int64_t num_experts, int64_t rows_bound, int64_t inter, cudaStream_t stream)
{
    int const kb = static_cast<int>(inter / 128);
    if (rows_bound * kb >= (1ll << 28)) {
        set_error("fso_moe_silu_mul_quantize_rows: %lld x %lld is beyond the kernel's index range",
            static_cast<long long>(rows_bound), static_cast<long long>(inter));
        return FSO_ERR_INVALID;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>((rows_bound * kb * 8 + 255) / 256), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (quantizer_pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    FSO_CUDA(cudaLaunchKernelEx(&cfg, silu_mul_quantize_rows_kernel, static_cast<const uint8_t*>(gu),
        static_cast<uint4*>(q), static_cast<uint32_t*>(sf), masked_m, blk0, blk_expert, static_cast<int>(num_experts),
        static_cast<uint32_t>(rows_bound), static_cast<uint32_t>(kb)));
    return launch_status("silu_mul_quantize_rows_kernel");
}

inline int launch_silu_mul_quantize(const void* gu, void* q, void* sf, int64_t m, int64_t inter, cudaStream_t stream)
{
    int64_t const m_pad = (m + 127) / 128 * 128;
    int const kb = static_cast<int>(inter / 128);
    if (m_pad * kb >= (1ll << 28)) {
        set_error("fso_silu_mul_quantize_1x32: %lld x %lld is beyond the kernel's index range; split the call by rows",
            static_cast<long long>(m), static_cast<long long>(inter));
        return FSO_ERR_INVALID;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>((m_pad * kb * 8 + 255) / 256), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (quantizer_pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    FSO_CUDA(cudaLaunchKernelEx(&cfg, silu_mul_quantize_kernel, static_cast<const uint8_t*>(gu), static_cast<uint4*>(q),
        static_cast<uint32_t*>(sf), static_cast<uint32_t>(m), static_cast<uint32_t>(m_pad), static_cast<uint32_t>(kb)));
    return launch_status("silu_mul_quantize_kernel");
}

// ---------------------------------------------------------------------------------------------------- block-FP8 -> MXFP8

// 16 e4m3 codes per thread (one 16-byte load); 2 lanes per 32-element block, 8 lanes per 128-element chunk.
// value = bf16_rne(float(code) * s_tile) in fp32 with one rounding, then the 1x32 rule on those bf16 values.
__global__ void __launch_bounds__(256) requant_bs128_kernel(const uint4* __restrict__ wq, const float* __restrict__ s128,
    uint4* __restrict__ q, uint32_t* __restrict__ sf, int64_t n, int kb, int64_t interleave_i)
{
    int const sub = threadIdx.x & 7;
    int64_t const c = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;   // chunk (row, kp)
    int64_t const total = n * kb;
    bool const live = c < total;
    int64_t const row = live ? c / kb : 0;
    int const kp = live ? static_cast<int>(c - row * kb) : 0;
    uint4 v = make_uint4(0, 0, 0, 0);
    float s = 0.f;
    if (live) {
        int64_t src = row;
        if (interleave_i > 0) {
            int64_t const two_i = 2 * interleave_i;
            int64_t const g = src / two_i, o = src - g * two_i;
            src = g * two_i + ((o & 1) ? interleave_i + (o >> 1) : (o >> 1));
        }
        v = __ldg(wq + (src * kb + kp) * 8 + sub);
        s = __ldg(s128 + (src >> 7) * kb + kp);
    }
    float f[16];
    uint32_t const w[4] = {v.x, v.y, v.z, v.w};
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            __half2_raw const hr = __nv_cvt_fp8x2_to_halfraw2(
                static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * h)) & 0xFFFFu), __NV_E4M3);
            float2 const p = __half22float2(*reinterpret_cast<const __half2*>(&hr));
            float const a = __bfloat162float(__float2bfloat16_rn(__fmul_rn(p.x, s)));
            float const b = __bfloat162float(__float2bfloat16_rn(__fmul_rn(p.y, s)));
            f[i * 4 + h * 2] = a;
            f[i * 4 + h * 2 + 1] = b;
            amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
        }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, 1e-10f);
    float qs;
    uint32_t const byte = e8m0_from_amax(amax, qs);
    uint4 out;
    out.x = fp8x4(__fmul_rn(f[0], qs), __fmul_rn(f[1], qs), __fmul_rn(f[2], qs), __fmul_rn(f[3], qs));
    out.y = fp8x4(__fmul_rn(f[4], qs), __fmul_rn(f[5], qs), __fmul_rn(f[6], qs), __fmul_rn(f[7], qs));
    out.z = fp8x4(__fmul_rn(f[8], qs), __fmul_rn(f[9], qs), __fmul_rn(f[10], qs), __fmul_rn(f[11], qs));
    out.w = fp8x4(__fmul_rn(f[12], qs), __fmul_rn(f[13], qs), __fmul_rn(f[14], qs), __fmul_rn(f[15], qs));
    uint32_t word = byte << (8 * (sub >> 1));
    word |= __shfl_xor_sync(0xFFFFFFFFu, word, 2);
    word |= __shfl_xor_sync(0xFFFFFFFFu, word, 4);
    if (live) {
        q[(row * kb + kp) * 8 + sub] = out;
        if (sub == 0) sf[sf_word_index(row, kp, kb)] = word;
    }
}

// The same with 32 codes per thread (one 256-bit load, one 256-bit store): one lane per 1x32 block, so the amax
// needs no shuffle, 4 lanes per scale word, 32-bit index arithmetic. Needs 32-byte aligned wq / q and
// n * K/128 * 4 < 2^31.
__global__ void __launch_bounds__(256) requant_bs128_wide_kernel(const uint8_t* __restrict__ wq,
    const float* __restrict__ s128, uint8_t* __restrict__ q, uint32_t* __restrict__ sf, uint32_t n, uint32_t kb,
    uint32_t interleave_i)
{
    uint32_t const sub = threadIdx.x & 3;
    uint32_t const c = (blockIdx.x * blockDim.x + threadIdx.x) >> 2;        // chunk (row, kp)
    bool const live = c < n * kb;
    uint32_t const row = live ? c / kb : 0;
    uint32_t const kp = live ? c - row * kb : 0;
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = 0;
    float s = 0.f;
    if (live) {
        uint32_t src = row;
        if (interleave_i > 0) {
            uint32_t const two_i = 2 * interleave_i;
            uint32_t const g = src / two_i, o = src - g * two_i;
            src = g * two_i + ((o & 1) ? interleave_i + (o >> 1) : (o >> 1));
        }
        ld_nc_256(wq + (static_cast<size_t>(src) * kb + kp) * 128 + sub * 32, w);
        s = __ldg(s128 + static_cast<size_t>(src >> 7) * kb + kp);
    }
    float f[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            __half2_raw const hr = __nv_cvt_fp8x2_to_halfraw2(
                static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * h)) & 0xFFFFu), __NV_E4M3);
            float2 const p = __half22float2(*reinterpret_cast<const __half2*>(&hr));
            float const a = __bfloat162float(__float2bfloat16_rn(__fmul_rn(p.x, s)));
            float const b = __bfloat162float(__float2bfloat16_rn(__fmul_rn(p.y, s)));
            f[i * 4 + h * 2] = a;
            f[i * 4 + h * 2 + 1] = b;
            amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
        }
    }
    amax = fmaxf(amax, 1e-10f);
    float qs;
    uint32_t const byte = e8m0_from_amax(amax, qs);
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        o[i] = fp8x4(__fmul_rn(f[4 * i], qs), __fmul_rn(f[4 * i + 1], qs), __fmul_rn(f[4 * i + 2], qs),
            __fmul_rn(f[4 * i + 3], qs));
    uint32_t word = byte << (8 * sub);
    word |= __shfl_xor_sync(0xFFFFFFFFu, word, 1);
    word |= __shfl_xor_sync(0xFFFFFFFFu, word, 2);
    if (live) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"l"(q + (static_cast<size_t>(row) * kb + kp) * 128 + sub * 32), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                     "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                     : "memory");
        if (sub == 0) sf[sf_word_index(row, kp, kb)] = word;
    }
}

inline int launch_requant_bs128(const void* wq, const float* s128, void* q, void* sf, int64_t n, int64_t k,
    int64_t interleave_i, cudaStream_t stream)
{
    int const kb = static_cast<int>(k / 128);
    if (((reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(q)) & 31u) == 0
        && n * kb * 4 < (1ll << 31) - 4096 && interleave_i < (1ll << 30)) {
        int64_t const wblocks = (n * kb * 4 + 255) / 256;
        requant_bs128_wide_kernel<<<static_cast<unsigned>(wblocks), 256, 0, stream>>>(static_cast<const uint8_t*>(wq),
            s128, static_cast<uint8_t*>(q), static_cast<uint32_t*>(sf), static_cast<uint32_t>(n),
            static_cast<uint32_t>(kb), static_cast<uint32_t>(interleave_i));
        return launch_status("fso_requant_bs128_to_mx");
    }
    int64_t const blocks = (n * kb * 8 + 255) / 256;
    requant_bs128_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const uint4*>(wq), s128,
        static_cast<uint4*>(q), static_cast<uint32_t*>(sf), n, kb, interleave_i);
    return launch_status("fso_requant_bs128_to_mx");
}

// ---------------------------------------------------------------------------------------------------- scale packer

// One thread per output word (group, padded row, kp); padded rows get zero words.
__global__ void __launch_bounds__(256) pack_ue8m0_kernel(const uint8_t* __restrict__ s, uint32_t* __restrict__ out,
    int64_t g, int64_t n, int64_t n_pad, int kb, int64_t interleave_i)
{
    int64_t const idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    int64_t const slab = n_pad * kb;
    if (idx >= g * slab) return;
    int64_t const e = idx / slab;
    int64_t const rem = idx - e * slab;
    int64_t const r = rem / kb;
    int const kp = static_cast<int>(rem - r * kb);
    uint32_t word = 0;
    if (r < n) {
        int64_t src = r;
        if (interleave_i > 0) src = (r & 1) ? interleave_i + (r >> 1) : (r >> 1);
        const uint8_t* b = s + ((e * n + src) * kb + kp) * 4;
        word = static_cast<uint32_t>(b[0]) | (static_cast<uint32_t>(b[1]) << 8) | (static_cast<uint32_t>(b[2]) << 16)
            | (static_cast<uint32_t>(b[3]) << 24);
    }
    out[e * slab + sf_word_index(r, kp, kb)] = word;
}

inline int launch_pack_ue8m0(const void* s, void* out, int64_t g, int64_t n, int64_t k, int64_t interleave_i,
    cudaStream_t stream)
{
    int const kb = static_cast<int>(k / 128);
    int64_t const n_pad = (n + 127) / 128 * 128;
    int64_t const total = g * n_pad * kb;
    pack_ue8m0_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
        static_cast<const uint8_t*>(s), static_cast<uint32_t*>(out), g, n, n_pad, kb, interleave_i);
    return launch_status("fso_pack_ue8m0");
}

}  // namespace fso
