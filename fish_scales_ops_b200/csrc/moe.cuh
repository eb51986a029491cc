// MoE glue kernels around the grouped GEMMs: compact routing (deterministic order), token gather + quantize,
// and the top-k weighted un-permute / reduce. All of them are integer / byte work bound by HBM or latency.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"
#include "quant.cuh"

namespace fso {

constexpr int kRouteSeg = 1024;   // pairs per routing segment == threads per routing CTA

// Rank of every pair of one 1024-pair segment among the segment's pairs of the same expert, in ascending flat
// index, and the segment's per-expert totals.
//   in : e (expert of this thread's pair, any value when !valid)
//   out: returns the rank; s_cnt[x] = pairs of expert x in this segment (valid after the function returns)
// s_wbase is [32][num_experts] uint16 scratch. Deterministic: no atomics.
__device__ __forceinline__ int segment_rank(int e, bool valid, int num_experts, int* s_cnt, uint16_t* s_wbase)
{
    int const tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 32 * num_experts; i += kRouteSeg) s_wbase[i] = 0;
    __syncthreads();
    unsigned const peers = __match_any_sync(0xFFFFFFFFu, valid ? e : -1);
    int const rank_w = __popc(peers & ((1u << lane) - 1u));
    if (valid && rank_w == 0) s_wbase[warp * num_experts + e] = static_cast<uint16_t>(__popc(peers));
    __syncthreads();
    for (int x = tid; x < num_experts; x += kRouteSeg) {
        int run = 0;
#pragma unroll 4
        for (int w = 0; w < 32; ++w) {
            int const c = s_wbase[w * num_experts + x];
            s_wbase[w * num_experts + x] = static_cast<uint16_t>(run);
            run += c;
        }
        s_cnt[x] = run;
    }
    __syncthreads();
    return valid ? static_cast<int>(s_wbase[warp * num_experts + e]) + rank_w : 0;
}

// Exclusive scan over experts of ceil(cnt / 128) by one 1024-thread CTA (num_experts <= 1024); thread x returns
// the prefix of expert x, *total gets the sum. s_tmp is 33 ints.
__device__ __forceinline__ int block_prefix_blocks(int cnt, int* s_tmp, int* total)
{
    int const tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int const v = (cnt + 127) >> 7;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int const o = __shfl_up_sync(0xFFFFFFFFu, inc, d);
        if (lane >= d) inc += o;
    }
    if (lane == 31) s_tmp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = s_tmp[lane];
        int winc = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int const o = __shfl_up_sync(0xFFFFFFFFu, winc, d);
            if (lane >= d) winc += o;
        }
        s_tmp[lane] = winc - w;
        if (lane == 31) s_tmp[32] = winc;
    }
    __syncthreads();
    *total = s_tmp[32];
    return s_tmp[warp] + inc - v;
}

__device__ __forceinline__ void fill_block_experts(int x, int num_experts, int start, int cnt, int total_blocks,
    int num_blocks, int32_t* blk_expert)
{
    if (x < num_experts) {
        int const nb = (cnt + 127) >> 7;
        for (int b = start; b < start + nb && b < num_blocks; ++b) blk_expert[b] = x;
    }
    for (int b = total_blocks + x; b < num_blocks; b += kRouteSeg) blk_expert[b] = -1;
}

// pairs <= 1024: everything in one CTA.
__global__ void __launch_bounds__(kRouteSeg) route_small_kernel(const int32_t* __restrict__ ids, int pairs,
    int num_experts, int num_blocks, int32_t* __restrict__ masked_m, int32_t* __restrict__ blk0,
    int32_t* __restrict__ slot_of_flat, int32_t* __restrict__ blk_expert)
{
    extern __shared__ uint16_t s_wbase[];
    __shared__ int s_cnt[1024];
    __shared__ int s_blk[1024];
    __shared__ int s_tmp[33];
    int const tid = threadIdx.x;
    int const e = tid < pairs ? ids[tid] : -1;
    bool const valid = e >= 0 && e < num_experts;
    int const rank = segment_rank(e, valid, num_experts, s_cnt, s_wbase);
    int const cnt = tid < num_experts ? s_cnt[tid] : 0;
    int total;
    int const start = block_prefix_blocks(cnt, s_tmp, &total);
    if (tid < num_experts) {
        masked_m[tid] = cnt;
        blk0[tid] = start;
        s_blk[tid] = start;
    }
    if (tid == 0) blk0[num_experts] = total;
    fill_block_experts(tid, num_experts, start, cnt, total, num_blocks, blk_expert);
    __syncthreads();
    if (tid < pairs) slot_of_flat[tid] = valid ? s_blk[e] * 128 + rank : -1;
}

// pairs > 1024, pass 1: per-segment per-expert counts -> seg_cnt[segment][expert].
__global__ void __launch_bounds__(kRouteSeg) route_count_kernel(const int32_t* __restrict__ ids, int pairs,
    int num_experts, int32_t* __restrict__ seg_cnt)
{
    extern __shared__ uint16_t s_wbase[];
    __shared__ int s_cnt[1024];
    int const i = blockIdx.x * kRouteSeg + threadIdx.x;
    int const e = i < pairs ? ids[i] : -1;
    bool const valid = e >= 0 && e < num_experts;
    (void)segment_rank(e, valid, num_experts, s_cnt, s_wbase);
    for (int x = threadIdx.x; x < num_experts; x += kRouteSeg) seg_cnt[blockIdx.x * num_experts + x] = s_cnt[x];
}

// pass 2 (one CTA): seg_cnt -> exclusive prefix over segments (in place), expert totals, block prefix, block table.
__global__ void __launch_bounds__(kRouteSeg) route_scan_kernel(int32_t* __restrict__ seg_cnt, int segments,
    int num_experts, int num_blocks, int32_t* __restrict__ masked_m, int32_t* __restrict__ blk0,
    int32_t* __restrict__ blk_expert)
{
    __shared__ int s_tmp[33];
    int const tid = threadIdx.x;
    int cnt = 0;
    if (tid < num_experts) {
        for (int s = 0; s < segments; ++s) {
            int const c = seg_cnt[s * num_experts + tid];
            seg_cnt[s * num_experts + tid] = cnt;
            cnt += c;
        }
    }
    int total;
    int const start = block_prefix_blocks(cnt, s_tmp, &total);
    if (tid < num_experts) {
        masked_m[tid] = cnt;
        blk0[tid] = start;
    }
    if (tid == 0) blk0[num_experts] = total;
    fill_block_experts(tid, num_experts, start, cnt, total, num_blocks, blk_expert);
}

// pass 3: place every pair.
__global__ void __launch_bounds__(kRouteSeg) route_place_kernel(const int32_t* __restrict__ ids, int pairs,
    int num_experts, const int32_t* __restrict__ seg_base, const int32_t* __restrict__ blk0,
    int32_t* __restrict__ slot_of_flat)
{
    extern __shared__ uint16_t s_wbase[];
    __shared__ int s_cnt[1024];
    int const i = blockIdx.x * kRouteSeg + threadIdx.x;
    int const e = i < pairs ? ids[i] : -1;
    bool const valid = e >= 0 && e < num_experts;
    int const rank = segment_rank(e, valid, num_experts, s_cnt, s_wbase);
    if (i < pairs)
        slot_of_flat[i] = valid ? blk0[e] * 128 + seg_base[blockIdx.x * num_experts + e] + rank : -1;
}

// ---------------------------------------------------------------------------------------------------- gather + quantize

// One (token, 128-element chunk) per half-warp and step: the token is quantized once and its codes and scale word
// are stored to each of its top-k compact rows (skipped pairs store nothing).
template <int kUnroll>
__global__ void __launch_bounds__(256) gather_quant_kernel(const uint4* __restrict__ hidden,
    const int32_t* __restrict__ slot_of_flat, int64_t tokens, int topk, int kb, uint2* __restrict__ hq,
    uint32_t* __restrict__ sh)
{
    // 32-bit index arithmetic (the launcher refuses more than 2^31 chunks)
    uint32_t const sub = threadIdx.x & 15;
    uint32_t const half = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    uint32_t const total = static_cast<uint32_t>(tokens) * static_cast<uint32_t>(kb);
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        uint32_t const c = half * kUnroll + u;
        v[u] = c < total ? __ldg(hidden + static_cast<size_t>(c) * 16 + sub) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        uint32_t const c = half * kUnroll + u;
        uint2 codes;
        uint32_t const byte = quant8_shared4(v[u], codes);
        uint32_t const word = word_from_16lanes(byte, sub);
        if (c < total) {
            uint32_t const t = c / static_cast<uint32_t>(kb);
            int const kp = static_cast<int>(c - t * kb);
            for (int j = 0; j < topk; ++j) {
                int const slot = __ldg(slot_of_flat + static_cast<size_t>(t) * topk + j);
                if (slot >= 0) {
                    hq[(static_cast<int64_t>(slot) * kb + kp) * 16 + sub] = codes;
                    if (sub == 0) sh[sf_word_index(slot, kp, kb)] = word;
                }
            }
        }
    }
}

// The same with 16 elements per thread (256-bit loads, 128-bit stores, 8 lanes per chunk); needs a 32-byte aligned
// hidden tensor.
template <int kUnroll>
__global__ void __launch_bounds__(256) gather_quant_wide_kernel(const uint8_t* __restrict__ hidden,
    const int32_t* __restrict__ slot_of_flat, int64_t tokens, int topk, int kb, uint4* __restrict__ hq,
    uint32_t* __restrict__ sh)
{
    uint32_t const sub = threadIdx.x & 7;
    uint32_t const oct = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    uint32_t const total = static_cast<uint32_t>(tokens) * static_cast<uint32_t>(kb);
    uint32_t v[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        uint32_t const c = oct * kUnroll + u;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = 0;
        if (c < total) ld_nc_256(hidden + (static_cast<size_t>(c) * 8 + sub) * 32, v[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        uint32_t const c = oct * kUnroll + u;
        uint4 codes;
        uint32_t const byte = quant16_shared2(v[u], codes);
        uint32_t const word = word_from_8lanes(byte, sub);
        if (c < total) {
            uint32_t const t = c / static_cast<uint32_t>(kb);
            int const kp = static_cast<int>(c - t * kb);
            for (int j = 0; j < topk; ++j) {
                int const slot = __ldg(slot_of_flat + static_cast<size_t>(t) * topk + j);
                if (slot >= 0) {
                    hq[(static_cast<int64_t>(slot) * kb + kp) * 8 + sub] = codes;
                    if (sub == 0) sh[sf_word_index(slot, kp, kb)] = word;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------- combine

// One (token, 8 columns) per thread: fp32 FMA chain over the token's top-k rows in ascending j, then the bias term,
// one rounding to bf16.
template <int kMaxTopk>
__global__ void __launch_bounds__(256) combine_kernel(const uint4* __restrict__ dn,
    const int32_t* __restrict__ slot_of_flat, const float* __restrict__ topk_w, const uint4* __restrict__ bias,
    const float* __restrict__ bias_scale, uint4* __restrict__ out, int64_t tokens, int topk, int h8)
{
    // 32-bit index arithmetic (the launcher refuses tokens * H/8 >= 2^31)
    uint32_t const idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= static_cast<uint32_t>(tokens) * static_cast<uint32_t>(h8)) return;
    uint32_t const t32 = idx / static_cast<uint32_t>(h8);
    int const c = static_cast<int>(idx - t32 * h8);
    int64_t const t = t32;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto fma_row = [&](uint4 const& raw, float w) {
        uint32_t const ws[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] = fmaf(w, __uint_as_float(ws[i] << 16), acc[2 * i]);
            acc[2 * i + 1] = fmaf(w, __uint_as_float(ws[i] & 0xFFFF0000u), acc[2 * i + 1]);
        }
    };
    if (topk <= kMaxTopk) {
        int slots[kMaxTopk];
        float ws[kMaxTopk];
        uint4 raws[kMaxTopk];
#pragma unroll
        for (int j = 0; j < kMaxTopk; ++j)
            if (j < topk) {
                slots[j] = __ldg(slot_of_flat + t * topk + j);
                ws[j] = __ldg(topk_w + t * topk + j);
            }
#pragma unroll
        for (int j = 0; j < kMaxTopk; ++j)
            if (j < topk) raws[j] = slots[j] >= 0 ? __ldg(dn + static_cast<int64_t>(slots[j]) * h8 + c)
                                                   : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < kMaxTopk; ++j)
            if (j < topk && slots[j] >= 0) fma_row(raws[j], ws[j]);
    } else {
        for (int j = 0; j < topk; ++j) {
            int const slot = __ldg(slot_of_flat + t * topk + j);
            if (slot >= 0) fma_row(__ldg(dn + static_cast<int64_t>(slot) * h8 + c), __ldg(topk_w + t * topk + j));
        }
    }
    if (bias != nullptr) fma_row(__ldg(bias + t * h8 + c), bias_scale != nullptr ? __ldg(bias_scale + t) : 1.f);
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    out[idx] = o;
}

// Where the combine's output rows go when they are not one dense [tokens, H] tensor: token t, which lies in
// [recv_off[s], recv_off[s + 1]) for exactly one s < world, is written to row back_base[s] + (t - recv_off[s]) of the
// bf16 [*, H] buffer at address peer_back[s] (another GPU's memory under expert parallelism). world == 0: dense.
// Tokens are then visited in the order (v * row_mul) mod tokens (row_mul coprime to tokens) so that the rows in flight
// at any moment are spread over all destinations. The kernel issues no system-scope fence of its own (one per CTA
// cost 0.3 ms per layer, the CTA stays resident until every peer store is acknowledged): its stores are complete
// when the kernel is, and the next rank reads them only after a stream-ordered collective that follows the kernel.
struct RowScatter {
    const int64_t* recv_off;
    const int64_t* back_base;
    const uint64_t* peer_back;
    int world;
    int64_t row_mul;
};

// The combine with 256-bit accesses: one thread owns kGroups x 16 columns of one token, so that about eight 32-byte
// row loads are in flight per thread whatever the top-k (top-2 -> 4 groups, top-8 -> 1 group). Same arithmetic and
// order as combine_kernel. Needs 32-byte aligned dn / out / bias and H % (16 * kGroups) == 0.
template <int kMaxTopk, int kGroups>
__global__ void __launch_bounds__(256) combine_wide_kernel(const uint8_t* __restrict__ dn,
    const int32_t* __restrict__ slot_of_flat, const float* __restrict__ topk_w, const uint8_t* __restrict__ bias,
    const float* __restrict__ bias_scale, uint8_t* __restrict__ out, int64_t tokens, int topk, int h_bytes,
    RowScatter sc)
{
    constexpr int kSpan = 32 * kGroups;                      // bytes of one row this thread owns
    uint32_t const per_row = static_cast<uint32_t>(h_bytes) / kSpan;
    uint32_t const idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= static_cast<uint32_t>(tokens) * per_row) return;
    uint32_t const t32 = idx / per_row;
    size_t const col = static_cast<size_t>(idx - t32 * per_row) * kSpan;
    int64_t const t = sc.world > 0
        ? static_cast<int64_t>((static_cast<unsigned long long>(t32) * sc.row_mul) % static_cast<unsigned long long>(tokens))
        : static_cast<int64_t>(t32);
    float acc[16 * kGroups];
#pragma unroll
    for (int i = 0; i < 16 * kGroups; ++i) acc[i] = 0.f;
    auto fma_row = [&](uint32_t const (&raw)[8], float w, int g) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[g * 16 + 2 * i] = fmaf(w, __uint_as_float(raw[i] << 16), acc[g * 16 + 2 * i]);
            acc[g * 16 + 2 * i + 1] = fmaf(w, __uint_as_float(raw[i] & 0xFFFF0000u), acc[g * 16 + 2 * i + 1]);
        }
    };
    int slots[kMaxTopk];
    float ws[kMaxTopk];
#pragma unroll
    for (int j = 0; j < kMaxTopk; ++j) {
        slots[j] = j < topk ? __ldg(slot_of_flat + t * topk + j) : -1;
        ws[j] = j < topk ? __ldg(topk_w + t * topk + j) : 0.f;
    }
#pragma unroll
    for (int g = 0; g < kGroups; ++g) {
        uint32_t raw[kMaxTopk][8];
#pragma unroll
        for (int j = 0; j < kMaxTopk; ++j)
            if (slots[j] >= 0) ld_nc_256(dn + static_cast<size_t>(slots[j]) * h_bytes + col + 32 * g, raw[j]);
#pragma unroll
        for (int j = 0; j < kMaxTopk; ++j)
            if (slots[j] >= 0) fma_row(raw[j], ws[j], g);
    }
    if (bias != nullptr) {
        float const bs = bias_scale != nullptr ? __ldg(bias_scale + t) : 1.f;
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
            uint32_t raw[8];
            ld_nc_256(bias + static_cast<size_t>(t) * h_bytes + col + 32 * g, raw);
            fma_row(raw, bs, g);
        }
    }
    uint8_t* out_row = out + static_cast<size_t>(t) * h_bytes;
    if (sc.world > 0) {
        int s = 0;
        while (s + 1 < sc.world && t >= __ldg(sc.recv_off + s + 1)) ++s;
        out_row = reinterpret_cast<uint8_t*>(__ldg(sc.peer_back + s))
                  + static_cast<size_t>(__ldg(sc.back_base + s) + (t - __ldg(sc.recv_off + s))) * h_bytes;
    }
#pragma unroll
    for (int g = 0; g < kGroups; ++g) {
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = pack_bf16x2(acc[g * 16 + 2 * i], acc[g * 16 + 2 * i + 1]);
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"l"(out_row + col + 32 * g), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                     "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                     : "memory");
    }
}

// The combine for rows most of whose top-k slots are -1 (one expert-parallel rank: a received row has only the ids
// of the local experts). One CTA walks rows (in the permuted order of RowScatter); per row the first warp reads the
// top-k slots and weights once and compacts the live ones into shared memory (order kept), then every thread owns
// four 16-column pieces and adds the live rows in ascending j with the next row's loads in flight: the same sums, in the
// same order, as combine_wide_kernel, with one index read per row instead of one per thread.
// Needs 32-byte aligned dn and H % 64 == 0; output rows go where `sc` says (scatter mode only).
template <int kMaxTopk>
__global__ void __launch_bounds__(128, 3) combine_sparse_kernel(const uint8_t* __restrict__ dn,
    const int32_t* __restrict__ slot_of_flat, const float* __restrict__ topk_w, int64_t tokens, int topk, int h_bytes,
    RowScatter sc)
{
    constexpr int kGroups = 4;
    __shared__ int s_slot[2][kMaxTopk];
    __shared__ float s_w[2][kMaxTopk];
    __shared__ int s_live[2];
    int buf = 0;
    for (int64_t v = blockIdx.x; v < tokens; v += gridDim.x, buf ^= 1) {
        int64_t const t = static_cast<int64_t>(
            (static_cast<unsigned long long>(v) * sc.row_mul) % static_cast<unsigned long long>(tokens));
        if (threadIdx.x < 32) {
            int const j = threadIdx.x;
            int const s = j < topk ? __ldg(slot_of_flat + t * topk + j) : -1;
            float const w = j < topk ? __ldg(topk_w + t * topk + j) : 0.f;
            unsigned const livemask = __ballot_sync(0xffffffffu, s >= 0);
            if (s >= 0) {
                int const pos = __popc(livemask & ((1u << j) - 1u));
                s_slot[buf][pos] = s;
                s_w[buf][pos] = w;
            }
            if (j == 0) s_live[buf] = __popc(livemask);
        }
        __syncthreads();          // double-buffered: the next row's header goes to the other buffer
        int const live = s_live[buf];
        int s = 0;
        while (s + 1 < sc.world && t >= __ldg(sc.recv_off + s + 1)) ++s;
        uint8_t* const out_row = reinterpret_cast<uint8_t*>(__ldg(sc.peer_back + s))
                                 + static_cast<size_t>(__ldg(sc.back_base + s) + (t - __ldg(sc.recv_off + s))) * h_bytes;
        // Thread c owns, in pass p and group g, the 32 bytes at ((p * kGroups + g) * blockDim + c) * 32: every
        // warp-level load and store covers 1 KB of contiguous memory (stores to another GPU travel as full packets;
        // with 128 contiguous bytes per thread instead, each instruction scattered 32-byte pieces and the layer was
        // 0.5 ms slower on 8 GPUs).
        int const chunks = h_bytes / 32;
        for (int base = 0; base < chunks; base += kGroups * static_cast<int>(blockDim.x)) {
            int ch[kGroups];
#pragma unroll
            for (int g = 0; g < kGroups; ++g) ch[g] = base + g * static_cast<int>(blockDim.x) + static_cast<int>(threadIdx.x);
            float acc[16 * kGroups];
#pragma unroll
            for (int i = 0; i < 16 * kGroups; ++i) acc[i] = 0.f;
            uint32_t cur[kGroups][8], nxt[kGroups][8];
            if (live > 0) {
#pragma unroll
                for (int g = 0; g < kGroups; ++g)
                    if (ch[g] < chunks)
                        ld_nc_256(dn + static_cast<size_t>(s_slot[buf][0]) * h_bytes + static_cast<size_t>(ch[g]) * 32,
                            cur[g]);
            }
            for (int q = 0; q < live; ++q) {
                if (q + 1 < live) {
#pragma unroll
                    for (int g = 0; g < kGroups; ++g)
                        if (ch[g] < chunks)
                            ld_nc_256(dn + static_cast<size_t>(s_slot[buf][q + 1]) * h_bytes
                                    + static_cast<size_t>(ch[g]) * 32, nxt[g]);
                }
                float const w = s_w[buf][q];
#pragma unroll
                for (int g = 0; g < kGroups; ++g)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        acc[g * 16 + 2 * i] = fmaf(w, __uint_as_float(cur[g][i] << 16), acc[g * 16 + 2 * i]);
                        acc[g * 16 + 2 * i + 1]
                            = fmaf(w, __uint_as_float(cur[g][i] & 0xFFFF0000u), acc[g * 16 + 2 * i + 1]);
                    }
#pragma unroll
                for (int g = 0; g < kGroups; ++g)
#pragma unroll
                    for (int i = 0; i < 8; ++i) cur[g][i] = nxt[g][i];
            }
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
                if (ch[g] >= chunks) continue;
                uint32_t o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = pack_bf16x2(acc[g * 16 + 2 * i], acc[g * 16 + 2 * i + 1]);
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                             ::"l"(out_row + static_cast<size_t>(ch[g]) * 32), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]),
                             "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                             : "memory");
            }
        }
    }
}

}  // namespace fso
