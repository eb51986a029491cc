// Router top-k: logits [M, E] -> top-k expert ids (descending weight, ties to the lower id), softmax weights
// (renormalized over the selected k or over all experts), padded-row sentinel, expert-parallel id map, shared
// expert's sigmoid gate. One warp per token, experts strided over the lanes (expert e lives in lane e % 32).
//
// The selection works on order-preserving 32-bit keys of the fp32 logits: per pick every lane offers its best
// remaining key, one warp max-reduction (redux.sync) finds the winning value and one min-reduction over the ids of
// the lanes that hold it finds the lowest expert id with that value.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace fso {

constexpr int kRouterMaxTopk = 8;
constexpr int kRouterMaxExperts = 1024;

__device__ __forceinline__ float logit_to_float(float v) { return v; }
__device__ __forceinline__ float logit_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float logit_to_float(__half v) { return __half2float(v); }

// fp32 -> uint32 whose unsigned order is the float order (-inf lowest, +inf highest); 0 is below every float.
__device__ __forceinline__ uint32_t order_key(float v)
{
    uint32_t const b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float key_value(uint32_t k)
{
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

template <typename TLogit, int kSlots>
__global__ void __launch_bounds__(256) router_topk_kernel(const TLogit* __restrict__ logits, int64_t ld, int m, int e,
    int topk, int renormalize, const int32_t* __restrict__ n_valid, const int32_t* __restrict__ expert_map,
    int32_t* __restrict__ out_ids, float* __restrict__ out_w, float* __restrict__ shared_gate)
{
    int const lane = threadIdx.x & 31;
    int const token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= m) return;
    const TLogit* const row = logits + static_cast<int64_t>(token) * ld;
    // the shared expert's gate logit is column E; padded rows get a value too (their shared output is zero anyway)
    if (shared_gate != nullptr && lane == 0) shared_gate[token] = 1.f / (1.f + expf(-logit_to_float(row[e])));
    if (n_valid != nullptr && token >= __ldg(n_valid)) {
        // padded row of a graph bucket: the sentinel id (num_experts, through the map when there is one), weight 0
        if (lane < topk) {
            out_ids[static_cast<int64_t>(token) * topk + lane] = expert_map != nullptr ? __ldg(expert_map + e) : e;
            out_w[static_cast<int64_t>(token) * topk + lane] = 0.f;
        }
        return;
    }
    uint32_t key[kSlots];
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
        int const x = lane + 32 * s;
        key[s] = x < e ? order_key(logit_to_float(row[x])) : 0u;
    }
    // softmax denominator over all experts (only without renormalization): max, then sum of exp in a fixed order
    float full_denom = 0.f;
    if (!renormalize) {
        uint32_t kmax = 0;
#pragma unroll
        for (int s = 0; s < kSlots; ++s) kmax = max(kmax, key[s]);
        kmax = __reduce_max_sync(0xffffffffu, kmax);
        float const top = key_value(kmax);
        float part = 0.f;
#pragma unroll
        for (int s = 0; s < kSlots; ++s)
            if (lane + 32 * s < e) part += expf(key_value(key[s]) - top);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        full_denom = part;
    }
    // k picks. Lane j keeps pick j.
    float my_v = 0.f;
    int my_id = 0;
    float first_v = 0.f;
    for (int j = 0; j < topk; ++j) {
        uint32_t best = 0;
        int best_s = 0;
#pragma unroll
        for (int s = 0; s < kSlots; ++s)
            if (key[s] > best) {            // strictly greater, ascending s: the lower id wins inside a lane
                best = key[s];
                best_s = s;
            }
        uint32_t const win = __reduce_max_sync(0xffffffffu, best);
        uint32_t const cand = best == win ? static_cast<uint32_t>(lane + 32 * best_s) : 0xFFFFFFFFu;
        int const id = static_cast<int>(__reduce_min_sync(0xffffffffu, cand));
        float const v = key_value(win);
        if (j == 0) first_v = v;
        if (lane == j) {
            my_v = v;
            my_id = id;
        }
        if ((id & 31) == lane) {
#pragma unroll
            for (int s = 0; s < kSlots; ++s)
                if (s == (id >> 5)) key[s] = 0u;
        }
    }
    // weights: exp(l - max) over the selected, summed in pick order (the order torch sums its top-k output)
    float const ex = lane < topk ? expf(my_v - first_v) : 0.f;
    float denom = 0.f;
    for (int j = 0; j < topk; ++j) denom += __shfl_sync(0xffffffffu, ex, j);
    if (!renormalize) denom = full_denom;
    if (lane < topk) {
        out_ids[static_cast<int64_t>(token) * topk + lane] = expert_map != nullptr ? __ldg(expert_map + my_id) : my_id;
        out_w[static_cast<int64_t>(token) * topk + lane] = ex * (1.f / denom);
    }
}

template <typename TLogit>
inline int launch_router_topk(const void* logits, int64_t ld, int64_t m, int64_t e, int64_t topk, bool renormalize,
    const int32_t* n_valid, const int32_t* expert_map, int32_t* ids, float* w, float* gate, cudaStream_t stream)
{
    unsigned const blocks = static_cast<unsigned>((m + 7) / 8);
    auto* l = static_cast<const TLogit*>(logits);
#define FSO_ROUTER_CASE(SLOTS)                                                                                     \
    if (e <= 32 * SLOTS) {                                                                                         \
        router_topk_kernel<TLogit, SLOTS><<<blocks, 256, 0, stream>>>(l, ld, static_cast<int>(m),                  \
            static_cast<int>(e), static_cast<int>(topk), renormalize ? 1 : 0, n_valid, expert_map, ids, w, gate);  \
    } else
    FSO_ROUTER_CASE(1)
    FSO_ROUTER_CASE(2)
    FSO_ROUTER_CASE(4)
    FSO_ROUTER_CASE(8)
    FSO_ROUTER_CASE(16)
    FSO_ROUTER_CASE(32)
    {
        set_error("fso_moe_topk_from_logits: num_experts = %lld is beyond %d", static_cast<long long>(e),
            kRouterMaxExperts);
        return FSO_ERR_INVALID;
    }
#undef FSO_ROUTER_CASE
    return launch_status("router_topk_kernel");
}

}  // namespace fso
