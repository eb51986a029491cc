// Expert-parallel exchange over peer memory: kernels that store token rows straight into another GPU's receive
// buffers (plain st.global on peer-mapped addresses, NVLink through NVSwitch) and that unpack what arrived.
//
// Nothing here waits on another GPU. A kernel only writes peer memory; the ranks order their steps on the host side
// with a stream-ordered collective between the writing kernel and the first kernel that reads what was written
// (a kernel's peer stores are complete when the kernel is, so the kernels issue no system-scope fence themselves).
// The reference has no communication code (docs/guide.md:139-141 leaves sharding to the caller), so these kernels
// serve this library's own expert_parallel_layer helper.
#pragma once

#include "common.cuh"
#include "quant.cuh"

namespace fso {

// Plan, step 1: bit r of rank_mask[t] = token t has at least one top-k id in rank r's expert range (ids outside
// [0, world * experts_per_rank) belong to nobody); row[r] += number of tokens bound for rank r (row is zeroed by the
// launcher, integer atomics: the result does not depend on the order), row[world] = tokens.
__global__ void __launch_bounds__(256) ep_plan_count_kernel(const int32_t* __restrict__ topk_ids, int64_t tokens,
    int topk, int experts_per_rank, int world, uint64_t* __restrict__ rank_mask, unsigned long long* __restrict__ row)
{
    __shared__ unsigned int cnt[64];
    if (threadIdx.x < 64) cnt[threadIdx.x] = 0;
    __syncthreads();
    int64_t const t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    uint64_t mask = 0;
    if (t < tokens) {
        for (int j = 0; j < topk; ++j) {
            int const id = __ldg(topk_ids + t * topk + j);
            if (id >= 0) {
                int const r = id / experts_per_rank;
                if (r < world) mask |= 1ull << r;
            }
        }
        rank_mask[t] = mask;
    }
    for (int r = 0; r < world; ++r) {
        unsigned const votes = __ballot_sync(0xffffffffu, (mask >> r) & 1ull);
        if ((threadIdx.x & 31) == 0 && votes != 0) atomicAdd(&cnt[r], __popc(votes));
    }
    __syncthreads();
    if (threadIdx.x < world && cnt[threadIdx.x] != 0) atomicAdd(row + threadIdx.x, cnt[threadIdx.x]);
    if (blockIdx.x == 0 && threadIdx.x == 0) row[world] = static_cast<unsigned long long>(tokens);
}

// Plan, step 2, one CTA per destination rank r, from the gathered table (table[s * (world + 1) + d] = rows rank s
// sends to rank d): the offsets every later kernel needs, this rank's send list for r (tokens ascending, at
// send_off[r]) and column r of the slot table of the final reduction (position of the token's row in the send
// order, which is where rank r's partial row comes back to; -1 = nothing from r).
__global__ void __launch_bounds__(1024) ep_plan_place_kernel(const uint64_t* __restrict__ rank_mask,
    const int64_t* __restrict__ table, int64_t tokens, int world, int rank, int64_t* __restrict__ send_token,
    int64_t* __restrict__ send_rank, int64_t* __restrict__ send_off, int64_t* __restrict__ dst_base,
    int64_t* __restrict__ recv_off, int64_t* __restrict__ back_base, int32_t* __restrict__ slot)
{
    __shared__ int64_t s_off;
    __shared__ int warp_sum[32];
    int const r = blockIdx.x;
    int const stride = world + 1;
    if (threadIdx.x == 0) {
        int64_t so = 0, db = 0, ro = 0, bb = 0;
        for (int d = 0; d < r; ++d) so += table[rank * stride + d];
        for (int s = 0; s < rank; ++s) db += table[s * stride + r];
        for (int s = 0; s <= r; ++s) ro += table[s * stride + rank];
        for (int d = 0; d < rank; ++d) bb += table[r * stride + d];
        send_off[r] = so;
        dst_base[r] = db;
        recv_off[r + 1] = ro;
        if (r == 0) recv_off[0] = 0;
        back_base[r] = bb;
        s_off = so;
    }
    int64_t const chunk = (tokens + blockDim.x - 1) / blockDim.x;
    int64_t const t0 = threadIdx.x * chunk;
    int64_t const t1 = t0 + chunk < tokens ? t0 + chunk : tokens;
    int mine = 0;
    for (int64_t t = t0; t < t1; ++t) mine += static_cast<int>((__ldg(rank_mask + t) >> r) & 1ull);
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int const v = __shfl_up_sync(0xffffffffu, incl, o);
        if ((threadIdx.x & 31) >= o) incl += v;
    }
    if ((threadIdx.x & 31) == 31) warp_sum[threadIdx.x >> 5] = incl;
    __syncthreads();
    if (threadIdx.x < 32) {
        int const w = threadIdx.x < (blockDim.x >> 5) ? warp_sum[threadIdx.x] : 0;
        int acc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int const v = __shfl_up_sync(0xffffffffu, acc, o);
            if (threadIdx.x >= o) acc += v;
        }
        warp_sum[threadIdx.x] = acc - w;
    }
    __syncthreads();
    int64_t pos = s_off + warp_sum[threadIdx.x >> 5] + incl - mine;
    for (int64_t t = t0; t < t1; ++t) {
        bool const on = (__ldg(rank_mask + t) >> r) & 1ull;
        slot[t * world + r] = on ? static_cast<int32_t>(pos) : -1;
        if (on) {
            send_token[pos] = t;
            send_rank[pos] = r;
            ++pos;
        }
    }
}

// One CTA per sent row i: token send_token[i] goes to rank send_rank[i], row dst_base[rank] + (i - send_off[rank])
// of that rank's receive buffers. What travels: the H e4m3 codes, the H/128 scale words of the row (taken out of
// the 128-row atom layout into row-major order), the top-k ids rewritten to the destination's local expert range
// (-1 for experts of other ranks) and the top-k weights.
__global__ void __launch_bounds__(128) ep_push_rows_kernel(const uint4* __restrict__ xq, const uint32_t* __restrict__ xs,
    const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_w, const int64_t* __restrict__ send_token,
    const int64_t* __restrict__ send_rank, const int64_t* __restrict__ send_off, const int64_t* __restrict__ dst_base,
    const uint64_t* __restrict__ peer_q, const uint64_t* __restrict__ peer_w, const uint64_t* __restrict__ peer_ids,
    const uint64_t* __restrict__ peer_wt, int topk, int kb, int experts_per_rank, int64_t rows, int64_t row_mul)
{
    // CTA b takes row (b * row_mul) mod rows, row_mul coprime to rows: the rows in flight at any moment are spread
    // over all destinations, instead of every rank storing into the same GPU at the same time
    int64_t const i = static_cast<int64_t>((static_cast<unsigned long long>(blockIdx.x) * row_mul) % rows);
    int64_t const tok = __ldg(send_token + i);
    int const rk = static_cast<int>(__ldg(send_rank + i));
    int64_t const row = __ldg(dst_base + rk) + (i - __ldg(send_off + rk));
    int const h16 = kb * 8;
    uint4* const dq = reinterpret_cast<uint4*>(__ldg(peer_q + rk)) + row * h16;
    const uint4* const sq = xq + tok * h16;
    for (int c = threadIdx.x; c < h16; c += blockDim.x) dq[c] = __ldg(sq + c);
    uint32_t* const dw = reinterpret_cast<uint32_t*>(__ldg(peer_w + rk)) + row * kb;
    for (int kp = threadIdx.x; kp < kb; kp += blockDim.x) dw[kp] = __ldg(xs + sf_word_index(tok, kp, kb));
    if (threadIdx.x < topk) {
        int const id = __ldg(topk_ids + tok * topk + threadIdx.x);
        int const lo = rk * experts_per_rank;
        reinterpret_cast<int32_t*>(__ldg(peer_ids + rk))[row * topk + threadIdx.x]
            = (id >= lo && id < lo + experts_per_rank) ? id - lo : -1;
        reinterpret_cast<float*>(__ldg(peer_wt + rk))[row * topk + threadIdx.x] = __ldg(topk_w + tok * topk + threadIdx.x);
    }
}

// Received rows (codes row-major, scale words row-major) -> the compact slot order the grouped GEMM reads: codes to
// every slot of the row, scale words into the 128-row atom layout. One thread per 16 codes.
__global__ void __launch_bounds__(256) gather_rows_q_kernel(const uint4* rx_q, const uint32_t* rx_w,
    const int32_t* __restrict__ slot_of_flat, int64_t rows, int topk, int kb, uint4* __restrict__ hq,
    uint32_t* __restrict__ sh)
{
    uint32_t const idx = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t const h16 = static_cast<uint32_t>(kb) * 8;
    if (idx >= static_cast<uint32_t>(rows) * h16) return;
    uint32_t const r = idx / h16;
    uint32_t const c = idx - r * h16;
    uint4 const v = rx_q[idx];
    bool const lead = (c & 7u) == 0;
    int const kp = static_cast<int>(c >> 3);
    uint32_t const word = lead ? rx_w[static_cast<size_t>(r) * kb + kp] : 0u;
    for (int j = 0; j < topk; ++j) {
        int const slot = __ldg(slot_of_flat + static_cast<size_t>(r) * topk + j);
        if (slot >= 0) {
            hq[static_cast<int64_t>(slot) * h16 + c] = v;
            if (lead) sh[sf_word_index(slot, kp, kb)] = word;
        }
    }
}

}  // namespace fso
