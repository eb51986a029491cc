// Expert-parallel exchange over peer memory: kernels that store token rows straight into another GPU's receive
// buffers (plain st.global on peer-mapped addresses, NVLink through NVSwitch) and that unpack what arrived.
//
// Nothing here waits on another GPU. A kernel only writes peer memory; the ranks order their steps on the host side
// with a stream-ordered collective between the writing kernel and the first kernel that reads what was written.
// The reference has no communication code (docs/guide.md:139-141 leaves sharding to the caller), so these kernels
// serve this library's own expert_parallel_layer helper.
#pragma once

#include "common.cuh"
#include "quant.cuh"

namespace fso {

// One CTA per sent row i: token send_token[i] goes to rank send_rank[i], row dst_base[rank] + (i - send_off[rank])
// of that rank's receive buffers. What travels: the H e4m3 codes, the H/128 scale words of the row (taken out of
// the 128-row atom layout into row-major order), the top-k ids rewritten to the destination's local expert range
// (-1 for experts of other ranks) and the top-k weights.
__global__ void __launch_bounds__(128) ep_push_rows_kernel(const uint4* __restrict__ xq, const uint32_t* __restrict__ xs,
    const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_w, const int64_t* __restrict__ send_token,
    const int64_t* __restrict__ send_rank, const int64_t* __restrict__ send_off, const int64_t* __restrict__ dst_base,
    const uint64_t* __restrict__ peer_q, const uint64_t* __restrict__ peer_w, const uint64_t* __restrict__ peer_ids,
    const uint64_t* __restrict__ peer_wt, int topk, int kb, int experts_per_rank)
{
    int64_t const i = blockIdx.x;
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
    __threadfence_system();
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
