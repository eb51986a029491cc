// The large-M dense GEMM on CTA pairs: one 256 x 256 x 32 tcgen05.mma (cta_group::2) per instruction across a
// cluster of two CTAs. Each CTA stages its own 128 rows of A and HALF of the 256 weight rows per K block (the
// tensor cores read the other half from the peer's shared memory), which cuts the operand bytes that travel
// L2 -> SM per flop by a third against the single-CTA kernel (32 KB instead of 48 KB per SM and K block) and leaves
// room for six pipeline stages. Each CTA keeps its 128 x 256 fp32 accumulators in its own tensor memory and runs its
// own epilogue.
//
// Protocol (rank 0 of the pair is the leader):
//   * TMA producers of BOTH CTAs load into their own shared memory and count completion bytes on the LEADER's
//     "full" mbarrier of the stage (cta_group::2 form of the tiled load); scale factors go through tiled loads too
//     (the atom layout seen as rows of 128 32-bit words) so that they can signal the leader as well. Every CTA loads
//     its own A scale block and BOTH weight scale blocks (each CTA's tensor memory needs all 256 columns' scales).
//   * the leader's MMA thread waits on "full", issues the scale copies and the four MMAs of the K block for the pair,
//     and commits with one instruction to the "empty" mbarrier of the stage in both CTAs and, per tile, to each
//     CTA's "accumulator full".
//   * two accumulators per CTA that share 32 tensor-memory columns (see GemmCfg::kOverlapAcc): the epilogue warps of
//     both CTAs drain the shared columns first and arrive on the leader's barrier for them, drain the rest into
//     packed bf16 registers, arrive on the leader's "accumulator empty" and then store.
// No load in this kernel is a cluster broadcast: every byte a CTA needs in its own shared memory it loads itself.
#pragma once

#include "gemm.cuh"

namespace fso {


struct Gemm2Cfg {
    static constexpr int kBM = 128;          // accumulator rows per CTA (256 per pair)
    static constexpr int kBN = 256;
    static constexpr int kStages = 6;
    static constexpr int kEpiWarps = 8;
    static constexpr int kThreads = 128 + 32 * kEpiWarps;
    static constexpr int kABytes = 128 * 128;
    static constexpr int kBBytes = 128 * 128;    // this CTA's half of the 256 weight rows
    static constexpr int kSfaBytes = 512;
    static constexpr int kSfbBytes = 1024;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 512;
    static constexpr int kAccStride = 224;       // accumulator 1 starts inside the last 32 columns of accumulator 0
    static constexpr int kSfCol0 = kAccStride + kBN;
    static constexpr int kSfBufCols = 12;
    static constexpr int kTmemCols = 512;
    static_assert(kSfCol0 + 2 * kSfBufCols <= kTmemCols, "tensor memory budget");
    static_assert(kSmemBytes <= 227 * 1024 && kSmemBytes > 116 * 1024, "one CTA per SM");
};

__host__ __device__ constexpr uint32_t make_idesc_mxf8_pair(uint32_t n)
{
    return (1u << 23) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}

// One thread of the leader CTA: one arrival on the mbarrier at this shared-memory offset in each CTA of the pair,
// once every tcgen05 operation this thread issued before has completed in both CTAs.
__device__ __forceinline__ void tc_commit_pair_both(uint32_t bar)
{
    uint16_t const mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(mask)
        : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Gemm2Cfg::kThreads, 1)
gemm_mxf8_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
    const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb, const GemmParams p)
{
    using C = Gemm2Cfg;
    constexpr int S = C::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint32_t const raw = smem_u32(smem_raw);
    uint32_t const base = (raw + 1023u) & ~1023u;
    uint8_t* const gbase = smem_raw + (base - raw);

    uint32_t const sA = base;
    uint32_t const sB = sA + S * C::kABytes;
    uint32_t const sSfa = sB + S * C::kBBytes;
    uint32_t const sSfb = sSfa + S * C::kSfaBytes;
    uint32_t const bars = sSfb + S * C::kSfbBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * S + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * S + 2 + a); };
    uint32_t const ovl_bar = bars + 8u * (2 * S + 4);
    uint32_t const misc_off = static_cast<uint32_t>(S) * C::kStageBytes + 8u * (2 * S + 5);
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(gbase + misc_off);
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(gbase + misc_off + 4);

    // broadcast from lane 0: the compiler then knows the warp index (and every branch on it) to be warp-uniform
    int const warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    int const lane = threadIdx.x & 31;
    // read per thread: the broadcast form (as for the warp index above) measured 12 % slower on this kernel
    uint32_t const rank = cluster_ctarank();
    bool const leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 2 * C::kEpiWarps);      // the epilogue warps of both CTAs
        }
        mbar_init(ovl_bar, 2 * 4);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        prefetch_tensormap(&tm_sfa);
        prefetch_tensormap(&tm_sfb);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_slot), C::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    uint32_t const tmem_base = *tmem_slot;

    int const pair = blockIdx.x >> 1;
    int const num_pairs = gridDim.x >> 1;
    int const tiles_total = p.tiles_a * p.tiles_b;     // tiles_a counts 256-row tiles here

    auto decode = [&](int t, int& tile_m, int& tile_n) {
        int const group_span = p.group_a * p.tiles_b;
        int const g = t / group_span;
        int const first = g * p.group_a;
        int const gsz = min(p.group_a, p.tiles_a - first);
        int const in_g = t - g * group_span;
        tile_n = in_g / gsz;
        tile_m = first + (in_g - tile_n * gsz);
    };

    if (warp == 0) {
        // ------------------------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            constexpr uint32_t kPairBytes = 2u * C::kStageBytes;
            for (int t = pair; ok && t < tiles_total; t += num_pairs) {
                int tile_m, tile_n;
                decode(t, tile_m, tile_n);
                int const a_row0 = tile_m * 256 + static_cast<int>(rank) * 128;
                int const b_row0 = tile_n * 256 + static_cast<int>(rank) * 128;
                for (int kb = 0; kb < p.kb_total; ++kb) {
                    if (!wait_or_abort(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        record_abort(FSO_DEV_WAIT_PRODUCER, abort_flag);
                        ok = false;
                        break;
                    }
                    uint32_t const fb = map_to_cta(full_bar(stage), 0);
                    if (leader) mbar_expect_tx(full_bar(stage), kPairBytes);
                    tma_load_2d_pair(sA + stage * C::kABytes, &tm_a, fb, kb * 128, a_row0);
                    tma_load_2d_pair(sB + stage * C::kBBytes, &tm_b, fb, kb * 128, b_row0);
                    tma_load_2d_pair(sSfa + stage * C::kSfaBytes, &tm_sfa, fb, 0, (a_row0 >> 7) * p.kb_total + kb);
                    tma_load_2d_pair(sSfb + stage * C::kSfbBytes, &tm_sfb, fb, 0, (tile_n * 2) * p.kb_total + kb);
                    tma_load_2d_pair(sSfb + stage * C::kSfbBytes + 512, &tm_sfb, fb, 0,
                        (tile_n * 2 + 1) * p.kb_total + kb);
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer (leader only)
        if (leader && elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            int sfbuf = 0;
            int tiles_done = 0;
            constexpr uint32_t idesc = make_idesc_mxf8_pair(C::kBN);
            bool ok = true;
            for (int t = pair; ok && t < tiles_total; t += num_pairs) {
                // the tile two before this one used the same accumulator: all of it must have been drained
                if (!wait_or_abort(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
                    record_abort(FSO_DEV_WAIT_MMA_TMEM, abort_flag);
                    break;
                }
                uint32_t const d_tmem = tmem_base + static_cast<uint32_t>(acc * C::kAccStride);
                for (int kb = 0; kb < p.kb_total; ++kb) {
                    if (!wait_or_abort(full_bar(stage), phase, abort_flag)) {
                        record_abort(FSO_DEV_WAIT_MMA_FULL, abort_flag);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    uint32_t const sf_col = tmem_base + C::kSfCol0 + sfbuf * C::kSfBufCols;
                    tc_cp_32x128b_warpx4_pair(sf_col, make_desc_sf(sSfa + stage * C::kSfaBytes));
                    tc_cp_32x128b_warpx4_pair(sf_col + 4, make_desc_sf(sSfb + stage * C::kSfbBytes));
                    tc_cp_32x128b_warpx4_pair(sf_col + 8, make_desc_sf(sSfb + stage * C::kSfbBytes + 512));
                    if (kb == 0) {
                        // the tile before this one sits in the other accumulator: the columns both use must have
                        // left before the first MMA writes them (the operands and the scale copies did not wait)
                        if (tiles_done > 0
                            && !wait_or_abort(ovl_bar, static_cast<uint32_t>(tiles_done - 1) & 1u, abort_flag)) {
                            record_abort(FSO_DEV_WAIT_MMA_TMEM, abort_flag);
                            ok = false;
                            break;
                        }
                        ++tiles_done;
                        tc_fence_after();
                    }
                    uint64_t const adesc = make_desc_sw128(sA + stage * C::kABytes);
                    uint64_t const bdesc = make_desc_sw128(sB + stage * C::kBBytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma_mxf8_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc | sf_id_bits(k), sf_col,
                            sf_col + 4, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair_both(empty_bar(stage));
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    sfbuf ^= 1;
                }
                if (!ok) break;
                tc_commit_pair_both(tfull_bar(acc));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------------------------------ epilogue (both CTAs)
        int const quarter = warp & 3;
        int const half = (warp - 4) >> 2;
        constexpr int kColsPerWarp = C::kBN / 2;
        constexpr int kChunks = kColsPerWarp / 32;
        int acc = 0;
        uint32_t acc_phase = 0;
        uint32_t const leader_ovl = map_to_cta(ovl_bar, 0);
        for (int t = pair; t < tiles_total; t += num_pairs) {
            int tile_m, tile_n;
            decode(t, tile_m, tile_n);
            if (!wait_or_abort(tfull_bar(acc), acc_phase, abort_flag)) {
                if (lane == 0) record_abort(FSO_DEV_WAIT_EPILOGUE, abort_flag);
                break;
            }
            tc_fence_after();
            // the shared columns are the last 32 of accumulator 0 and the first 32 of accumulator 1: chunks are walked
            // from the end in accumulator 0 and from the start in accumulator 1, the owners of the shared columns
            // report them drained after their first chunk
            bool const rev = acc == 0;
            bool const ovl_owner = half == (acc == 0 ? 1 : 0);
            auto chunk_col = [&](int j) { return 32 * (rev ? kChunks - 1 - j : j); };
            uint32_t const t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16)
                + static_cast<uint32_t>(acc * C::kAccStride + half * kColsPerWarp);
            int const a_row = tile_m * 256 + static_cast<int>(rank) * 128 + quarter * 32 + lane;
            int const col0 = tile_n * C::kBN + half * kColsPerWarp;
            uint32_t packed[kChunks * 16];
            uint32_t ra[32], rb[32];
            tmem_ld_32x32(t_row + static_cast<uint32_t>(chunk_col(0)), ra);
            tmem_ld_wait();
            if (ovl_owner) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leader_ovl);
            }
#pragma unroll
            for (int j = 0; j < kChunks; j += 2) {
                tmem_ld_32x32(t_row + static_cast<uint32_t>(chunk_col(j + 1)), rb);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    packed[16 * j + i] = pack_bf16x2(__uint_as_float(ra[2 * i]), __uint_as_float(ra[2 * i + 1]));
                tmem_ld_wait();
                if (j + 2 < kChunks) tmem_ld_32x32(t_row + static_cast<uint32_t>(chunk_col(j + 2)), ra);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    packed[16 * (j + 1) + i] = pack_bf16x2(__uint_as_float(rb[2 * i]), __uint_as_float(rb[2 * i + 1]));
                if (j + 2 < kChunks) tmem_ld_wait();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
            if (a_row < p.rows_a) {
                __nv_bfloat16* const orow = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(a_row) * p.ldo + col0;
#pragma unroll
                for (int g = 0; g < 2 * kChunks; ++g) {
                    int const c0 = chunk_col(g >> 1) + 16 * (g & 1);
                    uint32_t const* v = &packed[8 * g];
                    if (p.out_align32) {
                        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                     ::"l"(orow + c0), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]),
                                     "r"(v[6]), "r"(v[7])
                                     : "memory");
                    } else {
                        uint4* dst = reinterpret_cast<uint4*>(orow + c0);
                        dst[0] = make_uint4(v[0], v[1], v[2], v[3]);
                        dst[1] = make_uint4(v[4], v[5], v[6], v[7]);
                    }
                }
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        __syncwarp();
    }

    // ---------------------------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();      // neither CTA leaves (or frees tensor memory) while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::kTmemCols);
    }
}

}  // namespace fso
