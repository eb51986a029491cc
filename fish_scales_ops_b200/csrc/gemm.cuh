// MXFP8 block-scaled GEMM for sm_100a: tcgen05.mma kind::mxf8f6f4.block_scale, operands fed by TMA into a
// multi-stage shared-memory ring, UE8M0 scale factors copied shared -> tensor memory per K block, fp32
// accumulators in tensor memory, persistent CTAs (one per SM) with a static tile schedule.
//
// One kernel template serves four uses:
//   * dense, normal orientation   activation rows on MMA-M (128), weight rows on MMA-N (128 / 256)
//   * dense, swapped orientation  weight rows on MMA-M (128), the (<= 64) activation rows on MMA-N (16 / 32 / 64):
//                                 the weight stream is what the decode-sized problem costs
//   * split-K of either           fp32 partials to a workspace, summed in slice order by a second kernel
//   * grouped (MoE)               A rows are the 128-row blocks of the compact activation, the weight of each block
//                                 is picked through the block -> expert table; optional fused SiLU(gate)*up
//                                 requantize epilogue (FC1) that writes e4m3 + scale words directly
//
// Warp roles: warp 0 = TMA producer (one lane), warp 1 = tensor-memory owner and MMA issuer (one lane),
// warps 4.. = epilogue (warp w reads the 32-lane quarter w % 4 of the accumulator).
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"
#include "quant.cuh"

namespace fso {

// EPI_CLUSTER (swapped orientation only): split-K inside a thread-block cluster. The CTAs of a cluster take the K
// slices of one tile; slices 1.. store their fp32 accumulators into CTA 0's shared memory (distributed shared memory),
// CTA 0 adds them in slice order and writes bf16: the same sums as EPI_PARTIAL + splitk_reduce_kernel, in one launch
// and without a workspace.
// EPI_QUANT (normal orientation): the output leaves in the activation contract instead of bf16: per row and 32
// output columns act(acc + bias) is rounded to bf16 (so that the bytes equal quantizing the bf16 output afterwards),
// then amax -> UE8M0 byte -> e4m3 codes; `out` is e4m3 [M, N], `out_sf` its scale words.
enum : int { EPI_BF16 = 0, EPI_PARTIAL = 1, EPI_SWIGLU = 2, EPI_CLUSTER = 3, EPI_QUANT = 4 };

struct GemmParams {
    const uint8_t* sfa;        // scale words of the operand on MMA-M
    const uint8_t* sfb;        // scale words of the operand on MMA-N
    void* out;                 // bf16 [M, N]; EPI_SWIGLU: e4m3 [rows, I]; EPI_QUANT: e4m3 [M, N]
    uint32_t* out_sf;          // EPI_SWIGLU / EPI_QUANT: scale words of the e4m3 output
    float* ws;                 // EPI_PARTIAL: fp32 [splits, M, N]
    const int32_t* blk0;       // grouped: blk0[num_experts] = blocks in use
    const int32_t* blk_expert; // grouped: expert of each 128-row block
    const int32_t* masked_m;   // grouped + swapped: routed rows of each expert
    int subs;                  // grouped + swapped: token sub-tiles per 128-row block (128 / BN, fewer for a handful of pairs)
    int out_f32;               // grouped + swapped: `out` is fp32 [rows, ldo] (the accumulators, not rounded)
    int rows_a;                // valid rows of the MMA-M operand
    int rows_b;                // valid rows of the MMA-N operand (per expert when grouped)
    int kb_total;              // K / 128
    int kb_per_split;
    int splits;
    int tiles_a;               // 128-row tiles of the MMA-M operand (grouped: bound on the blocks)
    int tiles_b;               // BN-row tiles of the MMA-N operand
    int ldo;                   // leading dimension of out / ws rows, in elements
    int num_experts;
    int group_a;               // raster: tiles of A walked together before B advances
    int out_align32;           // the output base is 32-byte aligned (256-bit stores are usable)
    int stream_b_hint;         // grouped: the weight tiles of an expert with a single block are loaded evict-first
    int64_t out_rows;          // rows of the output (row stride of one split's partial = out_rows * ldo)
    // dense epilogue (kFused kernels and the split-K reduce): out = bf16(act(acc + bias[n]) + residual[m, n])
    const __nv_bfloat16* bias;      // [N] or nullptr
    const __nv_bfloat16* residual;  // [M, N] or nullptr
    int act;                        // 0 = identity, 1 = erf-GELU
};

// The bias as the epilogue adds it: +0.0 becomes -0.0, so that a zero bias changes no accumulator value (not even
// the sign of a zero) and bias = 0 gives the bytes of bias = None.
__device__ __forceinline__ float bias_term(__nv_bfloat16 b)
{
    uint32_t const bits = static_cast<uint32_t>(__bfloat16_as_ushort(b)) << 16;
    return __uint_as_float(bits == 0u ? 0x80000000u : bits);
}

// act(acc + bias) in fp32; erf-GELU as 0.5 v (1 + erf(v / sqrt 2)) with the constant rounded to fp32 first.
__device__ __forceinline__ float epilogue_value(float acc, float bias_f, bool has_bias, int act)
{
    float v = has_bias ? acc + bias_f : acc;
    if (act == 1) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));
    return v;
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

template <int BN, int EPI = 0>
struct GemmCfg {
    static constexpr int kBM = 128;
    static constexpr int kBK = 128;                                   // bytes == elements along K per stage
    // epilogue warps: 4 quarters x {1, 2, 4} column slices. The SwiGLU epilogue takes 64-column slices so that a
    // slice fits in registers and the accumulator can be handed back before the activation math starts.
    static constexpr int kEpiWarps = EPI == 2 /* EPI_SWIGLU */ ? 16 : BN >= 128 ? 8 : 4;
    static constexpr int kThreads = 128 + 32 * kEpiWarps;
    // Two accumulators, drained by the epilogue while the next tile's MMAs fill the other one. 2 x 256 columns plus
    // the scale-factor buffers do not fit in the 512 columns of tensor memory, so at BN = 256 the two accumulators
    // share 32 columns: accumulator 0 is columns [0, 256), accumulator 1 is [224, 480). The epilogue of a tile
    // drains the shared columns first and signals a barrier of their own; the MMAs of the next tile wait for that
    // barrier only (and for the complete drain of the tile before, which used the same accumulator).
    static constexpr bool kOverlapAcc = BN == 256;
    static constexpr int kAccStages = 2;
    static constexpr int kAccStride = kOverlapAcc ? 224 : BN;
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBBytes = BN * kBK;
    static constexpr int kSfaBytes = 512;
    static constexpr int kSfbAtoms = BN > 128 ? BN / 128 : 1;
    static constexpr int kSfbBytes = 512 * kSfbAtoms;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    // Token tiles of 64 and fewer (the swapped, decode-sized kernels) take half an SM's shared memory, so that two
    // CTAs share an SM: every tile of a 1.5-wave problem is resident at once, and under programmatic dependent launch
    // the next kernel's CTAs load weights beside the last CTAs of this one.
    static constexpr bool kTwoPerSm = BN <= 64;
    static constexpr int kSmemBudget = (kTwoPerSm ? 113 : 227) * 1024 - 1024 /*alignment slack*/ - 512 /*barriers*/;
    static constexpr int kStagesMax = kSmemBudget / kStageBytes;
    static constexpr int kStages = kStagesMax > 12 ? 12 : kStagesMax;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 512;
    // EPI_CLUSTER: the other slices' accumulators, [slice - 1][BN columns][128 rows] fp32, land in CTA 0's stage
    // buffers once its own main loop is over
    static constexpr int kRedSlices = (kStages * kStageBytes) / (BN * 512);
    // tensor-memory columns: accumulators first, then two alternating scale-factor buffers
    static constexpr int kAccCols = kAccStride * (kAccStages - 1) + BN;
    static constexpr int kSfaCols = 4;
    static constexpr int kSfbCols = 4 * kSfbAtoms;
    static constexpr int kSfBufCols = kSfaCols + kSfbCols;
    static constexpr int kColsUsed = kAccCols + 2 * kSfBufCols;
    static constexpr int kTmemCols = kColsUsed <= 32 ? 32 : kColsUsed <= 64 ? 64 : kColsUsed <= 128 ? 128
        : kColsUsed <= 256 ? 256 : 512;
    static_assert(kColsUsed <= 512, "tensor memory budget");
    static_assert(kStages >= 3, "pipeline depth");
    static_assert(kSmemBytes > 116 * 1024 || kTmemCols <= 256, "CTAs that share an SM must share its 512 columns");
};

struct TileCoord {
    int a_tile;     // 128-row tile of the MMA-M operand (grouped: block index; grouped + swapped: weight panel)
    int b_tile;     // BN-row tile of the MMA-N operand (grouped + swapped: block index)
    int split;
    int expert;     // grouped: expert of the block; otherwise 0
    int sub;        // grouped + swapped: token sub-tile of the block
    int live;       // grouped + swapped: routed rows in this sub-tile (<= 0: nothing to do)
};

// Static schedule: work item t of (tiles_a_used * tiles_b * splits). A tiles advance fastest inside a group of
// `group_a`, then B tiles, then the next group; the split index is the slowest inside a tile pair.
// With kClusterK the split index is the fastest (the CTAs of one cluster share a tile).
template <bool kGrouped, bool kClusterK = false>
__device__ __forceinline__ bool decode_tile(GemmParams const& p, int t, int tiles_a_used, TileCoord& c)
{
    int const per_split = tiles_a_used * p.tiles_b;
    if (t >= per_split * p.splits) return false;
    c.split = kClusterK ? t % p.splits : t / per_split;
    int const r = kClusterK ? t / p.splits : t - c.split * per_split;
    int const group_span = p.group_a * p.tiles_b;
    int const g = r / group_span;
    int const first_a = g * p.group_a;
    int const gsz = min(p.group_a, tiles_a_used - first_a);
    int const in_g = r - g * group_span;
    c.b_tile = in_g / gsz;
    c.a_tile = first_a + (in_g - c.b_tile * gsz);
    c.expert = 0;
    if constexpr (kGrouped) c.expert = p.blk_expert[c.a_tile];
    return true;
}

// Grouped + swapped (the decode band of the MoE layer): weight rows of one expert on MMA-M, the (few) routed rows of
// one 128-row block on MMA-N. Work item t of (blocks in use x weight panels x sub-tiles x splits), weight panels
// fastest so that neighbouring CTAs stream neighbouring weight rows. A sub-tile past the block's routed rows is
// returned with live <= 0 and skipped by every role.
template <int BN, bool kClusterK>
__device__ __forceinline__ bool decode_tile_gs(GemmParams const& p, int t, int blocks_used, TileCoord& c)
{
    int const panels = p.tiles_a;
    int const items = blocks_used * panels * p.subs;
    if (t >= items * p.splits) return false;
    c.split = kClusterK ? t % p.splits : t / items;
    int const r = kClusterK ? t / p.splits : t - c.split * items;
    c.a_tile = r % panels;
    int const q = r / panels;
    c.sub = q % p.subs;
    c.b_tile = q / p.subs;
    c.expert = p.blk_expert[c.b_tile];
    int const in_block = min(128, p.masked_m[c.expert] - 128 * (c.b_tile - p.blk0[c.expert]));
    c.live = min(BN, in_block - c.sub * BN);
    return true;
}

__device__ __forceinline__ void record_abort(int code, volatile int* abort_flag)
{
    atomicCAS(&g_dev_status, 0, code);
    *abort_flag = 1;
}

// Bounded wait that also leaves when another role of this CTA has already given up.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    if (mbar_try_wait(bar, parity)) return true;
    long long const t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) return false;
    }
}

__device__ __forceinline__ float silu_mul(float g, float u)
{
    // silu(g) = g * sigmoid(g) = 0.5 * g * (1 + tanh(0.5 * g)), with the hardware tanh approximation
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * g));
    return (0.5f * g) * (1.f + t) * u;
}

// kFused: the bf16-writing epilogues also apply bias / activation / residual (separate instantiations, so that a call
// without them runs the code it always ran).
template <int BN, int EPI, bool kSwap, bool kGrouped, bool kFused = false>
__global__ void __launch_bounds__(GemmCfg<BN, EPI>::kThreads, 1)
gemm_mxf8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
    const GemmParams p)
{
    using C = GemmCfg<BN, EPI>;
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
    uint32_t const ovl_bar = bars + 8u * (2 * S + 4);      // the columns both accumulators use have been drained
    uint32_t const misc_off = static_cast<uint32_t>(S) * C::kStageBytes + 8u * (2 * S + 5);
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(gbase + misc_off);
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(gbase + misc_off + 4);
    constexpr uint32_t red_off = 0;       // EPI_CLUSTER: the other slices' accumulators reuse the stage buffers
    static_assert(EPI != EPI_CLUSTER || kSwap, "cluster split-K serves the swapped orientation");
    // EPI_CLUSTER: this thread's accumulator row (epilogue warps), kept in registers across the cluster barrier
    float red_v[EPI == EPI_CLUSTER ? BN : 1];
    bool red_have = false;
    TileCoord red_c{};

    // broadcast from lane 0: the compiler then knows the warp index (and every branch on it) to be warp-uniform
    int const warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    int const lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), C::kEpiWarps);
        }
        mbar_init(ovl_bar, 4);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        if constexpr (kSwap && !kGrouped) {
            // Decode-sized dense call: the weight side (MMA-M operand and its scales) of the first tile's first stages
            // goes out here, before the CTA's set-up barrier and the tensor-memory allocation (which may have to wait
            // for a predecessor's CTA on the same SM under programmatic dependent launch). Weights are immutable, so
            // this needs no wait for the preceding kernel; the activation side follows in the producer after its wait.
            TileCoord c0;
            if (decode_tile<false, EPI == EPI_CLUSTER>(p, blockIdx.x, p.tiles_a, c0)) {
                int const kb0 = c0.split * p.kb_per_split;
                int const kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                int const a_row0 = c0.a_tile * C::kBM;
                int const npre = min(S, kb1 - kb0);
                for (int i = 0; i < npre; ++i) {
                    uint32_t const fb = full_bar(i);
                    mbar_expect_tx(fb, C::kABytes + C::kBBytes + C::kSfaBytes + 512u);
                    tma_load_2d(sA + i * C::kABytes, &tm_a, fb, (kb0 + i) * C::kBK, a_row0);
                    bulk_load(sSfa + i * C::kSfaBytes,
                        p.sfa + (static_cast<int64_t>(a_row0 / 128) * p.kb_total + kb0 + i) * 512, 512, fb);
                }
            }
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t const tmem_base = *tmem_slot;
    // Decode-sized calls are chained with programmatic dependent launch: the next kernel may start its set-up and its
    // weight loads while this one runs, and this one has done the same under its predecessor. Before its
    // griddep_wait() a kernel reads only weights (immutable) and writes nothing outside its own CTA.
    if constexpr (kSwap) griddep_launch_dependents();
    constexpr bool kGS = kSwap && kGrouped;
    static_assert(!kGS || (BN >= 32 && (EPI == EPI_BF16 || EPI == EPI_CLUSTER)),
        "grouped + swapped: token tiles of 32 / 64 rows (scale columns cover 32 rows), bf16 output");
    // the routing tensors are the output of kernels earlier in the stream: nothing of them is read before the wait
    if constexpr (kGS) griddep_wait();

    int tiles_a_used = p.tiles_a;
    if constexpr (kGrouped && !kSwap) tiles_a_used = min(p.tiles_a, p.blk0[p.num_experts]);
    if constexpr (kGS) tiles_a_used = min(p.tiles_b, p.blk0[p.num_experts]);      // blocks in use
    int const rows_b_pad = (p.rows_b + 127) & ~127;
    auto next_tile = [&](int t, TileCoord& c) {
        if constexpr (kGS) return decode_tile_gs<BN, EPI == EPI_CLUSTER>(p, t, tiles_a_used, c);
        else return decode_tile<kGrouped, EPI == EPI_CLUSTER>(p, t, tiles_a_used, c);
    };

    if (warp == 0) {
        // ------------------------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            TileCoord c;
            bool ok = true;
            bool first_tile = true;
            for (int t = blockIdx.x; ok && next_tile(t, c); t += gridDim.x) {
                if constexpr (kGS) {
                    if (c.live <= 0) continue;
                }
                int kb0 = c.split * p.kb_per_split;
                int const kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                // grouped + swapped: the expert's weight rows follow each other in the [E * rows_a, K] weight, and
                // the token rows are the block's rows from its sub-tile on
                int const a_row0 = kGS ? c.expert * p.rows_a + c.a_tile * C::kBM : c.a_tile * C::kBM;
                int const b_row0 = kGS ? c.b_tile * 128 + c.sub * BN : c.b_tile * BN;
                int const b_coord = (kGrouped && !kSwap) ? c.expert * p.rows_b + b_row0 : b_row0;
                const uint8_t* sfb_base = p.sfb
                    + ((kGrouped && !kSwap) ? static_cast<int64_t>(c.expert) * (rows_b_pad / 128) * p.kb_total * 512 : 0);
                int sfb_atoms = 0;
                for (int j = 0; j < C::kSfbAtoms; ++j)
                    if (b_row0 + j * 128 < rows_b_pad) ++sfb_atoms;
                uint32_t const bytes = C::kABytes + C::kBBytes + C::kSfaBytes + 512u * sfb_atoms;
                // grouped: an expert with one block streams its weight tile exactly once; marking those lines
                // evict-first leaves L2 to the activation rows (read by every weight tile of the block) and to the
                // weight tiles a second block of the same expert is about to read again
                bool stream_b = false;
                uint64_t pol_first = 0;
                if constexpr (kGrouped && !kSwap) {
                    if (p.stream_b_hint != 0 && p.blk0[c.expert + 1] - p.blk0[c.expert] == 1) {
                        stream_b = true;
                        pol_first = policy_evict_first();
                    }
                }
                if constexpr (kSwap && !kGrouped) {
                    if (first_tile) {
                        // The weight side of the first stages went out during the CTA's set-up (above); the
                        // activation side, which the preceding kernel may still be writing, follows its completion.
                        // All stages are free at this point, no empty-barrier wait is needed.
                        first_tile = false;
                        int const npre = min(S, kb1 - kb0);
                        griddep_wait();
                        for (int i = 0; i < npre; ++i) {
                            uint32_t const fb = full_bar(i);
                            tma_load_2d(sB + i * C::kBBytes, &tm_b, fb, (kb0 + i) * C::kBK, b_coord);
                            for (int j = 0; j < sfb_atoms; ++j)
                                bulk_load(sSfb + i * C::kSfbBytes + j * 512,
                                    sfb_base + (static_cast<int64_t>(b_row0 / 128 + j) * p.kb_total + kb0 + i) * 512,
                                    512, fb);
                        }
                        kb0 += npre;
                        stage = npre == S ? 0 : npre;
                        phase = npre == S ? 1u : 0u;
                    }
                }
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!wait_or_abort(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        record_abort(FSO_DEV_WAIT_PRODUCER, abort_flag);
                        ok = false;
                        break;
                    }
                    uint32_t const fb = full_bar(stage);
                    mbar_expect_tx(fb, bytes);
                    tma_load_2d(sA + stage * C::kABytes, &tm_a, fb, kb * C::kBK, a_row0);
                    if (stream_b) tma_load_2d_hint(sB + stage * C::kBBytes, &tm_b, fb, kb * C::kBK, b_coord, pol_first);
                    else tma_load_2d(sB + stage * C::kBBytes, &tm_b, fb, kb * C::kBK, b_coord);
                    bulk_load(sSfa + stage * C::kSfaBytes,
                        p.sfa + (static_cast<int64_t>(a_row0 / 128) * p.kb_total + kb) * 512, 512, fb);
                    for (int j = 0; j < sfb_atoms; ++j)
                        bulk_load(sSfb + stage * C::kSfbBytes + j * 512,
                            sfb_base + (static_cast<int64_t>(b_row0 / 128 + j) * p.kb_total + kb) * 512, 512, fb);
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            int sfbuf = 0;
            int tiles_done = 0;
            constexpr uint32_t idesc = make_idesc_mxf8(BN);
            TileCoord c;
            bool ok = true;
            for (int t = blockIdx.x; ok && next_tile(t, c); t += gridDim.x) {
                if constexpr (kGS) {
                    if (c.live <= 0) continue;
                }
                int const kb0 = c.split * p.kb_per_split;
                int const kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                if (!wait_or_abort(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
                    record_abort(FSO_DEV_WAIT_MMA_TMEM, abort_flag);
                    break;
                }
                tc_fence_after();
                uint32_t const d_tmem = tmem_base + static_cast<uint32_t>(acc * C::kAccStride);
                uint32_t const sfb_col_off = kGS ? static_cast<uint32_t>((c.sub * BN) >> 5)
                    : BN < 128 ? static_cast<uint32_t>(((c.b_tile * BN) & 127) >> 5) : 0u;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!wait_or_abort(full_bar(stage), phase, abort_flag)) {
                        record_abort(FSO_DEV_WAIT_MMA_FULL, abort_flag);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    uint32_t const sf_col = tmem_base + C::kAccCols + sfbuf * C::kSfBufCols;
                    tc_cp_32x128b_warpx4(sf_col, make_desc_sf(sSfa + stage * C::kSfaBytes));
#pragma unroll
                    for (int j = 0; j < C::kSfbAtoms; ++j)
                        tc_cp_32x128b_warpx4(sf_col + C::kSfaCols + 4 * j,
                            make_desc_sf(sSfb + stage * C::kSfbBytes + j * 512));
                    if constexpr (C::kOverlapAcc) {
                        if (kb == kb0) {
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
                    }
                    uint64_t const adesc = make_desc_sw128(sA + stage * C::kABytes);
                    uint64_t const bdesc = make_desc_sw128(sB + stage * C::kBBytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma_mxf8(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc | sf_id_bits(k), sf_col,
                            sf_col + C::kSfaCols + sfb_col_off, (kb > kb0 || k > 0) ? 1u : 0u);
                    tc_commit(empty_bar(stage));
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    sfbuf ^= 1;
                }
                if (!ok) break;
                tc_commit(tfull_bar(acc));
                if (++acc == C::kAccStages) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------------------------------ epilogue
        if constexpr (kSwap) griddep_wait();              // before this kernel's first global store
        int const ew = warp - 4;
        int const quarter = warp & 3;
        int const half = ew >> 2;
        constexpr int kColsPerWarp = BN / (C::kEpiWarps / 4);
        int acc = 0;
        uint32_t acc_phase = 0;
        TileCoord c;
        for (int t = blockIdx.x; next_tile(t, c); t += gridDim.x) {
            if constexpr (kGS) {
                if (c.live <= 0) continue;
            }
            if (!wait_or_abort(tfull_bar(acc), acc_phase, abort_flag)) {
                if (lane == 0) record_abort(FSO_DEV_WAIT_EPILOGUE, abort_flag);
                break;
            }
            tc_fence_after();
            uint32_t const t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16)
                + static_cast<uint32_t>(acc * C::kAccStride);
            int const a_row = c.a_tile * C::kBM + quarter * 32 + lane;   // this thread's row of the MMA-M operand
            // Overlapping accumulators: the 32 shared columns are the last 32 of accumulator 0 and the first 32 of
            // accumulator 1. A warp walks its 32-column chunks from the end in accumulator 0 and from the start in
            // accumulator 1, so the warps whose slice holds the shared columns drain them first and say so.
            constexpr int kSlices = C::kEpiWarps / 4;
            bool const rev = C::kOverlapAcc && acc == 0;
            bool const ovl_owner = C::kOverlapAcc && half == (acc == 0 ? kSlices - 1 : 0);
            auto release_shared_columns = [&]() {
                if (ovl_owner) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(ovl_bar);
                }
            };
            int const b_row0 = kGS ? c.b_tile * 128 + c.sub * BN : c.b_tile * BN;
            int const b_bound = kGS ? b_row0 + c.live : p.rows_b;        // swapped: first token row past this tile's
            bool released = false;

            if constexpr (EPI == EPI_CLUSTER) {
                // one work item per CTA: keep the accumulator row in registers for the reduction after the loop
#pragma unroll
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld_32x16(t_row + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) red_v[c0 + j] = __uint_as_float(r[j]);
                }
                red_have = true;
                red_c = c;
            } else if constexpr (EPI == EPI_SWIGLU) {
                // 64 interleaved (gate, up) accumulator columns per warp -> 32 outputs = one 1x32 block per row.
                // The slice is drained into registers and the accumulator handed back before the math starts.
                static_assert(kColsPerWarp == 64, "one 1x32 output block per warp");
                int const inter = p.ldo;
                uint32_t r0[32], r1[32];
                tmem_ld_32x32(t_row + half * 64, r0);
                tmem_ld_32x32(t_row + half * 64 + 32, r1);
                tmem_ld_wait();
                release_shared_columns();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                released = true;
                float h[32];
                float amax = 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    h[j] = silu_mul(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
                    h[16 + j] = silu_mul(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
                    amax = fmaxf(amax, fmaxf(fabsf(h[j]), fabsf(h[16 + j])));
                }
                amax = fmaxf(amax, 1e-10f);
                float qs;
                uint32_t const byte = e8m0_from_amax(amax, qs);
                uint32_t o[8];
#pragma unroll
                for (int v = 0; v < 8; ++v)
                    o[v] = fp8x4(__fmul_rn(h[4 * v], qs), __fmul_rn(h[4 * v + 1], qs), __fmul_rn(h[4 * v + 2], qs),
                        __fmul_rn(h[4 * v + 3], qs));
                if (a_row < p.out_rows) {
                    uint8_t* const dst = static_cast<uint8_t*>(p.out) + static_cast<int64_t>(a_row) * inter
                        + c.b_tile * (BN / 2) + half * 32;
                    if (p.out_align32) {
                        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                     ::"l"(dst), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]),
                                     "r"(o[6]), "r"(o[7])
                                     : "memory");
                    } else {
                        reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
                        reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                    // byte `half` (0..3) of the row's scale word for K block b_tile of the output
                    reinterpret_cast<uint8_t*>(p.out_sf)[sf_word_index(a_row, c.b_tile, inter / 128) * 4 + half]
                        = static_cast<uint8_t>(byte);
                } else if constexpr (!kGrouped) {
                    // dense call: the rows between M and the next multiple of 128 carry zero scale words, as every
                    // producer of the activation contract leaves them
                    reinterpret_cast<uint8_t*>(p.out_sf)[sf_word_index(a_row, c.b_tile, inter / 128) * 4 + half] = 0;
                }
            } else if constexpr (!kSwap && EPI == EPI_BF16) {
                // row = output row, columns = output columns. The accumulator slice is drained into packed bf16
                // registers first and handed back to the MMA issuer; the global stores then overlap the next tile.
                constexpr int kChunks = kColsPerWarp / 32;
                static_assert(kChunks % 2 == 0, "chunks are drained two at a time");
                uint32_t packed[kChunks * 16];
                int const col_w = b_row0 + half * kColsPerWarp;          // first output column of this warp
                auto chunk_col = [&](int j) { return 32 * (rev ? kChunks - 1 - j : j); };
                auto load_chunk = [&](int j, uint32_t (&r)[32]) {
                    tmem_ld_32x32(t_row + static_cast<uint32_t>(half * kColsPerWarp + chunk_col(j)), r);
                };
                // bias per column (the same for every row: broadcast loads), residual from this row
                auto fuse32 = [&](uint32_t (&r)[32], int col) {
                    if (col >= p.rows_b) return;
                    bool const has_bias = p.bias != nullptr;
                    bool const has_res = p.residual != nullptr && a_row < p.rows_a;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 bw = make_uint4(0, 0, 0, 0), rw = make_uint4(0, 0, 0, 0);
                        if (has_bias) bw = __ldg(reinterpret_cast<const uint4*>(p.bias + col + 8 * q));
                        if (has_res)
                            rw = __ldg(reinterpret_cast<const uint4*>(
                                p.residual + static_cast<int64_t>(a_row) * p.ldo + col + 8 * q));
                        uint32_t const bws[4] = {bw.x, bw.y, bw.z, bw.w};
                        uint32_t const rws[4] = {rw.x, rw.y, rw.z, rw.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float lo = epilogue_value(__uint_as_float(r[8 * q + 2 * i]),
                                bias_term(__ushort_as_bfloat16(static_cast<unsigned short>(bws[i] & 0xFFFFu))),
                                has_bias, p.act);
                            float hi = epilogue_value(__uint_as_float(r[8 * q + 2 * i + 1]),
                                bias_term(__ushort_as_bfloat16(static_cast<unsigned short>(bws[i] >> 16))),
                                has_bias, p.act);
                            if (has_res) {
                                lo += bf16_lo(rws[i]);
                                hi += bf16_hi(rws[i]);
                            }
                            r[8 * q + 2 * i] = __float_as_uint(lo);
                            r[8 * q + 2 * i + 1] = __float_as_uint(hi);
                        }
                    }
                };
                uint32_t ra[32], rb[32];
                load_chunk(0, ra);
                tmem_ld_wait();
                release_shared_columns();
#pragma unroll
                for (int j = 0; j < kChunks; j += 2) {
                    // one load in flight while the chunk before it is packed
                    load_chunk(j + 1, rb);
                    if constexpr (kFused) fuse32(ra, col_w + chunk_col(j));
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        packed[16 * j + i] = pack_bf16x2(__uint_as_float(ra[2 * i]), __uint_as_float(ra[2 * i + 1]));
                    tmem_ld_wait();
                    if (j + 2 < kChunks) load_chunk(j + 2, ra);
                    if constexpr (kFused) fuse32(rb, col_w + chunk_col(j + 1));
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        packed[16 * (j + 1) + i]
                            = pack_bf16x2(__uint_as_float(rb[2 * i]), __uint_as_float(rb[2 * i + 1]));
                    if (j + 2 < kChunks) tmem_ld_wait();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                released = true;
                if (a_row < p.rows_a) {
                    __nv_bfloat16* const orow = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(a_row) * p.ldo
                        + col_w;
#pragma unroll
                    for (int g = 0; g < 2 * kChunks; ++g) {
                        int const c0 = chunk_col(g >> 1) + 16 * (g & 1);
                        if (col_w + c0 < p.rows_b) {
                            uint32_t const* v = &packed[8 * g];
                            if (p.out_align32) {
                                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                             ::"l"(orow + c0), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]),
                                             "r"(v[5]), "r"(v[6]), "r"(v[7])
                                             : "memory");
                            } else {
                                uint4* dst = reinterpret_cast<uint4*>(orow + c0);
                                dst[0] = make_uint4(v[0], v[1], v[2], v[3]);
                                dst[1] = make_uint4(v[4], v[5], v[6], v[7]);
                            }
                        }
                    }
                }
            } else if constexpr (!kSwap && EPI == EPI_QUANT) {
                // row = output row; per 32 columns one 1x32 block of the next layer's activation
                static_assert(kColsPerWarp == 128 || kColsPerWarp == 64, "whole or half scale words per warp");
                uint32_t codes[kColsPerWarp / 4];
                uint32_t word = 0;
                int const col_w = b_row0 + half * kColsPerWarp;          // first output column of this warp
                constexpr int kChunks = kColsPerWarp / 32;
                auto chunk_col = [&](int j) { return 32 * (rev ? kChunks - 1 - j : j); };
#pragma unroll
                for (int j = 0; j < kChunks; ++j) {
                    int const c0 = chunk_col(j);
                    uint32_t r[32];
                    tmem_ld_32x32(t_row + static_cast<uint32_t>(half * kColsPerWarp + c0), r);
                    tmem_ld_wait();
                    if (j == 0) release_shared_columns();
                    if constexpr (kFused) {
                        if (col_w + c0 < p.rows_b) {
                            bool const has_bias = p.bias != nullptr;
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint4 bw = make_uint4(0, 0, 0, 0);
                                if (has_bias) bw = __ldg(reinterpret_cast<const uint4*>(p.bias + col_w + c0 + 8 * q));
                                uint32_t const bws[4] = {bw.x, bw.y, bw.z, bw.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    r[8 * q + 2 * i] = __float_as_uint(epilogue_value(__uint_as_float(r[8 * q + 2 * i]),
                                        bias_term(__ushort_as_bfloat16(static_cast<unsigned short>(bws[i] & 0xFFFFu))),
                                        has_bias, p.act));
                                    r[8 * q + 2 * i + 1] = __float_as_uint(epilogue_value(
                                        __uint_as_float(r[8 * q + 2 * i + 1]),
                                        bias_term(__ushort_as_bfloat16(static_cast<unsigned short>(bws[i] >> 16))),
                                        has_bias, p.act));
                                }
                            }
                        }
                    }
                    float v[32];
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        v[i] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[i])));   // the bf16 output's value
                        amax = fmaxf(amax, fabsf(v[i]));
                    }
                    amax = fmaxf(amax, 1e-10f);
                    float qs;
                    word |= e8m0_from_amax(amax, qs) << (8 * (c0 / 32));
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        codes[8 * j + q] = fp8x4(__fmul_rn(v[4 * q], qs), __fmul_rn(v[4 * q + 1], qs),
                            __fmul_rn(v[4 * q + 2], qs), __fmul_rn(v[4 * q + 3], qs));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                released = true;
                if (col_w < p.rows_b) {
                    int const kp = col_w >> 7;
                    uint8_t* const sfb = reinterpret_cast<uint8_t*>(p.out_sf) + sf_word_index(a_row, kp, p.ldo / 128) * 4;
                    if (a_row < p.rows_a) {
                        uint8_t* const dst = static_cast<uint8_t*>(p.out) + static_cast<int64_t>(a_row) * p.ldo + col_w;
#pragma unroll
                        for (int j = 0; j < kChunks; ++j) {
                            int const c0 = chunk_col(j);
                            uint32_t const* o = &codes[8 * j];
                            if (p.out_align32) {
                                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                             ::"l"(dst + c0), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]),
                                             "r"(o[5]), "r"(o[6]), "r"(o[7])
                                             : "memory");
                            } else {
                                reinterpret_cast<uint4*>(dst + c0)[0] = make_uint4(o[0], o[1], o[2], o[3]);
                                reinterpret_cast<uint4*>(dst + c0)[1] = make_uint4(o[4], o[5], o[6], o[7]);
                            }
                        }
                    } else {
                        word = 0;                        // rows between M and the next multiple of 128: zero words
                    }
                    if constexpr (kColsPerWarp == 128)
                        *reinterpret_cast<uint32_t*>(sfb) = word;
                    else
                        *reinterpret_cast<uint16_t*>(sfb + ((col_w & 127) >> 5)) = static_cast<uint16_t>(word);
                }
            } else if constexpr (!kSwap) {
                // split-K partial, normal orientation: fp32 rows straight from tensor memory
                constexpr int kChunks = kColsPerWarp / 32;
#pragma unroll 1
                for (int j = 0; j < kChunks; ++j) {
                    int const c0 = half * kColsPerWarp + 32 * (rev ? kChunks - 1 - j : j);
                    uint32_t r[32];
                    tmem_ld_32x32(t_row + static_cast<uint32_t>(c0), r);
                    tmem_ld_wait();
                    if (j == 0) release_shared_columns();
                    int const col = b_row0 + c0;
                    if (a_row < p.rows_a && col < p.rows_b) {
                        uint4* dst = reinterpret_cast<uint4*>(p.ws + static_cast<int64_t>(c.split) * p.out_rows * p.ldo
                            + static_cast<int64_t>(a_row) * p.ldo + col);
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            dst[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                    }
                }
            } else {
                // swapped: this thread's row is an output COLUMN (a weight row), tensor-memory columns are tokens
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld_32x16(t_row + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        int const m = b_row0 + c0 + j;
                        if (m < b_bound && a_row < p.rows_a) {
                            if constexpr (EPI == EPI_BF16) {
                                float v = __uint_as_float(r[j]);
                                if constexpr (kFused) {
                                    v = epilogue_value(v, p.bias != nullptr ? bias_term(p.bias[a_row]) : 0.f,
                                        p.bias != nullptr, p.act);
                                    if (p.residual != nullptr)
                                        v += __bfloat162float(p.residual[static_cast<int64_t>(m) * p.ldo + a_row]);
                                }
                                if (kGS && p.out_f32)
                                    static_cast<float*>(p.out)[static_cast<int64_t>(m) * p.ldo + a_row] = v;
                                else
                                    static_cast<__nv_bfloat16*>(p.out)[static_cast<int64_t>(m) * p.ldo + a_row]
                                        = __float2bfloat16_rn(v);
                            } else
                                p.ws[static_cast<int64_t>(c.split) * p.out_rows * p.ldo
                                    + static_cast<int64_t>(m) * p.ldo + a_row] = __uint_as_float(r[j]);
                        }
                    }
                }
            }
            if (!released) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
            }
            if (++acc == C::kAccStages) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        __syncwarp();
    }

    if constexpr (EPI == EPI_CLUSTER) {
        // ------------------------------------------------------------------ split-K reduction inside the cluster
        uint32_t const rank = cluster_ctarank();
        int const row = (warp & 3) * 32 + lane;
        // Every thread of the cluster has left its main loop: the epilogue warps arrive after their accumulator is
        // complete, so no MMA or TMA of CTA 0 still touches its stage buffers, which now receive the other slices.
        cluster_arrive();
        cluster_wait();
        if (warp >= 4 && red_have && rank != 0) {
#pragma unroll
            for (int j = 0; j < BN; ++j)
                st_cluster_f32(map_to_cta(base + red_off + 4u * (((rank - 1u) * BN + j) * 128u + row), 0u), red_v[j]);
        }
        cluster_arrive();
        cluster_wait();                                   // the other slices' rows are in CTA 0's shared memory
        if (warp >= 4 && red_have && rank == 0) {
            const float* const red = reinterpret_cast<const float*>(gbase + red_off);
            for (int s2 = 1; s2 < p.splits; ++s2)
#pragma unroll
                for (int j = 0; j < BN; ++j) red_v[j] += red[((s2 - 1) * BN + j) * 128 + row];
            int const a_row = red_c.a_tile * C::kBM + row;
            int const b_row0 = kGS ? red_c.b_tile * 128 + red_c.sub * BN : red_c.b_tile * BN;
            int const b_bound = kGS ? b_row0 + red_c.live : p.rows_b;
#pragma unroll
            for (int j = 0; j < BN; ++j) {
                int const m = b_row0 + j;
                if (m < b_bound && a_row < p.rows_a) {
                    float v = red_v[j];
                    if constexpr (kFused) {
                        v = epilogue_value(v, p.bias != nullptr ? bias_term(p.bias[a_row]) : 0.f, p.bias != nullptr,
                            p.act);
                        if (p.residual != nullptr)
                            v += __bfloat162float(p.residual[static_cast<int64_t>(m) * p.ldo + a_row]);
                    }
                    if (kGS && p.out_f32)
                        static_cast<float*>(p.out)[static_cast<int64_t>(m) * p.ldo + a_row] = v;
                    else
                        static_cast<__nv_bfloat16*>(p.out)[static_cast<int64_t>(m) * p.ldo + a_row] = __float2bfloat16_rn(v);
                }
            }
        }
    }

    // ---------------------------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out somewhere: give copies that may still be in flight time to land before the CTA leaves
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// Sums the split-K partials in slice order, applies the dense epilogue when there is one (bias / act / residual all
// absent: the plain sum) and rounds once to bf16. n % 4 == 0.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float4* __restrict__ ws, uint2* __restrict__ out,
    int64_t quads, int splits, int n, const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
    int act)
{
    griddep_launch_dependents();
    griddep_wait();                                       // the partials are the preceding kernel's output
    int64_t const i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= quads) return;
    float4 acc = ws[i];
    for (int s = 1; s < splits; ++s) {
        float4 const v = ws[static_cast<int64_t>(s) * quads + i];
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
    }
    if (bias != nullptr || residual != nullptr || act != 0) {
        int const col = static_cast<int>((i * 4) % n);
        bool const hb = bias != nullptr;
        acc.x = epilogue_value(acc.x, hb ? bias_term(bias[col]) : 0.f, hb, act);
        acc.y = epilogue_value(acc.y, hb ? bias_term(bias[col + 1]) : 0.f, hb, act);
        acc.z = epilogue_value(acc.z, hb ? bias_term(bias[col + 2]) : 0.f, hb, act);
        acc.w = epilogue_value(acc.w, hb ? bias_term(bias[col + 3]) : 0.f, hb, act);
        if (residual != nullptr) {
            uint2 const rw = *reinterpret_cast<const uint2*>(residual + i * 4);
            acc.x += bf16_lo(rw.x);
            acc.y += bf16_hi(rw.x);
            acc.z += bf16_lo(rw.y);
            acc.w += bf16_hi(rw.y);
        }
    }
    uint2 o;
    o.x = pack_bf16x2(acc.x, acc.y);
    o.y = pack_bf16x2(acc.z, acc.w);
    out[i] = o;
}

}  // namespace fso
