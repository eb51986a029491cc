// Host side of the GEMM family: tensor-map encoding, the shape -> (orientation, tile, split) picker and launchers.
#pragma once

#include <algorithm>
#include <atomic>
#include <mutex>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "gemm.cuh"
#include "gemm2.cuh"

namespace fso {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Tensor map of a row-major byte matrix [rows, k] read in boxes of 128 bytes x box_rows with the 128-byte swizzle.
inline int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return FSO_ERR_UNSUPPORTED;
    }
    cuuint64_t const dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    cuuint64_t const strides[1] = {static_cast<cuuint64_t>(k)};
    cuuint32_t const box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t const estr[2] = {1u, 1u};
    CUresult const r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows %lld, k %lld, box %d)", static_cast<int>(r),
            static_cast<long long>(rows), static_cast<long long>(k), box_rows);
        return FSO_ERR_INTERNAL;
    }
    return 0;
}

// The route one dense shape takes. Pure host arithmetic on (M, N, K, SMs).
struct DensePlan {
    bool swap;      // weight rows on MMA-M, activation rows on MMA-N
    int bn;         // MMA-N tile
    int splits;
    int kb_per_split;
    int tiles_a, tiles_b;
    int group_a;
    int64_t ws_bytes;
    double cost;    // normal orientation: rounds of the persistent schedule x tile width (see plan_dense)
};

// FSO_B200_DENSE_TILE=256 | 128 | pair forces the tile of the normal-orientation calls where that tile can serve the
// shape (measurement; read once per process). Unset: the picker below decides.
inline int forced_dense_tile()
{
    static int const v = [] {
        const char* e = std::getenv("FSO_B200_DENSE_TILE");
        if (e == nullptr) return 0;
        if (std::strcmp(e, "pair") == 0) return 2;
        int const t = std::atoi(e);
        return (t == 256 || t == 128) ? t : 0;
    }();
    return v;
}

// Rounds a persistent grid of `slots` CTAs (or CTA pairs) needs for `tiles` equal tiles.
inline double schedule_rounds(int64_t tiles, int64_t slots)
{
    return static_cast<double>((tiles + slots - 1) / slots);
}

// A 128-wide tile moves twice the weight bytes per flop of a 256-wide one, so a round of 128-wide tiles is charged
// more than half a round of 256-wide ones: 1.17-1.22 measured on five shapes with both tiles forced (1024 x 28672,
// 4096 x 4096, 1024 x 6144, 2048 x 6144, 512 x 28672; K = 4096).
constexpr double kNarrowTilePenalty = 1.18;

// Fraction of the (persistent, one CTA per SM) grid kept busy by `items` equal work items.
inline double wave_efficiency(int64_t items, int sms)
{
    int64_t const rounds = (items + sms - 1) / sms;
    return static_cast<double>(items) / static_cast<double>(rounds * sms);
}

// Largest split count the cluster form takes for a token tile (room for the other slices' accumulators in CTA 0's
// shared memory; 8 is the portable cluster size).
inline int cluster_split_limit(int bn)
{
    int const slices = bn == 16 ? GemmCfg<16, EPI_CLUSTER>::kRedSlices : bn == 32 ? GemmCfg<32, EPI_CLUSTER>::kRedSlices
        : bn == 64 ? GemmCfg<64, EPI_CLUSTER>::kRedSlices : 0;
    return slices + 1 < 8 ? slices + 1 : 8;
}

inline void pick_splits(int64_t tiles, int kb, int sms, int min_kb, int max_s, int* splits, int* kb_per)
{
    int best_s = 1;
    double best = wave_efficiency(tiles, sms);
    if (tiles * 2 <= sms) {
        for (int s = 2; s <= max_s; ++s) {
            int const per = (kb + s - 1) / s;
            if (per < min_kb) break;
            int const real = (kb + per - 1) / per;
            if (real != s) continue;
            double const e = wave_efficiency(tiles * s, sms) * (static_cast<double>(kb) / (per * s));
            if (e > best + 0.02) {
                best = e;
                best_s = s;
            }
        }
    }
    *splits = best_s;
    *kb_per = (kb + best_s - 1) / best_s;
}

// Decode-sized (swapped) problems are latency-bound, not wave-bound: measured on the four Llama-3-8B shapes at M = 16,
// about 128-200 half-SM CTAs is the best grid (gate_up: 224 tiles unsplit; qkv 48 x 4; o_proj and down 32 x 4; eight
// slices of the same shapes are slower again). So: the largest slice count that keeps tiles * slices <= 200, at
// most 4 once the tiles alone fill a sixth of the slots, every slice at least 4 K blocks and none empty.
inline void pick_decode_splits(int64_t tiles, int kb, int limit, int* splits, int* kb_per)
{
    int best = 1;
    int const smax = tiles >= 25 ? (limit < 4 ? limit : 4) : limit;
    for (int s = 2; s <= smax; ++s) {
        int const per = (kb + s - 1) / s;
        if (per < 4) break;
        if ((kb + per - 1) / per != s) continue;
        if (tiles * s <= 200) best = s;
    }
    *splits = best;
    *kb_per = (kb + best - 1) / best;
}

// FSO_B200_DENSE_TWO_TOKEN_TILES=0 keeps calls of 65..128 rows in the normal orientation (measurement).
inline bool two_token_tiles_enabled()
{
    static int const v = [] {
        const char* e = std::getenv("FSO_B200_DENSE_TWO_TOKEN_TILES");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    return v != 0;
}

inline DensePlan plan_dense(int64_t m, int64_t n, int64_t k, int sms)
{
    DensePlan p{};
    int const kb = static_cast<int>(k / 128);
    if (m <= 64) {
        p.swap = true;
        p.bn = m <= 16 ? 16 : m <= 32 ? 32 : 64;
        p.tiles_a = static_cast<int>(n / 128);
        p.tiles_b = 1;
        p.group_a = p.tiles_a;
        pick_decode_splits(p.tiles_a, kb, cluster_split_limit(p.bn), &p.splits, &p.kb_per_split);
    } else if (m <= 128 && n / 128 <= sms && two_token_tiles_enabled()) {
        // 65..128 rows on a weight of at most one 128-row panel per SM: still a weight-streaming problem. Two 64-row
        // token tiles per weight panel in the swapped orientation, neighbours in the schedule (the second reads the
        // panel from L2), K slices summed inside clusters: one launch, where the normal orientation would run a
        // third of the SMs on 128-wide tiles and sum its K slices through the fp32 workspace in a second launch
        // (qkv 6144 x 4096 at M = 128: 15.0 us that way, 12.7 us this way, cuBLAS 11.4; o_proj and down alike).
        p.swap = true;
        p.bn = 64;
        p.tiles_a = static_cast<int>(n / 128);
        p.tiles_b = 2;
        p.group_a = 1;
        // (K slices up to 130 / 200 / 296 CTAs measured alike on the Llama shapes: the decode rule's 200 is kept)
        pick_decode_splits(static_cast<int64_t>(p.tiles_a) * 2, kb, cluster_split_limit(p.bn), &p.splits,
            &p.kb_per_split);
    } else {
        p.swap = false;
        int const tiles_m = static_cast<int>((m + 127) / 128);
        // Tile width by the rounds of the persistent schedule: a round costs its tile width (an MMA's time is
        // proportional to N). Whole problems of at most half a round of 256-wide tiles and shapes that leave the last
        // round of 256-wide tiles nearly empty (1024 x 6144: 192 tiles on 148 SMs) take 128-wide tiles.
        double const c256 = n % 256 == 0 ? schedule_rounds(static_cast<int64_t>(tiles_m) * (n / 256), sms) * 256.0 : 1e30;
        double const c128 = schedule_rounds(static_cast<int64_t>(tiles_m) * ((n + 127) / 128), sms) * 128.0
            * kNarrowTilePenalty;
        p.bn = c256 <= c128 ? 256 : 128;
        if (forced_dense_tile() == 128 || (forced_dense_tile() == 256 && n % 256 == 0)) p.bn = forced_dense_tile();
        p.cost = p.bn == 256 ? c256 : c128;
        p.tiles_a = tiles_m;
        p.tiles_b = static_cast<int>((n + p.bn - 1) / p.bn);
        p.group_a = tiles_m < 16 ? tiles_m : 16;
        pick_splits(static_cast<int64_t>(p.tiles_a) * p.tiles_b, kb, sms, 8, 16, &p.splits, &p.kb_per_split);
    }
    p.ws_bytes = p.splits > 1 ? static_cast<int64_t>(p.splits) * m * n * 4 : 0;
    return p;
}

template <typename Kernel>
inline int ensure_smem_attr(Kernel kernel, int smem_bytes, std::atomic<uint64_t>& done_mask)
{
    int const dev = current_device();
    uint64_t const bit = 1ull << (dev & 63);
    if ((done_mask.load(std::memory_order_acquire) & bit) == 0) {
        FSO_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        // all of the SM's configurable memory as shared memory: the half-SM kernels then fit two CTAs per SM
        FSO_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
            static_cast<int>(cudaSharedmemCarveoutMaxShared)));
        done_mask.fetch_or(bit, std::memory_order_release);
    }
    return 0;
}

// FSO_B200_PDL=0 launches the decode-sized kernels without programmatic dependent launch (plain stream order).
inline bool pdl_enabled()
{
    static int const v = [] {
        const char* e = getenv("FSO_B200_PDL");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    return v != 0;
}

// The launch attribute that lets a kernel start while its predecessor in the stream is still running (the kernel
// itself waits, with griddepcontrol.wait, before it touches anything the predecessor may produce).
inline int pdl_attribute(cudaLaunchAttribute* attr)
{
    if (!pdl_enabled()) return 0;
    attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr->val.programmaticStreamSerializationAllowed = 1;
    return 1;
}

// FSO_PRINT_TILE_INFO=1: print, once per kernel instantiation that is launched, the tile it runs, the stage count
// its shared-memory budget gave and the resources it asks for (host side, read once, off unless set; the reference's
// switch of the same name, arch/sm100/mxfp8/grouped_dispatch.cuh:162-176).
inline bool print_tile_info()
{
    static int const v = [] {
        const char* e = std::getenv("FSO_PRINT_TILE_INFO");
        return (e != nullptr && e[0] != '\0' && e[0] != '0') ? 1 : 0;
    }();
    return v != 0;
}

inline void print_tile_info_once(std::atomic<int>& printed, const char* kernel, int bm, int bn, int epi, bool swap,
    bool grouped, bool fused, int stages, int smem_bytes, int threads, int tmem_cols)
{
    if (!print_tile_info() || printed.exchange(1) != 0) return;
    std::fprintf(stderr,
        "[fso_b200] %s: tile %d x %d x 128, epilogue %d, %s orientation%s%s, %d stages, %d bytes of shared memory, "
        "%d threads, %d tensor-memory columns\n",
        kernel, bm, bn, epi, swap ? "swapped" : "normal", grouped ? ", grouped" : "", fused ? ", fused epilogue" : "",
        stages, smem_bytes, threads, tmem_cols);
}

template <int BN, int EPI, bool kSwap, bool kGrouped, bool kFused = false>
inline int launch_gemm_inst(CUtensorMap const& ta, CUtensorMap const& tb, GemmParams const& p, int grid,
    cudaStream_t stream)
{
    using C = GemmCfg<BN, EPI>;
    static std::atomic<uint64_t> done{0};
    auto kernel = gemm_mxf8_kernel<BN, EPI, kSwap, kGrouped, kFused>;
    int const rc = ensure_smem_attr(kernel, C::kSmemBytes, done);
    if (rc != 0) return rc;
    static std::atomic<int> printed{0};
    print_tile_info_once(printed, "gemm_mxf8_kernel", C::kBM, BN, EPI, kSwap, kGrouped, kFused, C::kStages, C::kSmemBytes,
        C::kThreads, C::kTmemCols);
    if constexpr (kSwap) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
        cfg.blockDim = dim3(C::kThreads, 1, 1);
        cfg.dynamicSmemBytes = C::kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        cfg.attrs = attr;
        cfg.numAttrs = pdl_attribute(&attr[0]);
        FSO_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, p));
    } else {
        kernel<<<grid, C::kThreads, C::kSmemBytes, stream>>>(ta, tb, p);
    }
    return launch_status("gemm_mxf8_kernel");
}

template <int BN>
inline void cluster_launch_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int items, int splits,
    cudaStream_t stream)
{
    using C = GemmCfg<BN, EPI_CLUSTER>;
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3(static_cast<unsigned>(items), 1, 1);
    cfg.blockDim = dim3(C::kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(splits);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
}

// How many clusters of `splits` CTAs of the cluster split-K kernel this device runs at the same time (one CTA per
// SM, a cluster inside one GPC); asked once per device and cluster size. 0 = cannot be launched.
template <int BN, bool kFused = false>
inline int cluster_capacity(int splits)
{
    using C = GemmCfg<BN, EPI_CLUSTER>;
    static std::atomic<int> cap[64][9];          // 0 = not asked yet, else capacity + 1
    static std::atomic<uint64_t> done{0};
    int const dev = current_device() & 63;
    if (splits < 2 || splits > 8) return 0;
    int v = cap[dev][splits].load(std::memory_order_acquire);
    if (v == 0) {
        auto kernel = gemm_mxf8_kernel<BN, EPI_CLUSTER, true, false, kFused>;
        int clusters = 0;
        if (ensure_smem_attr(kernel, C::kSmemBytes, done) == 0) {
            cudaLaunchConfig_t cfg;
            cudaLaunchAttribute attr[1];
            cluster_launch_config<BN>(cfg, attr, splits, splits, nullptr);
            if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {
                (void)cudaGetLastError();
                clusters = 0;
            }
        }
        v = clusters + 1;
        cap[dev][splits].store(v, std::memory_order_release);
    }
    return v - 1;
}

inline int cluster_capacity_bn(int bn, int splits, bool fused)
{
    if (fused)
        return bn == 16 ? cluster_capacity<16, true>(splits) : bn == 32 ? cluster_capacity<32, true>(splits)
            : bn == 64 ? cluster_capacity<64, true>(splits) : 0;
    return bn == 16 ? cluster_capacity<16>(splits) : bn == 32 ? cluster_capacity<32>(splits)
        : bn == 64 ? cluster_capacity<64>(splits) : 0;
}

// The swapped kernel with split-K inside thread-block clusters of `splits` CTAs (one CTA per work item).
template <int BN, bool kFused = false, bool kGrouped = false>
inline int launch_gemm_cluster(CUtensorMap const& ta, CUtensorMap const& tb, GemmParams const& p, int items,
    cudaStream_t stream)
{
    auto kernel = gemm_mxf8_kernel<BN, EPI_CLUSTER, true, kGrouped, kFused>;
    if constexpr (kGrouped) {
        static std::atomic<uint64_t> done{0};
        int const rc = ensure_smem_attr(kernel, GemmCfg<BN, EPI_CLUSTER>::kSmemBytes, done);
        if (rc != 0) return rc;
    }
    using C = GemmCfg<BN, EPI_CLUSTER>;
    static std::atomic<int> printed{0};
    print_tile_info_once(printed, "gemm_mxf8_kernel (split-K inside clusters)", C::kBM, BN, EPI_CLUSTER, true, kGrouped,
        kFused, C::kStages, C::kSmemBytes, C::kThreads, C::kTmemCols);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    cluster_launch_config<BN>(cfg, attr, items, p.splits, stream);
    cfg.numAttrs += pdl_attribute(&attr[1]);
    FSO_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, p));
    return launch_status("gemm_mxf8_kernel (cluster split-K)");
}

// Tensor map over a scale-word buffer seen as [atoms, 128] 32-bit words (one 512-byte atom per row), box = one atom.
inline int make_sf_map(CUtensorMap* map, const void* base, int64_t atoms)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return FSO_ERR_UNSUPPORTED;
    }
    cuuint64_t const dims[2] = {128u, static_cast<cuuint64_t>(atoms)};
    cuuint64_t const strides[1] = {512u};
    cuuint32_t const box[2] = {128u, 1u};
    cuuint32_t const estr[2] = {1u, 1u};
    CUresult const r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (scale words) failed with CUresult %d", static_cast<int>(r));
        return FSO_ERR_INTERNAL;
    }
    return 0;
}

// The CTA-pair kernel (gemm2.cuh) takes the normal-orientation calls without split-K and without a fused epilogue
// whose 256 x 256 tiles fill the SM pairs; it is bit-identical to the single-CTA kernel and a few per cent faster on
// those shapes on B200. FSO_B200_PAIR=0 keeps every call on the single-CTA kernel (read once per process).
inline bool pair_kernel_enabled()
{
    static int const v = [] {
        const char* e = std::getenv("FSO_B200_PAIR");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    return v != 0;
}

inline bool use_pair_kernel(int64_t m, int64_t n, int sms, bool swap, int splits)
{
    if (swap || splits != 1 || n % 256 != 0 || !pair_kernel_enabled()) return false;
    // an odd number of 128-row blocks leaves the second CTA of the last pair without rows: only when that is a
    // small part of the work
    int64_t const blocks = (m + 127) / 128;
    if (blocks % 2 != 0 && blocks < 15) return false;
    int64_t const tiles = ((m + 255) / 256) * (n / 256);
    return tiles >= sms / 2;
}

// Whether a plain (no fused epilogue) dense call of this plan runs on the CTA-pair kernel: the shape must suit it and
// its rounds (256 wide on SMs / 2 pairs, about 4 % cheaper than the single-CTA kernel's) must not cost more than the
// plan's.
inline bool dense_takes_pair(int64_t m, int64_t n, int sms, DensePlan const& pl)
{
    if (!use_pair_kernel(m, n, sms, pl.swap, pl.splits)) return false;
    int const forced = forced_dense_tile();
    if (forced != 0) return forced == 2;
    double const cpair = schedule_rounds(((m + 255) / 256) * (n / 256), sms / 2) * 256.0 * 0.96;
    return cpair <= pl.cost;
}

inline int launch_dense_pair(const void* a, const void* sfa, const void* w, const void* sfw, void* d, int64_t m,
    int64_t n, int64_t k, int sms, cudaStream_t stream)
{
    CUtensorMap ta, tb, tsa, tsb;
    int rc;
    int64_t const kb = k / 128;
    if ((rc = make_operand_map(&ta, a, m, k, 128)) != 0) return rc;
    if ((rc = make_operand_map(&tb, w, n, k, 128)) != 0) return rc;
    if ((rc = make_sf_map(&tsa, sfa, (m + 127) / 128 * kb)) != 0) return rc;
    if ((rc = make_sf_map(&tsb, sfw, n / 128 * kb)) != 0) return rc;
    GemmParams p{};
    p.out = d;
    p.rows_a = static_cast<int>(m);
    p.rows_b = static_cast<int>(n);
    p.kb_total = static_cast<int>(kb);
    p.kb_per_split = p.kb_total;
    p.splits = 1;
    p.tiles_a = static_cast<int>((m + 255) / 256);
    p.tiles_b = static_cast<int>(n / 256);
    p.group_a = p.tiles_a < 8 ? p.tiles_a : 8;
    p.ldo = static_cast<int>(n);
    p.out_rows = m;
    p.out_align32 = (reinterpret_cast<uintptr_t>(d) & 31u) == 0 ? 1 : 0;
    int64_t const tiles = static_cast<int64_t>(p.tiles_a) * p.tiles_b;
    int const pairs = static_cast<int>(tiles < sms / 2 ? tiles : sms / 2);
    static std::atomic<uint64_t> done{0};
    rc = ensure_smem_attr(gemm_mxf8_pair_kernel, Gemm2Cfg::kSmemBytes, done);
    if (rc != 0) return rc;
    static std::atomic<int> printed{0};
    print_tile_info_once(printed, "gemm_mxf8_pair_kernel (per CTA of the pair)", Gemm2Cfg::kBM, Gemm2Cfg::kBN, EPI_BF16,
        false, false, false, Gemm2Cfg::kStages, Gemm2Cfg::kSmemBytes, Gemm2Cfg::kThreads, Gemm2Cfg::kTmemCols);
    gemm_mxf8_pair_kernel<<<2 * pairs, Gemm2Cfg::kThreads, Gemm2Cfg::kSmemBytes, stream>>>(ta, tb, tsa, tsb, p);
    return launch_status("gemm_mxf8_pair_kernel");
}

// FSO_B200_SPLITK=workspace keeps the two-launch split-K (fp32 partials + reduce kernel) for the decode shapes too;
// both forms give the same bytes.
inline bool splitk_through_workspace()
{
    static int const v = [] {
        const char* e = getenv("FSO_B200_SPLITK");
        return (e != nullptr && strcmp(e, "workspace") == 0) ? 1 : 0;
    }();
    return v != 0;
}

// D[M, N] = A[M, K] * W[N, K]^T.
// The dense epilogue of one call: out = bf16(act(acc + bias[n]) + residual[m, n]); all absent = the plain GEMM.
struct DenseEpi {
    const void* bias = nullptr;
    const void* residual = nullptr;
    int act = 0;
    void* quant_sf = nullptr;        // set: the output leaves as e4m3 codes (d) + these scale words (EPI_QUANT)
    bool any() const { return bias != nullptr || residual != nullptr || act != 0; }
};

// The quantizing epilogue serves the shapes that run in the normal orientation without split-K (every other shape
// computes bf16 first and runs the activation quantizer behind it, which gives the same bytes).
inline bool dense_fuses_quantized_output(int64_t m, int64_t n, int64_t k, int sms)
{
    DensePlan const pl = plan_dense(m, n, k, sms);
    return !pl.swap && pl.splits == 1;
}

inline int launch_dense(const void* a, const void* sfa, const void* w, const void* sfw, void* d, int64_t m, int64_t n,
    int64_t k, void* ws, int64_t ws_bytes, cudaStream_t stream, DenseEpi epi = DenseEpi{})
{
    int const sms = sm_count();
    DensePlan const pl = plan_dense(m, n, k, sms);
    if (pl.ws_bytes > 0 && (ws == nullptr || ws_bytes < pl.ws_bytes)) {
        set_error("fso_gemm_mxfp8: this shape takes the split-K route and needs a workspace of %lld bytes "
                  "(fso_gemm_mxfp8_ws_bytes), got %lld", static_cast<long long>(pl.ws_bytes),
            static_cast<long long>(ws_bytes));
        return FSO_ERR_INVALID;
    }
    bool const fused = epi.any();
    bool const quant = epi.quant_sf != nullptr;
    if (quant && (pl.swap || pl.splits != 1)) {
        set_error("fso_gemm_mxfp8_quantized: M = %lld, N = %lld, K = %lld does not take the fused form "
                  "(fso_gemm_mxfp8_fuses_quantized_output)", static_cast<long long>(m), static_cast<long long>(n),
            static_cast<long long>(k));
        return FSO_ERR_UNSUPPORTED;
    }
    if (!fused && !quant && dense_takes_pair(m, n, sms, pl))
        return launch_dense_pair(a, sfa, w, sfw, d, m, n, k, sms, stream);
    CUtensorMap ta, tb;
    GemmParams p{};
    p.kb_total = static_cast<int>(k / 128);
    p.kb_per_split = pl.kb_per_split;
    p.splits = pl.splits;
    p.tiles_a = pl.tiles_a;
    p.tiles_b = pl.tiles_b;
    p.group_a = pl.group_a;
    p.ldo = static_cast<int>(n);
    p.out = d;
    p.out_sf = static_cast<uint32_t*>(epi.quant_sf);
    p.ws = static_cast<float*>(ws);
    p.out_rows = m;
    p.out_align32 = (reinterpret_cast<uintptr_t>(d) & 31u) == 0 ? 1 : 0;
    p.bias = static_cast<const __nv_bfloat16*>(epi.bias);
    p.residual = static_cast<const __nv_bfloat16*>(epi.residual);
    p.act = epi.act;
    int rc;
    if (pl.swap) {
        if ((rc = make_operand_map(&ta, w, n, k, 128)) != 0) return rc;
        if ((rc = make_operand_map(&tb, a, m, k, pl.bn)) != 0) return rc;
        p.sfa = static_cast<const uint8_t*>(sfw);
        p.sfb = static_cast<const uint8_t*>(sfa);
        p.rows_a = static_cast<int>(n);
        p.rows_b = static_cast<int>(m);
    } else {
        if ((rc = make_operand_map(&ta, a, m, k, 128)) != 0) return rc;
        if ((rc = make_operand_map(&tb, w, n, k, pl.bn)) != 0) return rc;
        p.sfa = static_cast<const uint8_t*>(sfa);
        p.sfb = static_cast<const uint8_t*>(sfw);
        p.rows_a = static_cast<int>(m);
        p.rows_b = static_cast<int>(n);
    }
    // Decode-sized problems sum their K slices inside clusters (one launch, no workspace traffic) when all the
    // clusters run at the same time: take the largest slice count <= the planned one whose clusters all fit.
    int splits = pl.splits;
    bool in_cluster = false;
    if (pl.swap && pl.splits > 1) {
        int const tiles = pl.tiles_a * pl.tiles_b;
        for (int s2 = pl.splits; s2 >= 2; --s2) {
            int const per = (p.kb_total + s2 - 1) / s2;
            if ((p.kb_total + per - 1) / per != s2) continue;
            // the occupancy query counts one CTA of a cluster per SM; two of these half-SM CTAs share one
            if (2 * cluster_capacity_bn(pl.bn, s2, fused) >= tiles) {
                if (s2 == pl.splits || tiles * s2 * 2 >= sms) {
                    splits = s2;
                    in_cluster = true;
                }
                break;
            }
        }
    }
    p.splits = splits;
    p.kb_per_split = (p.kb_total + splits - 1) / splits;
    int64_t const items = static_cast<int64_t>(pl.tiles_a) * pl.tiles_b * splits;
    int const slots = pl.swap ? 2 * sms : sms;          // the swapped kernels run two CTAs per SM
    int const grid = static_cast<int>(items < slots ? items : slots);
    if (in_cluster && !splitk_through_workspace()) {
        if (fused)
            return pl.bn == 16 ? launch_gemm_cluster<16, true>(ta, tb, p, static_cast<int>(items), stream)
                : pl.bn == 32 ? launch_gemm_cluster<32, true>(ta, tb, p, static_cast<int>(items), stream)
                              : launch_gemm_cluster<64, true>(ta, tb, p, static_cast<int>(items), stream);
        return pl.bn == 16 ? launch_gemm_cluster<16>(ta, tb, p, static_cast<int>(items), stream)
            : pl.bn == 32 ? launch_gemm_cluster<32>(ta, tb, p, static_cast<int>(items), stream)
                          : launch_gemm_cluster<64>(ta, tb, p, static_cast<int>(items), stream);
    }
    bool const partial = splits > 1;
    if (quant) {
        if (pl.bn == 256)
            return fused ? launch_gemm_inst<256, EPI_QUANT, false, false, true>(ta, tb, p, grid, stream)
                         : launch_gemm_inst<256, EPI_QUANT, false, false>(ta, tb, p, grid, stream);
        return fused ? launch_gemm_inst<128, EPI_QUANT, false, false, true>(ta, tb, p, grid, stream)
                     : launch_gemm_inst<128, EPI_QUANT, false, false>(ta, tb, p, grid, stream);
    }
#define FSO_DENSE_CASE(BN_, SWAP_)                                                                                 \
    if (pl.bn == BN_ && pl.swap == SWAP_) {                                                                        \
        rc = partial ? launch_gemm_inst<BN_, EPI_PARTIAL, SWAP_, false>(ta, tb, p, grid, stream)                   \
            : fused  ? launch_gemm_inst<BN_, EPI_BF16, SWAP_, false, true>(ta, tb, p, grid, stream)                \
                     : launch_gemm_inst<BN_, EPI_BF16, SWAP_, false>(ta, tb, p, grid, stream);                     \
    } else
    FSO_DENSE_CASE(16, true)
    FSO_DENSE_CASE(32, true)
    FSO_DENSE_CASE(64, true)
    FSO_DENSE_CASE(128, false)
    FSO_DENSE_CASE(256, false)
    {
        set_error("fso_gemm_mxfp8: no kernel for tile %d (swap %d)", pl.bn, static_cast<int>(pl.swap));
        return FSO_ERR_INTERNAL;
    }
#undef FSO_DENSE_CASE
    if (rc != 0) return rc;
    if (partial) {
        int64_t const quads = m * n / 4;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>((quads + 255) / 256), 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        cfg.attrs = attr;
        cfg.numAttrs = pl.swap ? pdl_attribute(&attr[0]) : 0;
        FSO_CUDA(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, static_cast<const float4*>(ws), static_cast<uint2*>(d),
            quads, splits, static_cast<int>(n), p.bias, p.residual, p.act));
        rc = launch_status("splitk_reduce_kernel");
    }
    return rc;
}

// The gate_up projection of a dense SwiGLU MLP with the activation fused: w is [2I, K] with its rows interleaved
// (gate_j, up_j adjacent), out = silu(gate) * up as e4m3 [M, I] + scale words: the grouped FC1 epilogue on a dense
// operand. Always the normal orientation (the epilogue needs a row's gate / up pairs in one thread).
inline int launch_dense_swiglu(const void* a, const void* sfa, const void* w, const void* sfw, void* dq, void* sd,
    int64_t m, int64_t two_i, int64_t k, cudaStream_t stream)
{
    int const sms = sm_count();
    CUtensorMap ta, tb;
    int rc;
    if ((rc = make_operand_map(&ta, a, m, k, 128)) != 0) return rc;
    if ((rc = make_operand_map(&tb, w, two_i, k, 256)) != 0) return rc;
    GemmParams p{};
    p.sfa = static_cast<const uint8_t*>(sfa);
    p.sfb = static_cast<const uint8_t*>(sfw);
    p.out = dq;
    p.out_sf = static_cast<uint32_t*>(sd);
    p.rows_a = static_cast<int>(m);
    p.rows_b = static_cast<int>(two_i);
    p.kb_total = static_cast<int>(k / 128);
    p.kb_per_split = p.kb_total;
    p.splits = 1;
    p.tiles_a = static_cast<int>((m + 127) / 128);
    p.tiles_b = static_cast<int>(two_i / 256);
    p.ldo = static_cast<int>(two_i / 2);
    p.group_a = p.tiles_a < 16 ? p.tiles_a : 16;
    p.out_rows = m;
    p.out_align32 = (reinterpret_cast<uintptr_t>(dq) & 31u) == 0 ? 1 : 0;
    int64_t const items = static_cast<int64_t>(p.tiles_a) * p.tiles_b;
    int const grid = static_cast<int>(items < sms ? items : sms);
    return launch_gemm_inst<256, EPI_SWIGLU, false, false>(ta, tb, p, grid, stream);
}

// FSO_B200_MOE_SPARSE_RASTER=0 keeps the 16-block walk and unhinted loads for every grouped call (measurement).
inline bool grouped_sparse_rules()
{
    static int const v = [] {
        const char* e = getenv("FSO_B200_MOE_SPARSE_RASTER");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    return v != 0;
}

// Grouped GEMM over the compact activation: block b (rows [128b, 128b+128) of `a`) times weight[blk_expert[b]]^T.
// weight is [E, n_w, k] contiguous, its scale words one atom slab of n_w * k/128 words per expert.
// swiglu: n_w = 2I interleaved gate/up rows, out = e4m3 [rows, I] with scale words out_sf; otherwise out = bf16
// [rows, n_w].
inline int launch_grouped(const void* a, const void* sfa, const void* weight, const void* sfw, const int32_t* blk0,
    const int32_t* blk_expert, int64_t num_experts, int64_t n_w, int64_t k, int64_t num_blocks, int64_t rows,
    void* out, void* out_sf, bool swiglu, cudaStream_t stream)
{
    int const sms = sm_count();
    int const bn = (n_w % 256 == 0) ? 256 : 128;
    if (swiglu && bn != 256) {
        set_error("fso_moe_fc1_swiglu: 2*I must be a multiple of 256");
        return FSO_ERR_INVALID;
    }
    CUtensorMap ta, tb;
    int rc;
    if ((rc = make_operand_map(&ta, a, rows, k, 128)) != 0) return rc;
    if ((rc = make_operand_map(&tb, weight, num_experts * n_w, k, bn)) != 0) return rc;
    GemmParams p{};
    p.sfa = static_cast<const uint8_t*>(sfa);
    p.sfb = static_cast<const uint8_t*>(sfw);
    p.out = out;
    p.out_sf = static_cast<uint32_t*>(out_sf);
    p.blk0 = blk0;
    p.blk_expert = blk_expert;
    p.rows_a = static_cast<int>(rows);
    p.rows_b = static_cast<int>(n_w);
    p.kb_total = static_cast<int>(k / 128);
    p.kb_per_split = p.kb_total;
    p.splits = 1;
    p.tiles_a = static_cast<int>(num_blocks);
    p.tiles_b = static_cast<int>(n_w / bn);
    p.ldo = swiglu ? static_cast<int>(n_w / 2) : static_cast<int>(n_w);
    p.num_experts = static_cast<int>(num_experts);
    // Raster. Many rows per expert (16 blocks walked before the weight tile advances): the blocks of one expert
    // share each weight tile while it is in L2. At most 128 rows per expert on average (num_blocks is the bound
    // ceil((pairs + 127 E) / 128), so the call's pairs follow from it): nothing shares a weight tile but a spilled
    // second block, and the walk is sized so that all weight tiles of a block run in one round of the grid and the
    // block's activation rows are read from memory once. Measured on the DeepSeek-V3 layer at 4096 tokens: FC1
    // 1464 -> 1409-1445 us, FC2 904-921 -> 887-892 us.
    int64_t const pairs_bound = 128 * num_blocks - 127 * num_experts;
    bool const sparse = grouped_sparse_rules() && pairs_bound <= 128 * num_experts && p.tiles_b <= sms;
    p.group_a = sparse ? std::max(1, sms / p.tiles_b) : 16;
    p.stream_b_hint = sparse ? 1 : 0;
    p.out_rows = rows;
    p.out_align32 = (reinterpret_cast<uintptr_t>(out) & 31u) == 0 ? 1 : 0;
    int64_t const items = static_cast<int64_t>(p.tiles_a) * p.tiles_b;
    int const grid = static_cast<int>(items < sms ? items : sms);
    if (swiglu) return launch_gemm_inst<256, EPI_SWIGLU, false, true>(ta, tb, p, grid, stream);
    if (bn == 256) return launch_gemm_inst<256, EPI_BF16, false, true>(ta, tb, p, grid, stream);
    return launch_gemm_inst<128, EPI_BF16, false, true>(ta, tb, p, grid, stream);
}

// The grouped GEMM of the MoE layer's decode band (at most 64 tokens): weight rows on MMA-M, the routed rows of one
// 128-row block of the compact activation on MMA-N in tiles of 32 / 64, one tile per (block in use, 128 weight rows,
// sub-tile); out = [rows, n_w], fp32 for FC1 (the interleaved gate / up accumulators, which the activation kernel
// behind it reads unrounded) and bf16 for FC2 (the down projection). With few
// experts in use and a long K the K blocks of a tile are split over the CTAs of a cluster (one launch, summed in
// slice order through distributed shared memory), otherwise persistent half-SM CTAs walk the tiles.
// `pairs` = tokens * top-k of the call: with the shapes it fixes every host decision (capturable, no device read).
inline int launch_grouped_swap(const void* a, const void* sfa, const void* weight, const void* sfw,
    const int32_t* masked_m, const int32_t* blk0, const int32_t* blk_expert, int64_t num_experts, int64_t n_w, int64_t k,
    int64_t num_blocks, int64_t rows, void* out, bool out_f32, int64_t tokens, int64_t pairs, cudaStream_t stream)
{
    int const sms = sm_count();
    int const bn = tokens <= 32 ? 32 : 64;
    CUtensorMap ta, tb;
    int rc;
    if ((rc = make_operand_map(&ta, weight, num_experts * n_w, k, 128)) != 0) return rc;
    if ((rc = make_operand_map(&tb, a, rows, k, bn)) != 0) return rc;
    GemmParams p{};
    p.sfa = static_cast<const uint8_t*>(sfw);
    p.sfb = static_cast<const uint8_t*>(sfa);
    p.out = out;
    p.blk0 = blk0;
    p.blk_expert = blk_expert;
    p.masked_m = masked_m;
    p.rows_a = static_cast<int>(n_w);
    p.rows_b = static_cast<int>(rows);
    p.kb_total = static_cast<int>(k / 128);
    p.tiles_a = static_cast<int>(n_w / 128);
    p.tiles_b = static_cast<int>(num_blocks);
    // token sub-tiles of a 128-row block that can hold rows at all: an expert has at most `pairs` rows, so with a
    // handful of tokens only the first sub-tile exists and the tile space (the grid of the one-shot form) shrinks
    int64_t const subs_needed = ((pairs < 128 ? pairs : 128) + bn - 1) / bn;
    p.subs = static_cast<int>(subs_needed < 1 ? 1 : subs_needed);
    p.ldo = static_cast<int>(n_w);
    p.num_experts = static_cast<int>(num_experts);
    p.group_a = 1;
    p.out_rows = rows;
    p.out_f32 = out_f32 ? 1 : 0;
    // expected live tiles: one block per expert in use (an expert holds at most `tokens` <= 64 rows when a token
    // names an expert once), every weight panel of it
    int64_t const live_experts = pairs < num_experts ? pairs : num_experts;
    int64_t const live_tiles = live_experts * p.tiles_a;
    int splits = 1, kb_per = p.kb_total;
    pick_decode_splits(live_tiles, p.kb_total, cluster_split_limit(bn), &splits, &kb_per);
    p.splits = splits;
    p.kb_per_split = kb_per;
    int64_t const bound = num_blocks * p.tiles_a * p.subs * splits;      // every tile a routing could make live
    if (bound >= (1ll << 30)) {
        set_error("fso_moe_grouped_gemm_decode: the tile space is beyond the kernel's index range");
        return FSO_ERR_INVALID;
    }
    if (splits > 1) {
        return bn == 32 ? launch_gemm_cluster<32, false, true>(ta, tb, p, static_cast<int>(bound), stream)
                        : launch_gemm_cluster<64, false, true>(ta, tb, p, static_cast<int>(bound), stream);
    }
    int const grid = static_cast<int>(bound < 2 * sms ? bound : 2 * sms);
    return bn == 32 ? launch_gemm_inst<32, EPI_BF16, true, true>(ta, tb, p, grid, stream)
                    : launch_gemm_inst<64, EPI_BF16, true, true>(ta, tb, p, grid, stream);
}

}  // namespace fso

