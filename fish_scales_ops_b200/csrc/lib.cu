// The one translation unit of libfso_b200.so: kernels (included headers) and the extern "C" entry points declared
// in include/fso_b200.h. Nothing here allocates device memory or synchronizes, except fso_b200_device_status.
#include <cstdarg>

#include "common.cuh"

namespace fso {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

int current_device()
{
    int dev = 0;
    cudaGetDevice(&dev);
    return dev;
}

int sm_count()
{
    static int cached[64] = {0};
    int const dev = current_device() & 63;
    if (cached[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = n > 0 ? n : 1;
    }
    return cached[dev];
}

}  // namespace fso

#include "gemm_host.cuh"
#include "moe.cuh"
#include "exchange.cuh"
#include "router.cuh"

using namespace fso;

static inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" {

int fso_b200_version(void) { return 1; }

const char* fso_b200_last_error(void) { return t_error; }

int fso_b200_device_status(int* status)
{
    FSO_REQUIRE(status != nullptr, "fso_b200_device_status: status is NULL");
    int v = 0;
    FSO_CUDA(cudaDeviceSynchronize());
    FSO_CUDA(cudaMemcpyFromSymbol(&v, g_dev_status, sizeof(int)));
    if (v != 0) {
        int const zero = 0;
        FSO_CUDA(cudaMemcpyToSymbol(g_dev_status, &zero, sizeof(int)));
    }
    *status = v;
    return 0;
}

// Self-test of the bounded waits: one thread waits on an mbarrier that nothing ever arrives at, for at most
// `limit_cycles` SM cycles, then records FSO_DEV_SELFTEST_WAIT in the device status word and returns, exactly as a
// wait of the GEMM kernels does when it runs out. Nothing can hang: the wait ends by itself.
__global__ void selftest_wait_kernel(long long limit_cycles)
{
    __shared__ __align__(8) unsigned long long bar;
    uint32_t const b = smem_u32(&bar);
    mbar_init(b, 1);
    mbar_fence_init();
    long long const t0 = clock64();
    bool done = false;
    while (!done && clock64() - t0 <= limit_cycles) done = mbar_try_wait(b, 0);
    if (!done) atomicCAS(&g_dev_status, 0, FSO_DEV_SELFTEST_WAIT);
}

int fso_b200_selftest_wait_expires(int64_t limit_cycles, void* stream)
{
    FSO_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000ll,
        "fso_b200_selftest_wait_expires: limit_cycles must be in (0, 2e9] (about a second of SM clock at most)");
    selftest_wait_kernel<<<1, 1, 0, as_stream(stream)>>>(static_cast<long long>(limit_cycles));
    return launch_status("selftest_wait_kernel");
}

int fso_quantize_1x32(const void* x, void* xq, void* sf, int64_t m, int64_t k, int64_t interleave_i, void* stream)
{
    FSO_REQUIRE(m >= 0 && k > 0 && k % 128 == 0, "fso_quantize_1x32: K = %lld must be a positive multiple of 128",
        static_cast<long long>(k));
    if (m == 0) return 0;
    FSO_REQUIRE(x && xq && sf, "fso_quantize_1x32: NULL pointer");
    FSO_REQUIRE(aligned16(x) && aligned16(xq) && (reinterpret_cast<uintptr_t>(sf) & 3u) == 0,
        "fso_quantize_1x32: x and xq must be 16-byte aligned and sf 4-byte aligned");
    FSO_REQUIRE(interleave_i >= 0 && (interleave_i == 0 || m % (2 * interleave_i) == 0),
        "fso_quantize_1x32: with interleave_i = %lld the row count %lld must be a multiple of 2*I",
        static_cast<long long>(interleave_i), static_cast<long long>(m));
    return launch_quantize_1x32(x, xq, sf, m, k, interleave_i, as_stream(stream));
}

int fso_quantize_activation_1x32(const void* x, void* xq, void* sf, int64_t m, int64_t k, void* stream)
{
    FSO_REQUIRE(m >= 0 && k > 0 && k % 128 == 0, "fso_quantize_activation_1x32: K = %lld must be a positive multiple of 128",
        static_cast<long long>(k));
    if (m == 0) return 0;
    FSO_REQUIRE(x && xq && sf, "fso_quantize_activation_1x32: NULL pointer");
    FSO_REQUIRE(aligned16(x) && aligned16(xq) && (reinterpret_cast<uintptr_t>(sf) & 3u) == 0,
        "fso_quantize_activation_1x32: x and xq must be 16-byte aligned and sf 4-byte aligned");
    return launch_quantize_1x32(x, xq, sf, m, k, 0, as_stream(stream), true);
}

int fso_silu_mul_quantize_1x32(const void* gu, void* xq, void* sf, int64_t m, int64_t inter, void* stream)
{
    FSO_REQUIRE(m >= 0 && inter > 0 && inter % 128 == 0,
        "fso_silu_mul_quantize_1x32: INTER = %lld must be a positive multiple of 128", static_cast<long long>(inter));
    if (m == 0) return 0;
    FSO_REQUIRE(gu && xq && sf, "fso_silu_mul_quantize_1x32: NULL pointer");
    FSO_REQUIRE((reinterpret_cast<uintptr_t>(gu) & 31u) == 0 && aligned16(xq) && (reinterpret_cast<uintptr_t>(sf) & 3u) == 0,
        "fso_silu_mul_quantize_1x32: gu must be 32-byte aligned, xq 16-byte aligned and sf 4-byte aligned");
    return launch_silu_mul_quantize(gu, xq, sf, m, inter, as_stream(stream));
}

__global__ void stream_fence_kernel() {}

int fso_stream_fence(void* stream)
{
    stream_fence_kernel<<<1, 1, 0, as_stream(stream)>>>();
    return launch_status("stream_fence_kernel");
}

int fso_requant_bs128_to_mx(const void* wq, const float* s128, void* out_q, void* out_sf, int64_t n, int64_t k,
    int64_t interleave_i, void* stream)
{
    FSO_REQUIRE(n > 0 && k > 0 && n % 128 == 0 && k % 128 == 0,
        "fso_requant_bs128_to_mx: N = %lld and K = %lld must be positive multiples of 128", static_cast<long long>(n),
        static_cast<long long>(k));
    FSO_REQUIRE(wq && s128 && out_q && out_sf, "fso_requant_bs128_to_mx: NULL pointer");
    FSO_REQUIRE(aligned16(wq) && aligned16(out_q) && (reinterpret_cast<uintptr_t>(out_sf) & 3u) == 0
            && (reinterpret_cast<uintptr_t>(s128) & 3u) == 0,
        "fso_requant_bs128_to_mx: wq and out_q must be 16-byte aligned, s128 and out_sf 4-byte aligned");
    FSO_REQUIRE(interleave_i >= 0 && (interleave_i == 0 || (n % (2 * interleave_i) == 0 && interleave_i % 128 == 0)),
        "fso_requant_bs128_to_mx: with interleave_i = %lld, N must be a multiple of 2*I and I a multiple of 128",
        static_cast<long long>(interleave_i));
    return launch_requant_bs128(wq, s128, out_q, out_sf, n, k, interleave_i, as_stream(stream));
}

int fso_pack_ue8m0(const void* sf_u8, void* out_sf, int64_t g, int64_t n, int64_t k, int64_t interleave_i,
    void* stream)
{
    FSO_REQUIRE(g > 0 && n > 0 && k > 0 && k % 128 == 0, "fso_pack_ue8m0: G, N positive and K a multiple of 128");
    FSO_REQUIRE(sf_u8 && out_sf && (reinterpret_cast<uintptr_t>(out_sf) & 3u) == 0,
        "fso_pack_ue8m0: NULL pointer or out_sf not 4-byte aligned");
    FSO_REQUIRE(interleave_i >= 0 && (interleave_i == 0 || n == 2 * interleave_i),
        "fso_pack_ue8m0: with interleave_i the row count per group must be 2*I");
    return launch_pack_ue8m0(sf_u8, out_sf, g, n, k, interleave_i, as_stream(stream));
}

static int check_gemm_shape(const char* op, int64_t m, int64_t n, int64_t k)
{
    FSO_REQUIRE(m >= 0 && n > 0 && k > 0, "%s: M >= 0, N > 0, K > 0 required", op);
    FSO_REQUIRE(n % 128 == 0 && k % 128 == 0, "%s: N = %lld and K = %lld must be multiples of 128", op,
        static_cast<long long>(n), static_cast<long long>(k));
    FSO_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), "%s: dimension too large", op);
    return 0;
}

int fso_gemm_mxfp8_ws_bytes(int64_t m, int64_t n, int64_t k, int64_t* bytes)
{
    FSO_REQUIRE(bytes != nullptr, "fso_gemm_mxfp8_ws_bytes: bytes is NULL");
    int const rc = check_gemm_shape("fso_gemm_mxfp8_ws_bytes", m, n, k);
    if (rc != 0) return rc;
    *bytes = m == 0 ? 0 : plan_dense(m, n, k, sm_count()).ws_bytes;
    return 0;
}

int fso_gemm_mxfp8_describe(int64_t m, int64_t n, int64_t k, int64_t sm_count_or_0, int32_t* out6)
{
    FSO_REQUIRE(out6 != nullptr, "fso_gemm_mxfp8_describe: out6 is NULL");
    FSO_REQUIRE(sm_count_or_0 >= 0 && sm_count_or_0 <= 4096, "fso_gemm_mxfp8_describe: sm_count_or_0 = %lld",
        static_cast<long long>(sm_count_or_0));
    int const rc = check_gemm_shape("fso_gemm_mxfp8_describe", m, n, k);
    if (rc != 0) return rc;
    for (int i = 0; i < 6; ++i) out6[i] = 0;
    if (m == 0) return 0;
    int const sms = sm_count_or_0 > 0 ? static_cast<int>(sm_count_or_0) : sm_count();
    DensePlan const pl = plan_dense(m, n, k, sms);
    bool const pair = dense_takes_pair(m, n, sms, pl);
    out6[0] = pl.swap ? 1 : 0;
    out6[1] = pair ? 256 : pl.bn;
    out6[2] = pl.splits;
    out6[3] = pl.kb_per_split;
    out6[4] = pair ? 1 : 0;
    out6[5] = pair ? static_cast<int32_t>(((m + 255) / 256) * (n / 256)) : pl.tiles_a * pl.tiles_b;
    return 0;
}

int fso_gemm_mxfp8(const void* a, const void* sfa, const void* w, const void* sfw, void* d, int64_t m, int64_t n,
    int64_t k, void* ws, int64_t ws_bytes, void* stream)
{
    int const rc = check_gemm_shape("fso_gemm_mxfp8", m, n, k);
    if (rc != 0) return rc;
    if (m == 0) return 0;
    FSO_REQUIRE(a && sfa && w && sfw && d, "fso_gemm_mxfp8: NULL pointer");
    FSO_REQUIRE(aligned16(a) && aligned16(sfa) && aligned16(w) && aligned16(sfw) && aligned16(d),
        "fso_gemm_mxfp8: every operand must be 16-byte aligned (TMA reads them in place)");
    FSO_REQUIRE(ws == nullptr || aligned16(ws), "fso_gemm_mxfp8: the workspace must be 16-byte aligned");
    return launch_dense(a, sfa, w, sfw, d, m, n, k, ws, ws_bytes, as_stream(stream));
}

int fso_gemm_mxfp8_epilogue(const void* a, const void* sfa, const void* w, const void* sfw, void* d, int64_t m,
    int64_t n, int64_t k, const void* bias, const void* residual, int64_t activation, void* ws, int64_t ws_bytes,
    void* stream)
{
    int const rc = check_gemm_shape("fso_gemm_mxfp8_epilogue", m, n, k);
    if (rc != 0) return rc;
    FSO_REQUIRE(activation == 0 || activation == 1,
        "fso_gemm_mxfp8_epilogue: activation must be 0 (identity) or 1 (erf-GELU), got %lld",
        static_cast<long long>(activation));
    if (m == 0) return 0;
    FSO_REQUIRE(a && sfa && w && sfw && d, "fso_gemm_mxfp8_epilogue: NULL pointer");
    FSO_REQUIRE(aligned16(a) && aligned16(sfa) && aligned16(w) && aligned16(sfw) && aligned16(d),
        "fso_gemm_mxfp8_epilogue: every operand must be 16-byte aligned (TMA reads them in place)");
    FSO_REQUIRE(ws == nullptr || aligned16(ws), "fso_gemm_mxfp8_epilogue: the workspace must be 16-byte aligned");
    FSO_REQUIRE((bias == nullptr || aligned16(bias)) && (residual == nullptr || aligned16(residual)),
        "fso_gemm_mxfp8_epilogue: bias and residual must be 16-byte aligned");
    DenseEpi epi;
    epi.bias = bias;
    epi.residual = residual;
    epi.act = static_cast<int>(activation);
    return launch_dense(a, sfa, w, sfw, d, m, n, k, ws, ws_bytes, as_stream(stream), epi);
}

int fso_gemm_mxfp8_fuses_quantized_output(int64_t m, int64_t n, int64_t k, int* yes)
{
    FSO_REQUIRE(yes != nullptr, "fso_gemm_mxfp8_fuses_quantized_output: yes is NULL");
    int const rc = check_gemm_shape("fso_gemm_mxfp8_fuses_quantized_output", m, n, k);
    if (rc != 0) return rc;
    *yes = (m > 0 && dense_fuses_quantized_output(m, n, k, sm_count())) ? 1 : 0;
    return 0;
}

int fso_gemm_mxfp8_quantized(const void* a, const void* sfa, const void* w, const void* sfw, void* out_q, void* out_sf,
    int64_t m, int64_t n, int64_t k, const void* bias, int64_t activation, void* stream)
{
    int const rc = check_gemm_shape("fso_gemm_mxfp8_quantized", m, n, k);
    if (rc != 0) return rc;
    FSO_REQUIRE(activation == 0 || activation == 1,
        "fso_gemm_mxfp8_quantized: activation must be 0 (identity) or 1 (erf-GELU), got %lld",
        static_cast<long long>(activation));
    if (m == 0) return 0;
    FSO_REQUIRE(a && sfa && w && sfw && out_q && out_sf, "fso_gemm_mxfp8_quantized: NULL pointer");
    FSO_REQUIRE(aligned16(a) && aligned16(sfa) && aligned16(w) && aligned16(sfw) && aligned16(out_q)
            && (reinterpret_cast<uintptr_t>(out_sf) & 3u) == 0 && (bias == nullptr || aligned16(bias)),
        "fso_gemm_mxfp8_quantized: operands, out_q and bias must be 16-byte aligned, out_sf 4-byte aligned");
    DenseEpi epi;
    epi.bias = bias;
    epi.act = static_cast<int>(activation);
    epi.quant_sf = out_sf;
    return launch_dense(a, sfa, w, sfw, out_q, m, n, k, nullptr, 0, as_stream(stream), epi);
}

int fso_gemm_mxfp8_swiglu(const void* a, const void* sfa, const void* w, const void* sfw, void* dq, void* sd, int64_t m,
    int64_t two_i, int64_t k, void* stream)
{
    int const rc = check_gemm_shape("fso_gemm_mxfp8_swiglu", m, two_i, k);
    if (rc != 0) return rc;
    FSO_REQUIRE(two_i % 256 == 0, "fso_gemm_mxfp8_swiglu: 2*I = %lld must be a multiple of 256",
        static_cast<long long>(two_i));
    if (m == 0) return 0;
    FSO_REQUIRE(a && sfa && w && sfw && dq && sd, "fso_gemm_mxfp8_swiglu: NULL pointer");
    FSO_REQUIRE(aligned16(a) && aligned16(sfa) && aligned16(w) && aligned16(sfw) && aligned16(dq)
            && (reinterpret_cast<uintptr_t>(sd) & 3u) == 0,
        "fso_gemm_mxfp8_swiglu: operands and dq must be 16-byte aligned, sd 4-byte aligned");
    return launch_dense_swiglu(a, sfa, w, sfw, dq, sd, m, two_i, k, as_stream(stream));
}

int fso_moe_plan_make(int64_t tokens, int64_t topk, int64_t num_experts, fso_moe_plan* plan)
{
    FSO_REQUIRE(plan != nullptr, "fso_moe_plan_make: plan is NULL");
    FSO_REQUIRE(tokens >= 0 && topk >= 1 && num_experts >= 1 && num_experts <= 1024,
        "fso_moe_plan_make: tokens >= 0, topk >= 1, 1 <= num_experts <= 1024 required");
    int64_t const pairs = tokens * topk;
    FSO_REQUIRE(pairs < (1ll << 24), "fso_moe_plan_make: tokens * topk = %lld is beyond the routing kernels' range",
        static_cast<long long>(pairs));
    int64_t const active = num_experts < pairs ? num_experts : pairs;
    int64_t nb = (pairs + 127 * active) / 128;
    if (nb < 1) nb = 1;
    plan->pairs = pairs;
    plan->num_blocks = nb;
    plan->rows = 128 * (nb + 1);
    plan->route_scratch_bytes = pairs > kRouteSeg ? ((pairs + kRouteSeg - 1) / kRouteSeg) * num_experts * 4 : 0;
    return 0;
}

// Shared memory of the routing kernels: 64 * E bytes of dynamic shared memory ([32 warps][E] uint16) on top of up to
// 8.3 KB of static arrays, which passes the 48 KB a kernel gets without opting in from E = 638 on. The opt-in is made
// once per device for the largest E the entry points accept, by the first routing call on that device whatever its
// size (so a small warm-up call prepares every later one; make it outside stream capture).
static int route_prepare_device()
{
    static std::atomic<uint64_t> done{0};
    int const dev = current_device();
    uint64_t const bit = 1ull << (dev & 63);
    if ((done.load(std::memory_order_acquire) & bit) == 0) {
        int const smem = 64 * 1024;
        FSO_CUDA(cudaFuncSetAttribute(route_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        FSO_CUDA(cudaFuncSetAttribute(route_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        FSO_CUDA(cudaFuncSetAttribute(route_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        done.fetch_or(bit, std::memory_order_release);
    }
    return 0;
}

static int launch_route(const int32_t* ids, int pairs, int e, int nb, int32_t* masked_m, int32_t* blk0,
    int32_t* slot_of_flat, int32_t* blk_expert, int32_t* seg, cudaStream_t st, const char* what)
{
    size_t const smem = static_cast<size_t>(64) * e;   // [32][E] uint16
    if (pairs <= kRouteSeg) {
        route_small_kernel<<<1, kRouteSeg, smem, st>>>(ids, pairs, e, nb, masked_m, blk0, slot_of_flat, blk_expert);
        return launch_status("route_small_kernel");
    }
    int const segs = (pairs + kRouteSeg - 1) / kRouteSeg;
    route_count_kernel<<<segs, kRouteSeg, smem, st>>>(ids, pairs, e, seg);
    route_scan_kernel<<<1, kRouteSeg, 0, st>>>(seg, segs, e, nb, masked_m, blk0, blk_expert);
    route_place_kernel<<<segs, kRouteSeg, smem, st>>>(ids, pairs, e, seg, blk0, slot_of_flat);
    return launch_status(what);
}

int fso_moe_route(const int32_t* ids, int64_t tokens, int64_t topk, int64_t num_experts, int64_t num_blocks,
    int32_t* masked_m, int32_t* blk0, int32_t* slot_of_flat, int32_t* blk_expert, void* scratch,
    int64_t scratch_bytes, void* stream)
{
    fso_moe_plan pl;
    int rc = fso_moe_plan_make(tokens, topk, num_experts, &pl);
    if (rc != 0) return rc;
    FSO_REQUIRE(num_blocks >= pl.num_blocks, "fso_moe_route: num_blocks = %lld is below the bound %lld of this call",
        static_cast<long long>(num_blocks), static_cast<long long>(pl.num_blocks));
    FSO_REQUIRE(masked_m && blk0 && blk_expert && (pl.pairs == 0 || (ids && slot_of_flat)), "fso_moe_route: NULL pointer");
    FSO_REQUIRE(pl.pairs <= kRouteSeg
            || (scratch != nullptr && scratch_bytes >= pl.route_scratch_bytes && (reinterpret_cast<uintptr_t>(scratch) & 3u) == 0),
        "fso_moe_route: this call needs %lld bytes of 4-byte aligned scratch", static_cast<long long>(pl.route_scratch_bytes));
    if ((rc = route_prepare_device()) != 0) return rc;
    return launch_route(ids, static_cast<int>(pl.pairs), static_cast<int>(num_experts), static_cast<int>(num_blocks),
        masked_m, blk0, slot_of_flat, blk_expert, static_cast<int32_t*>(scratch), as_stream(stream), "route kernels");
}

// ---------------------------------------------------------------------------------------------------------------
// Routing for callers that must not allocate.
//
// Some callers of this library cannot hand it scratch memory at the moment they need a routing: a serving engine
// that has given every free byte of the device to its own pool and forbids cudaMalloc in the forward pass, or a
// plugin that runs where an allocation would stall the stream. For them this entry point keeps the per-segment
// counts of the multi-segment routing in an array that is part of the library image itself (256 KiB, resident on
// every GPU that loads the library until the process exits). It calls no cudaMalloc / cudaFree and no allocating
// library routine; inputs and outputs are still the caller's.
//
// The array's name is only a host-side stand-in in host code, not a device address, so the device address is looked
// up once per device with cudaGetSymbolAddress (with that device current) and handed to the kernels. That lookup
// happens in the first call made on a device, whatever that call's size; make that first call outside any stream
// capture.
// Limits: tokens * topk <= kRouteStaticMaxPairs; larger calls are refused. The array is shared by every call and
// keeps the previous call's contents; the kernels overwrite every word they later read, so nothing needs clearing,
// but two calls that overlap on the GPU (different streams) race on it: serialize them.
constexpr int64_t kRouteStaticMaxPairs = 65536;
constexpr int64_t kRouteStaticWords = (kRouteStaticMaxPairs / kRouteSeg) * 1024;   // 64 segments x 1024 experts
static __device__ __align__(256) int32_t g_route_static_scratch[kRouteStaticWords];

static int route_static_scratch_ptr(int32_t** out)
{
    static std::mutex mu;
    static int32_t* ptrs[64] = {};
    int dev = 0;
    FSO_CUDA(cudaGetDevice(&dev));
    FSO_REQUIRE(dev >= 0 && dev < 64, "fso_moe_route_noalloc: device index %d is beyond the 64 this entry point tracks", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        FSO_CUDA(cudaGetSymbolAddress(&p, g_route_static_scratch));
        ptrs[dev] = static_cast<int32_t*>(p);
    }
    *out = ptrs[dev];
    return 0;
}

int fso_moe_route_noalloc(const int32_t* ids, int64_t tokens, int64_t topk, int64_t num_experts, int64_t num_blocks,
    int32_t* masked_m, int32_t* blk0, int32_t* slot_of_flat, int32_t* blk_expert, void* stream)
{
    fso_moe_plan pl;
    int rc = fso_moe_plan_make(tokens, topk, num_experts, &pl);
    if (rc != 0) return rc;
    FSO_REQUIRE(pl.pairs <= kRouteStaticMaxPairs,
        "fso_moe_route_noalloc: tokens * topk = %lld exceeds the %lld pairs its built-in scratch covers; use "
        "fso_moe_route with caller scratch", static_cast<long long>(pl.pairs), static_cast<long long>(kRouteStaticMaxPairs));
    FSO_REQUIRE(num_blocks >= pl.num_blocks, "fso_moe_route_noalloc: num_blocks = %lld is below the bound %lld of this call",
        static_cast<long long>(num_blocks), static_cast<long long>(pl.num_blocks));
    FSO_REQUIRE(masked_m && blk0 && blk_expert && (pl.pairs == 0 || (ids && slot_of_flat)),
        "fso_moe_route_noalloc: NULL pointer");
    // per-device set-up first, whatever the size of this call: the address of the built-in array and the routing
    // kernels' shared-memory opt-in, so that any first call on a device warms it for every later one
    int32_t* seg = nullptr;
    if ((rc = route_static_scratch_ptr(&seg)) != 0) return rc;
    if ((rc = route_prepare_device()) != 0) return rc;
    return launch_route(ids, static_cast<int>(pl.pairs), static_cast<int>(num_experts), static_cast<int>(num_blocks),
        masked_m, blk0, slot_of_flat, blk_expert, seg, as_stream(stream), "route kernels (built-in scratch)");
}

int fso_moe_gather_quant(const void* hidden, const int32_t* slot_of_flat, int64_t tokens, int64_t topk, int64_t h,
    int64_t rows, void* hq, void* sh, void* stream)
{
    FSO_REQUIRE(tokens >= 0 && topk >= 1 && h > 0 && h % 128 == 0 && rows > 0 && rows % 128 == 0,
        "fso_moe_gather_quant: H a multiple of 128 and rows a multiple of 128 required");
    if (tokens == 0) return 0;
    FSO_REQUIRE(hidden && slot_of_flat && hq && sh, "fso_moe_gather_quant: NULL pointer");
    FSO_REQUIRE(aligned16(hidden) && aligned16(hq) && (reinterpret_cast<uintptr_t>(sh) & 3u) == 0,
        "fso_moe_gather_quant: hidden and hq must be 16-byte aligned");
    constexpr int kUnroll = 2;
    int const kb = static_cast<int>(h / 128);
    FSO_REQUIRE(tokens * kb < (1ll << 31) - 4096, "fso_moe_gather_quant: tokens * H/128 is beyond the kernel's index range");
    if ((reinterpret_cast<uintptr_t>(hidden) & 31u) == 0) {
        int64_t const octs = (tokens * kb + kUnroll - 1) / kUnroll;
        gather_quant_wide_kernel<kUnroll><<<static_cast<unsigned>((octs * 8 + 255) / 256), 256, 0, as_stream(stream)>>>(
            static_cast<const uint8_t*>(hidden), slot_of_flat, tokens, static_cast<int>(topk), kb,
            static_cast<uint4*>(hq), static_cast<uint32_t*>(sh));
        return launch_status("gather_quant_wide_kernel");
    }
    int64_t const halves = (tokens * kb + kUnroll - 1) / kUnroll;
    int64_t const blocks = (halves * 16 + 255) / 256;
    gather_quant_kernel<kUnroll><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
        static_cast<const uint4*>(hidden), slot_of_flat, tokens, static_cast<int>(topk), kb, static_cast<uint2*>(hq),
        static_cast<uint32_t*>(sh));
    return launch_status("gather_quant_kernel");
}

static int check_grouped(const char* op, int64_t num_experts, int64_t h, int64_t inter, int64_t num_blocks, int64_t rows)
{
    FSO_REQUIRE(num_experts >= 1 && num_experts <= 1024 && h > 0 && inter > 0 && h % 128 == 0 && inter % 128 == 0,
        "%s: 1 <= E <= 1024 and H, I multiples of 128 required", op);
    FSO_REQUIRE(num_blocks >= 1 && rows >= 128 * num_blocks && rows % 128 == 0,
        "%s: rows = %lld must be a multiple of 128 covering num_blocks = %lld blocks", op, static_cast<long long>(rows),
        static_cast<long long>(num_blocks));
    FSO_REQUIRE(num_experts * 2 * inter < (1ll << 31) && rows < (1ll << 31), "%s: dimension too large", op);
    return 0;
}

int fso_moe_fc1_swiglu(const void* hq, const void* sh, const void* w13, const void* sw13, const int32_t* blk0,
    const int32_t* blk_expert, int64_t num_experts, int64_t h, int64_t inter, int64_t num_blocks, int64_t rows,
    void* dq, void* sd, void* stream)
{
    int const rc = check_grouped("fso_moe_fc1_swiglu", num_experts, h, inter, num_blocks, rows);
    if (rc != 0) return rc;
    FSO_REQUIRE(hq && sh && w13 && sw13 && blk0 && blk_expert && dq && sd, "fso_moe_fc1_swiglu: NULL pointer");
    FSO_REQUIRE(aligned16(hq) && aligned16(sh) && aligned16(w13) && aligned16(sw13) && aligned16(dq) && aligned16(sd),
        "fso_moe_fc1_swiglu: every operand must be 16-byte aligned");
    return launch_grouped(hq, sh, w13, sw13, blk0, blk_expert, num_experts, 2 * inter, h, num_blocks, rows, dq, sd, true,
        as_stream(stream));
}

int fso_moe_fc2(const void* dq, const void* sd, const void* w2, const void* sw2, const int32_t* blk0,
    const int32_t* blk_expert, int64_t num_experts, int64_t h, int64_t inter, int64_t num_blocks, int64_t rows,
    void* dn, void* stream)
{
    int const rc = check_grouped("fso_moe_fc2", num_experts, h, inter, num_blocks, rows);
    if (rc != 0) return rc;
    FSO_REQUIRE(dq && sd && w2 && sw2 && blk0 && blk_expert && dn, "fso_moe_fc2: NULL pointer");
    FSO_REQUIRE(aligned16(dq) && aligned16(sd) && aligned16(w2) && aligned16(sw2) && aligned16(dn),
        "fso_moe_fc2: every operand must be 16-byte aligned");
    return launch_grouped(dq, sd, w2, sw2, blk0, blk_expert, num_experts, h, inter, num_blocks, rows, dn, nullptr, false,
        as_stream(stream));
}

int fso_moe_grouped_gemm_decode(const void* act_q, const void* act_sf, const void* weight, const void* sfw,
    const int32_t* masked_m, const int32_t* blk0, const int32_t* blk_expert, int64_t num_experts, int64_t n_w, int64_t k,
    int64_t num_blocks, int64_t rows, void* out, int64_t out_is_f32, int64_t tokens, int64_t topk, void* stream)
{
    FSO_REQUIRE(num_experts >= 1 && num_experts <= 1024 && n_w > 0 && k > 0 && n_w % 128 == 0 && k % 128 == 0,
        "fso_moe_grouped_gemm_decode: 1 <= E <= 1024 and N_w, K multiples of 128 required");
    FSO_REQUIRE(num_blocks >= 1 && rows >= 128 * num_blocks && rows % 128 == 0,
        "fso_moe_grouped_gemm_decode: rows = %lld must be a multiple of 128 covering num_blocks = %lld blocks",
        static_cast<long long>(rows), static_cast<long long>(num_blocks));
    FSO_REQUIRE(tokens >= 1 && tokens <= 64 && topk >= 1,
        "fso_moe_grouped_gemm_decode: serves 1 to 64 tokens, got %lld (larger batches take fso_moe_fc1_swiglu / "
        "fso_moe_fc2)", static_cast<long long>(tokens));
    FSO_REQUIRE(num_experts * n_w < (1ll << 31) && rows < (1ll << 31), "fso_moe_grouped_gemm_decode: dimension too large");
    FSO_REQUIRE(act_q && act_sf && weight && sfw && masked_m && blk0 && blk_expert && out,
        "fso_moe_grouped_gemm_decode: NULL pointer");
    FSO_REQUIRE(aligned16(act_q) && aligned16(act_sf) && aligned16(weight) && aligned16(sfw) && aligned16(out),
        "fso_moe_grouped_gemm_decode: every operand must be 16-byte aligned");
    return launch_grouped_swap(act_q, act_sf, weight, sfw, masked_m, blk0, blk_expert, num_experts, n_w, k, num_blocks,
        rows, out, out_is_f32 != 0, tokens, tokens * topk, as_stream(stream));
}

int fso_moe_silu_mul_quantize_rows(const void* gu, const int32_t* masked_m, const int32_t* blk0,
    const int32_t* blk_expert, int64_t num_experts, int64_t rows, int64_t inter, void* dq, void* sd, void* stream)
{
    FSO_REQUIRE(num_experts >= 1 && rows > 0 && rows % 128 == 0 && inter > 0 && inter % 128 == 0,
        "fso_moe_silu_mul_quantize_rows: rows and I must be positive multiples of 128");
    FSO_REQUIRE(gu && masked_m && blk0 && blk_expert && dq && sd, "fso_moe_silu_mul_quantize_rows: NULL pointer");
    FSO_REQUIRE((reinterpret_cast<uintptr_t>(gu) & 31u) == 0 && aligned16(dq) && (reinterpret_cast<uintptr_t>(sd) & 3u) == 0,
        "fso_moe_silu_mul_quantize_rows: gu must be 32-byte aligned, dq 16-byte aligned and sd 4-byte aligned");
    return launch_silu_mul_quantize_rows(gu, dq, sd, masked_m, blk0, blk_expert, num_experts, rows, inter, as_stream(stream));
}

// A multiplier coprime to n (a prime that does not divide it): v -> (v * mul) mod n is then a permutation of [0, n).
static int64_t coprime_multiplier(int64_t n)
{
    for (int64_t p : {1000003ll, 999983ll, 7919ll, 104729ll})
        if (n % p != 0) return p;
    return 1;
}

static int launch_combine(const char* op, const void* dn, const int32_t* slot_of_flat, const float* topk_w,
    const void* bias, const float* bias_scale, void* out, int64_t tokens, int64_t topk, int64_t h, RowScatter sc,
    void* stream)
{
    int const h8 = static_cast<int>(h / 8);
    int64_t const total = tokens * h8;
    FSO_REQUIRE(total < (1ll << 31) - 4096, "%s: tokens * H/8 is beyond the kernel's index range", op);
    bool const wide_ok = ((reinterpret_cast<uintptr_t>(dn) | reinterpret_cast<uintptr_t>(out)
                              | reinterpret_cast<uintptr_t>(bias)) & 31u) == 0 && topk <= 8;
    int const groups = topk <= 2 ? 4 : topk <= 4 ? 2 : 1;
    if (wide_ok && h % (16 * groups) == 0) {
        int64_t const threads = tokens * (h / (16 * groups));
        unsigned const blocks = static_cast<unsigned>((threads + 255) / 256);
        auto* dnb = static_cast<const uint8_t*>(dn);
        auto* bb = static_cast<const uint8_t*>(bias);
        auto* ob = static_cast<uint8_t*>(out);
        int const hb = static_cast<int>(h * 2);
        if (groups == 4)
            combine_wide_kernel<2, 4><<<blocks, 256, 0, as_stream(stream)>>>(dnb, slot_of_flat, topk_w, bb, bias_scale, ob,
                tokens, static_cast<int>(topk), hb, sc);
        else if (topk <= 4)
            combine_wide_kernel<4, 2><<<blocks, 256, 0, as_stream(stream)>>>(dnb, slot_of_flat, topk_w, bb, bias_scale, ob,
                tokens, static_cast<int>(topk), hb, sc);
        else
            combine_wide_kernel<8, 1><<<blocks, 256, 0, as_stream(stream)>>>(dnb, slot_of_flat, topk_w, bb, bias_scale, ob,
                tokens, static_cast<int>(topk), hb, sc);
        return launch_status("combine_wide_kernel");
    }
    FSO_REQUIRE(sc.world == 0, "%s: needs 32-byte aligned rows, H a multiple of 64 and top-k <= 8", op);
    combine_kernel<8><<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(
        static_cast<const uint4*>(dn), slot_of_flat, topk_w, static_cast<const uint4*>(bias), bias_scale,
        static_cast<uint4*>(out), tokens, static_cast<int>(topk), h8);
    return launch_status("combine_kernel");
}

int fso_moe_combine(const void* dn, const int32_t* slot_of_flat, const float* topk_w, const void* bias,
    const float* bias_scale, void* out, int64_t tokens, int64_t topk, int64_t h, void* stream)
{
    FSO_REQUIRE(tokens >= 0 && topk >= 1 && h > 0 && h % 8 == 0, "fso_moe_combine: H must be a multiple of 8");
    if (tokens == 0) return 0;
    FSO_REQUIRE(dn && slot_of_flat && topk_w && out, "fso_moe_combine: NULL pointer");
    FSO_REQUIRE(aligned16(dn) && aligned16(out) && (bias == nullptr || aligned16(bias)),
        "fso_moe_combine: dn, out and bias must be 16-byte aligned");
    FSO_REQUIRE(bias != nullptr || bias_scale == nullptr, "fso_moe_combine: bias_scale scales bias and needs it");
    return launch_combine("fso_moe_combine", dn, slot_of_flat, topk_w, bias, bias_scale, out, tokens, topk, h,
        RowScatter{nullptr, nullptr, nullptr, 0, 1}, stream);
}

int fso_moe_combine_scatter(const void* dn, const int32_t* slot_of_flat, const float* topk_w, int64_t tokens,
    int64_t topk, int64_t h, const int64_t* recv_off, const int64_t* back_base, const uint64_t* peer_back,
    int64_t world, void* stream)
{
    FSO_REQUIRE(tokens >= 0 && topk >= 1 && topk <= 8 && h > 0 && h % 64 == 0 && world >= 1 && world <= 1024,
        "fso_moe_combine_scatter: 1 <= top-k <= 8, H a multiple of 64 and 1 <= world <= 1024 required");
    if (tokens == 0) return 0;
    FSO_REQUIRE(dn && slot_of_flat && topk_w && recv_off && back_base && peer_back,
        "fso_moe_combine_scatter: NULL pointer");
    FSO_REQUIRE((reinterpret_cast<uintptr_t>(dn) & 31u) == 0, "fso_moe_combine_scatter: dn must be 32-byte aligned");
    RowScatter const sc{recv_off, back_base, peer_back, static_cast<int>(world), coprime_multiplier(tokens)};
    // one CTA per row at a time, 128 threads over the row's 128-byte column groups; enough CTAs to fill the machine
    int64_t const cap = static_cast<int64_t>(sm_count()) * 32;
    int64_t const want = tokens < cap ? tokens : cap;
    combine_sparse_kernel<8><<<static_cast<unsigned>(want), 128, 0, as_stream(stream)>>>(
        static_cast<const uint8_t*>(dn), slot_of_flat, topk_w, tokens, static_cast<int>(topk), static_cast<int>(h * 2), sc);
    return launch_status("combine_sparse_kernel");
}

int fso_moe_topk_from_logits(const void* logits, int64_t logit_dtype, int64_t m, int64_t num_experts, int64_t ld,
    int64_t topk, int64_t renormalize, const int32_t* num_token_non_padded, const int32_t* expert_map,
    int32_t* topk_ids, float* topk_w, float* shared_gate, void* stream)
{
    FSO_REQUIRE(m >= 0 && m < (1ll << 31), "fso_moe_topk_from_logits: M out of range");
    FSO_REQUIRE(num_experts >= 1 && num_experts <= kRouterMaxExperts,
        "fso_moe_topk_from_logits: num_experts must be in [1, %d], got %lld", kRouterMaxExperts,
        static_cast<long long>(num_experts));
    FSO_REQUIRE(topk >= 1 && topk <= kRouterMaxTopk && topk <= num_experts,
        "fso_moe_topk_from_logits: topk must be in [1, min(%d, num_experts)], got %lld", kRouterMaxTopk,
        static_cast<long long>(topk));
    FSO_REQUIRE(ld >= num_experts + (shared_gate != nullptr ? 1 : 0),
        "fso_moe_topk_from_logits: the row stride %lld is shorter than a row", static_cast<long long>(ld));
    FSO_REQUIRE(logit_dtype >= 0 && logit_dtype <= 2, "fso_moe_topk_from_logits: logits must be bf16 (0), fp16 (1) or fp32 (2)");
    if (m == 0) return 0;
    FSO_REQUIRE(logits && topk_ids && topk_w, "fso_moe_topk_from_logits: NULL pointer");
    cudaStream_t const st = as_stream(stream);
    bool const rn = renormalize != 0;
    if (logit_dtype == 0)
        return launch_router_topk<__nv_bfloat16>(logits, ld, m, num_experts, topk, rn, num_token_non_padded, expert_map,
            topk_ids, topk_w, shared_gate, st);
    if (logit_dtype == 1)
        return launch_router_topk<__half>(logits, ld, m, num_experts, topk, rn, num_token_non_padded, expert_map,
            topk_ids, topk_w, shared_gate, st);
    return launch_router_topk<float>(logits, ld, m, num_experts, topk, rn, num_token_non_padded, expert_map, topk_ids,
        topk_w, shared_gate, st);
}

int fso_ep_plan_count(const int32_t* topk_ids, int64_t tokens, int64_t topk, int64_t experts_per_rank, int64_t world,
    uint64_t* rank_mask, int64_t* row, void* stream)
{
    FSO_REQUIRE(tokens >= 0 && tokens < (1ll << 31) && topk >= 1 && experts_per_rank >= 1
            && experts_per_rank < (1ll << 31) && world >= 1 && world <= 64,
        "fso_ep_plan_count: 1 <= world <= 64, top-k >= 1 and experts_per_rank >= 1 required");
    FSO_REQUIRE(row && (tokens == 0 || (topk_ids && rank_mask)), "fso_ep_plan_count: NULL pointer");
    FSO_CUDA(cudaMemsetAsync(row, 0, sizeof(int64_t) * (world + 1), as_stream(stream)));
    unsigned const blocks = tokens == 0 ? 1u : static_cast<unsigned>((tokens + 255) / 256);
    ep_plan_count_kernel<<<blocks, 256, 0, as_stream(stream)>>>(topk_ids, tokens, static_cast<int>(topk),
        static_cast<int>(experts_per_rank), static_cast<int>(world), rank_mask,
        reinterpret_cast<unsigned long long*>(row));
    return launch_status("ep_plan_count_kernel");
}

int fso_ep_plan_place(const uint64_t* rank_mask, const int64_t* table, int64_t tokens, int64_t world, int64_t rank,
    int64_t* send_token, int64_t* send_rank, int64_t* send_off, int64_t* dst_base, int64_t* recv_off,
    int64_t* back_base, int32_t* slot, void* stream)
{
    FSO_REQUIRE(tokens >= 0 && tokens < (1ll << 31) && world >= 1 && world <= 64 && rank >= 0 && rank < world,
        "fso_ep_plan_place: 1 <= world <= 64 and 0 <= rank < world required");
    FSO_REQUIRE(table && send_off && dst_base && recv_off && back_base, "fso_ep_plan_place: NULL pointer");
    FSO_REQUIRE(tokens == 0 || (rank_mask && send_token && send_rank && slot), "fso_ep_plan_place: NULL pointer");
    ep_plan_place_kernel<<<static_cast<unsigned>(world), 1024, 0, as_stream(stream)>>>(rank_mask, table, tokens,
        static_cast<int>(world), static_cast<int>(rank), send_token, send_rank, send_off, dst_base, recv_off, back_base,
        slot);
    return launch_status("ep_plan_place_kernel");
}

int fso_ep_dispatch_push(const void* xq, const void* xs, const int32_t* topk_ids, const float* topk_w,
    const int64_t* send_token, const int64_t* send_rank, const int64_t* send_off, const int64_t* dst_base,
    const uint64_t* peer_q, const uint64_t* peer_w, const uint64_t* peer_ids, const uint64_t* peer_wt, int64_t rows,
    int64_t topk, int64_t h, int64_t experts_per_rank, void* stream)
{
    FSO_REQUIRE(rows >= 0 && rows < (1ll << 31) && topk >= 1 && topk <= 128 && h > 0 && h % 128 == 0
            && experts_per_rank >= 1 && experts_per_rank < (1ll << 31),
        "fso_ep_dispatch_push: H a multiple of 128 and 1 <= top-k <= 128 required");
    if (rows == 0) return 0;
    FSO_REQUIRE(xq && xs && topk_ids && topk_w && send_token && send_rank && send_off && dst_base && peer_q && peer_w
            && peer_ids && peer_wt, "fso_ep_dispatch_push: NULL pointer");
    FSO_REQUIRE(aligned16(xq), "fso_ep_dispatch_push: xq must be 16-byte aligned");
    ep_push_rows_kernel<<<static_cast<unsigned>(rows), 128, 0, as_stream(stream)>>>(static_cast<const uint4*>(xq),
        static_cast<const uint32_t*>(xs), topk_ids, topk_w, send_token, send_rank, send_off, dst_base, peer_q, peer_w,
        peer_ids, peer_wt, static_cast<int>(topk), static_cast<int>(h / 128), static_cast<int>(experts_per_rank), rows,
        coprime_multiplier(rows));
    return launch_status("ep_push_rows_kernel");
}

int fso_moe_gather_rows(const void* rx_q, const void* rx_w, const int32_t* slot_of_flat, int64_t rows_in, int64_t topk,
    int64_t h, int64_t rows, void* hq, void* sh, void* stream)
{
    FSO_REQUIRE(rows_in >= 0 && topk >= 1 && h > 0 && h % 128 == 0 && rows > 0 && rows % 128 == 0,
        "fso_moe_gather_rows: H a multiple of 128 and rows a multiple of 128 required");
    if (rows_in == 0) return 0;
    FSO_REQUIRE(rx_q && rx_w && slot_of_flat && hq && sh, "fso_moe_gather_rows: NULL pointer");
    FSO_REQUIRE(aligned16(rx_q) && aligned16(hq) && (reinterpret_cast<uintptr_t>(sh) & 3u) == 0
            && (reinterpret_cast<uintptr_t>(rx_w) & 3u) == 0, "fso_moe_gather_rows: rx_q and hq must be 16-byte aligned");
    int64_t const total = rows_in * (h / 16);
    FSO_REQUIRE(total < (1ll << 31) - 4096, "fso_moe_gather_rows: rows * H/16 is beyond the kernel's index range");
    gather_rows_q_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(
        static_cast<const uint4*>(rx_q), static_cast<const uint32_t*>(rx_w), slot_of_flat, rows_in,
        static_cast<int>(topk), static_cast<int>(h / 128), static_cast<uint4*>(hq), static_cast<uint32_t*>(sh));
    return launch_status("gather_rows_q_kernel");
}

}  // extern "C"
