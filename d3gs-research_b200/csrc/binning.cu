// K2 inclusive scan of tile counts (single pass, decoupled look-back), K5 tile ranges, and the
// gather of per-pair splat records that the raster kernels stream.
//
// Reference semantics: d3sim/algos/d3gs/render.py:694-695 (cumsum + total), 896-939 (ranges),
// 1702-1716 (the per-batch gather this staging replaces).
#include <mutex>

#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 16;
constexpr int kScanTile = kScanThreads * kScanItems;

constexpr uint64_t kFlagAggregate = 1ull << 62;
constexpr uint64_t kFlagPrefix = 2ull << 62;
constexpr uint64_t kFlagMask = 3ull << 62;
constexpr uint64_t kValueMask = ~kFlagMask;

// workspace layout: [0] uint32 ticket, [1] uint32 pad, then uint64 status[num_tiles]
__global__ void __launch_bounds__(kScanThreads)
scan_lookback_kernel(const int32_t* __restrict__ in, int32_t* __restrict__ out, int64_t n, int64_t* __restrict__ total,
                     uint32_t* __restrict__ ticket, uint64_t* __restrict__ tile_status, uint32_t* __restrict__ status,
                     const TestHooks hooks) {
    __shared__ uint32_t s_tile;
    __shared__ int64_t s_warp[kScanThreads / 32];
    __shared__ int64_t s_prefix;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (t == 0) s_tile = atomicAdd(ticket, 1u);
    __syncthreads();
    const uint32_t tile = s_tile;
    const int64_t base = (int64_t)tile * kScanTile + (int64_t)t * kScanItems;
    int32_t v[kScanItems];
    if (base + kScanItems <= n && (((uintptr_t)(in + base)) & 15) == 0) {
#pragma unroll
        for (int k = 0; k < kScanItems / 4; ++k) {
            int4 q = *reinterpret_cast<const int4*>(in + base + k * 4);
            v[k * 4] = q.x; v[k * 4 + 1] = q.y; v[k * 4 + 2] = q.z; v[k * 4 + 3] = q.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) v[k] = (base + k < n) ? in[base + k] : 0;
    }
    int64_t run = 0;
    int64_t loc[kScanItems];
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) { run += v[k]; loc[k] = run; }
    // block-wide exclusive scan of the per-thread totals
    int64_t inc = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int64_t y = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += y;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    int64_t warp_off = 0, block_total = 0;
#pragma unroll
    for (int w = 0; w < kScanThreads / 32; ++w) {
        int64_t x = s_warp[w];
        if (w < warp) warp_off += x;
        block_total += x;
    }
    const int64_t thread_excl = warp_off + inc - run;
    // decoupled look-back by warp 0
    if (warp == 0) {
        int64_t excl = 0;
        const bool publish = (int)tile != hooks.hold;          // test hook: this tile never publishes
        const int spin_limit = hooks.poll_limit != 0 ? (int)hooks.poll_limit : (1 << 20);
        if (tile == 0) {
            if (lane == 0 && publish) {
                __threadfence();
                atomicExch((unsigned long long*)&tile_status[0], kFlagPrefix | ((uint64_t)block_total & kValueMask));
            }
        } else {
            if (lane == 0 && publish) {
                atomicExch((unsigned long long*)&tile_status[tile], kFlagAggregate | ((uint64_t)block_total & kValueMask));
            }
            int64_t look = (int64_t)tile - 1;
            bool gave_up = false;
            int spins = 0;
            while (true) {
                const int64_t idx = look - lane;
                uint64_t st = kFlagPrefix;   // lanes past the beginning behave like a zero prefix
                if (idx >= 0) st = *((volatile uint64_t*)&tile_status[idx]);
                const uint32_t invalid = __ballot_sync(0xffffffffu, (st & kFlagMask) == 0);
                const uint32_t prefix = __ballot_sync(0xffffffffu, (st & kFlagMask) == kFlagPrefix);
                // usable lanes: all lanes below the first invalid one
                const int first_invalid = invalid ? __ffs(invalid) - 1 : 32;
                const int first_prefix = prefix ? __ffs(prefix) - 1 : 32;
                if (first_prefix < first_invalid) {
                    int64_t contrib = (lane <= first_prefix) ? (int64_t)(st & kValueMask) : 0;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
                    excl += contrib;
                    break;
                }
                if (first_invalid > 0) {
                    // consume the aggregates in front of the first invalid tile
                    int64_t contrib = (lane < first_invalid) ? (int64_t)(st & kValueMask) : 0;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
                    excl += contrib;
                    look -= first_invalid;
                    spins = 0;
                } else {
                    if (++spins > spin_limit) { gave_up = true; break; }
                    __nanosleep(32);
                }
            }
            if (gave_up && lane == 0) atomicOr(status, D3GS_STATUS_SCAN_TIMEOUT);
            if (lane == 0 && publish) {
                __threadfence();
                atomicExch((unsigned long long*)&tile_status[tile],
                           kFlagPrefix | ((uint64_t)(excl + block_total) & kValueMask));
            }
        }
        if (lane == 0) s_prefix = excl;
    }
    __syncthreads();
    const int64_t off = s_prefix + thread_excl;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k)
        if (base + k < n) out[base + k] = (int32_t)(off + loc[k]);
    if (base <= n - 1 && n - 1 < base + kScanItems) total[0] = off + loc[(int)(n - 1 - base)];
}

__global__ void __launch_bounds__(256)
tile_ranges_kernel(const uint64_t* __restrict__ keys, int64_t n, int32_t* __restrict__ ranges, int shift) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const uint32_t t = (uint32_t)(keys[i] >> shift);
    if (i == 0) {
        ranges[(int64_t)t * 2] = 0;
    } else {
        const uint32_t lt = (uint32_t)(keys[i - 1] >> shift);
        if (t != lt) {
            ranges[(int64_t)lt * 2 + 1] = (int32_t)i;
            ranges[(int64_t)t * 2] = (int32_t)i;
        }
    }
    if (i == n - 1) ranges[(int64_t)t * 2 + 1] = (int32_t)n;
}

// Tiles by decreasing list length (in buckets of 32 entries): the raster grids take them in this order, so
// that the CTAs that start last are the cheapest.  One CTA: a shared-memory histogram over 64 length
// buckets, a scan from the longest bucket down, and a scatter; the order inside a bucket is arbitrary (the
// raster results do not depend on the order in which tiles are processed).
constexpr int kOrderBuckets = 64;
__device__ __forceinline__ int order_bucket(int len) { return kOrderBuckets - 1 - min(len >> 5, kOrderBuckets - 1); }

__global__ void __launch_bounds__(1024) tile_order_kernel(const int32_t* __restrict__ ranges, int num_tiles,
                                                         int32_t* __restrict__ order) {
    __shared__ int s_cnt[kOrderBuckets];
    __shared__ int s_off[kOrderBuckets];
    const int t = threadIdx.x;
    if (t < kOrderBuckets) s_cnt[t] = 0;
    __syncthreads();
    for (int i = t; i < num_tiles; i += 1024) atomicAdd(&s_cnt[order_bucket(ranges[i * 2 + 1] - ranges[i * 2])], 1);
    __syncthreads();
    if (t == 0) {
        int acc = 0;
        for (int b = 0; b < kOrderBuckets; ++b) {
            s_off[b] = acc;
            acc += s_cnt[b];
        }
    }
    __syncthreads();
    for (int i = t; i < num_tiles; i += 1024)
        order[atomicAdd(&s_off[order_bucket(ranges[i * 2 + 1] - ranges[i * 2])], 1)] = i;
}

// One 48-byte record per sorted (tile, Gaussian) pair:
//   [u, v, hx, hy] [ha, nb, hc, opacity] [r, g, b, thr]
// ha=-0.5*conic_a, nb=-conic_b, hc=-0.5*conic_c (exact scalings).
// thr = -ln(opacity/alpha_eps) - 0.01 is a conservative bound: power < thr implies
// opacity*exp(power) < 0.99*alpha_eps, so the blend loop may skip such a pixel without changing any result.
// (hx, hy) are the half extents of the axis-aligned box around {power >= thr}, slightly inflated and
// widened by the half size of a warp's 8x4 pixel block (3.5, 1.5): a warp whose block centre is further
// than (hx, hy) from (u, v) contains no pixel that the splat can touch.
__global__ void __launch_bounds__(256)
pack_splats_kernel(const int32_t* __restrict__ ids, int64_t n, const float* __restrict__ uvs,
                   const float* __restrict__ conic_opacity, const float* __restrict__ rgb, float alpha_eps,
                   float4* __restrict__ rec) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const int32_t id = ids[i];
    const float2 uv = __ldg(reinterpret_cast<const float2*>(uvs) + id);
    const float4 co = __ldg(reinterpret_cast<const float4*>(conic_opacity) + id);
    const float r = __ldg(rgb + (int64_t)id * 3), g = __ldg(rgb + (int64_t)id * 3 + 1), b = __ldg(rgb + (int64_t)id * 3 + 2);
    float4 r0, r1, r2;
    make_splat_record(uv, co, r, g, b, alpha_eps, r0, r1, r2);
    rec[i * 3] = r0;
    rec[i * 3 + 1] = r1;
    rec[i * 3 + 2] = r2;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" size_t d3gs_scan_workspace_bytes(int64_t n) {
    if (n < 0) n = 0;
    return 16 + (size_t)div_up64(n, kScanTile) * sizeof(uint64_t);
}

extern "C" int32_t d3gs_scan_tiles(const int32_t* in, int32_t* out, int64_t n, int64_t* total, void* workspace,
                                   size_t workspace_bytes, uint32_t* status, void* stream) {
    D3GS_REQUIRE(n >= 0, "negative element count");
    D3GS_REQUIRE(total != nullptr && status != nullptr, "total/status is NULL");
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        D3GS_CUDA(cudaMemsetAsync(total, 0, sizeof(int64_t), s));
        return D3GS_OK;
    }
    D3GS_REQUIRE(in != nullptr && out != nullptr && workspace != nullptr, "in/out/workspace is NULL");
    D3GS_REQUIRE(workspace_bytes >= d3gs_scan_workspace_bytes(n), "scan workspace too small: %zu < %zu",
                 workspace_bytes, d3gs_scan_workspace_bytes(n));
    D3GS_REQUIRE(((uintptr_t)workspace & 15) == 0, "scan workspace must be 16-byte aligned");
    const int64_t tiles = div_up64(n, kScanTile);
    D3GS_CUDA(cudaMemsetAsync(workspace, 0, d3gs_scan_workspace_bytes(n), s));
    uint32_t* ticket = reinterpret_cast<uint32_t*>(workspace);
    uint64_t* tstat = reinterpret_cast<uint64_t*>(reinterpret_cast<char*>(workspace) + 16);
    scan_lookback_kernel<<<(unsigned)tiles, kScanThreads, 0, s>>>(in, out, n, total, ticket, tstat, status, test_hooks());
    D3GS_LAUNCH_CHECK("scan_lookback_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_tile_ranges(const uint64_t* sorted_keys, int64_t n, int32_t* ranges, int64_t num_tiles,
                                    int32_t key_shift_bits, void* stream) {
    D3GS_REQUIRE(n >= 0 && num_tiles >= 0, "negative count");
    D3GS_REQUIRE(key_shift_bits == 0 || key_shift_bits == 32 || key_shift_bits == 18,
                 "key_shift_bits must be 32 (64-bit keys) or 18 (32-bit keys), got %d", key_shift_bits);
    D3GS_REQUIRE(ranges != nullptr || num_tiles == 0, "ranges is NULL");
    cudaStream_t s = (cudaStream_t)stream;
    if (num_tiles > 0) D3GS_CUDA(cudaMemsetAsync(ranges, 0, (size_t)num_tiles * 2 * sizeof(int32_t), s));
    if (n == 0) return D3GS_OK;
    D3GS_REQUIRE(sorted_keys != nullptr, "sorted_keys is NULL");
    D3GS_REQUIRE(n < (int64_t)1 << 31, "pair count %lld does not fit the int32 ranges", (long long)n);
    tile_ranges_kernel<<<(unsigned)div_up64(n, 256), 256, 0, s>>>(sorted_keys, n, ranges,
                                                                  key_shift_bits == 18 ? 18 : 32);
    D3GS_LAUNCH_CHECK("tile_ranges_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_tile_order(const int32_t* ranges, int64_t num_tiles, int32_t* order, void* stream) {
    D3GS_REQUIRE(num_tiles >= 0 && num_tiles < ((int64_t)1 << 31), "tile count out of range");
    if (num_tiles == 0) return D3GS_OK;
    D3GS_REQUIRE(ranges != nullptr && order != nullptr, "NULL argument");
    tile_order_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(ranges, (int)num_tiles, order);
    D3GS_LAUNCH_CHECK("tile_order_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_pack_splats(const int32_t* sorted_values, int64_t n, const D3gsSplatContext* ctx,
                                    float alpha_eps, float* records, void* stream) {
    D3GS_REQUIRE(n >= 0, "negative count");
    if (n == 0) return D3GS_OK;
    D3GS_REQUIRE(sorted_values && ctx && records, "NULL argument");
    D3GS_REQUIRE(ctx->uvs && ctx->conic_opacity && ctx->rgb_gaussian, "context tensor pointer is NULL");
    D3GS_REQUIRE(((uintptr_t)records & 15) == 0, "records must be 16-byte aligned");
    D3GS_REQUIRE(((uintptr_t)ctx->uvs & 7) == 0 && ((uintptr_t)ctx->conic_opacity & 15) == 0,
                 "uvs / conic_opacity must be 8 / 16-byte aligned");
    pack_splats_kernel<<<(unsigned)div_up64(n, 256), 256, 0, (cudaStream_t)stream>>>(
        sorted_values, n, ctx->uvs, ctx->conic_opacity, ctx->rgb_gaussian, alpha_eps, reinterpret_cast<float4*>(records));
    D3GS_LAUNCH_CHECK("pack_splats_kernel");
    return D3GS_OK;
}

// ---- allocation-free scan ----------------------------------------------------------------------
// Same single-pass scan as d3gs_scan_tiles, for callers that cannot hand the library a workspace because
// they are not able to obtain device memory at the moment of the call: a host application that gave its
// whole memory budget to another engine's pool, a plug-in running inside a frame loop where cudaMalloc's
// implicit device-wide synchronisation would stall the frame, or a thin C caller with no allocator of its
// own.  The tile-status words live in a fixed array inside the loaded module instead.
namespace d3gs {
namespace {

constexpr int64_t kStaticScanMaxItems = (int64_t)1 << 24;                          // 16,777,216 counts
constexpr size_t kStaticScanBytes = 16 + (size_t)(kStaticScanMaxItems / kScanTile) * sizeof(uint64_t);   // 32,784 B

// Held by every GPU that loads the library, from load to exit.
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScanBytes];

constexpr int kMaxDevices = 64;
void* g_static_scan_ptr[kMaxDevices] = {};    // guarded by g_static_scan_mutex
std::mutex g_static_scan_mutex;

}  // namespace
}  // namespace d3gs

extern "C" int64_t d3gs_scan_tiles_static_max_items(void) { return d3gs::kStaticScanMaxItems; }

extern "C" int32_t d3gs_scan_tiles_static(const int32_t* in, int32_t* out, int64_t n, int64_t* total, uint32_t* status,
                                          void* stream) {
    using namespace d3gs;
    D3GS_REQUIRE(n >= 0, "negative element count");
    D3GS_REQUIRE(n <= kStaticScanMaxItems,
                 "d3gs_scan_tiles_static handles at most %lld elements (built-in scratch of %zu bytes); got %lld -- "
                 "use d3gs_scan_tiles with a caller-provided workspace",
                 (long long)kStaticScanMaxItems, kStaticScanBytes, (long long)n);
    D3GS_REQUIRE(total != nullptr && status != nullptr, "total/status is NULL");
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        D3GS_CUDA(cudaMemsetAsync(total, 0, sizeof(int64_t), s));
        return D3GS_OK;
    }
    D3GS_REQUIRE(in != nullptr && out != nullptr, "in/out is NULL");
    int dev = -1;
    D3GS_CUDA(cudaGetDevice(&dev));
    D3GS_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d outside [0,%d)", dev, kMaxDevices);
    unsigned char* base = nullptr;
    {
        // Set-up, once per device, with that device current: in host code the array's name is only a
        // stand-in symbol, so its device address has to be asked for before it can be given to a kernel.
        // Host threads making their first calls at the same time take turns here.
        std::lock_guard<std::mutex> lock(g_static_scan_mutex);
        if (g_static_scan_ptr[dev] == nullptr) {
            void* p = nullptr;
            D3GS_CUDA(cudaGetSymbolAddress(&p, g_static_scan_scratch));
            D3GS_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned NULL");
            g_static_scan_ptr[dev] = p;
        }
        base = reinterpret_cast<unsigned char*>(g_static_scan_ptr[dev]);
    }
    const int64_t tiles = div_up64(n, kScanTile);
    // every call shares the array and finds the previous call's ticket and tile states in it: clear the part in use
    D3GS_CUDA(cudaMemsetAsync(base, 0, 16 + (size_t)tiles * sizeof(uint64_t), s));
    scan_lookback_kernel<<<(unsigned)tiles, kScanThreads, 0, s>>>(in, out, n, total, reinterpret_cast<uint32_t*>(base),
                                                                 reinterpret_cast<uint64_t*>(base + 16), status,
                                                                 test_hooks());
    D3GS_LAUNCH_CHECK("scan_lookback_kernel (static scratch)");
    return D3GS_OK;
}
