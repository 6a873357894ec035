// Tile-bucket binning: the same sorted per-tile lists and tile ranges as key duplication + radix sort + range
// extraction (d3sim/algos/d3gs/render.py:739-939), built without a global sort.
//
// The reference duplicates every visible Gaussian into one 64-bit key (tile << 32 | depth bits) per tile it
// touches, sorts all keys with a stable radix sort over 32 + log2(tiles) bits (d3sim/csrc/devsort.py:74-127) and
// reads each tile's [start, end) off the sorted keys.  The upper key bits only say which tile a pair belongs
// to, and that is known the moment the pair is produced.  So here
//   1. the preprocess counts, per tile, the Gaussians that touch it (one atomic add per pair);
//   2. an inclusive scan of the tile counts gives every tile its range directly (d3gs_scan_tiles over the
//      tiles, then d3gs_bucket_prepare: ranges, per-tile write cursors, the longest list);
//   3. d3gs_bucket_emit writes every pair as one 8-byte entry (depth bits << 32 | flat Gaussian index) into
//      its tile's range at a position drawn from the tile's cursor (arrival order, arbitrary);
//   4. d3gs_bucket_sort sorts every tile's entries in shared memory (thread-local sorting network, then
//      merge-path merge passes) and writes the Gaussian indices -- and, on request, the reference's 64-bit
//      keys -- in sorted order.
// An entry is unique (a Gaussian appears once per tile), so ordering the 64-bit entries orders a tile's list
// by depth with ties by ascending flat index, which is exactly what the reference's stable sort of pairs
// emitted in index order yields.  Pairs cross HBM twice (8 bytes written by 3, read by 4) plus 4 bytes of
// sorted indices, instead of 24 bytes per pair and digit pass.  Lists longer than the shared-memory capacity
// are not handled: the caller reads the longest list with its pair count and takes the radix-sort path then.
#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kSortCapacity = 16384;        // entries per tile the largest kernel instance holds in shared memory
constexpr uint64_t kPadEntry = ~0ull;       // sorts behind every real entry

__global__ void __launch_bounds__(256)
bucket_prepare_kernel(const int32_t* __restrict__ counts, const int32_t* __restrict__ incl, int64_t num_tiles,
                      int32_t* __restrict__ ranges, int32_t* __restrict__ cursor, int64_t* __restrict__ max_count,
                      int64_t pair_capacity) {
    const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
    // A caller that sized the pair buffers before it knew the pair count (from the previous launch) passes their
    // capacity: when the pairs do not fit, every range is left empty, so that the kernels already queued behind
    // this one touch nothing, and the caller, who reads the count afterwards, repeats the launch with larger buffers.
    const bool fits = pair_capacity <= 0 || (int64_t)incl[num_tiles - 1] <= pair_capacity;
    int c = 0;
    if (t < num_tiles) {
        c = counts[t];
        const int end = incl[t], start = end - c;
        // render.py:897: the reference zero-fills the ranges and writes only the tiles that own pairs
        ranges[t * 2] = c > 0 && fits ? start : 0;
        ranges[t * 2 + 1] = c > 0 && fits ? end : 0;
        cursor[t] = start;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c = max(c, __shfl_xor_sync(0xffffffffu, c, o));
    if ((threadIdx.x & 31) == 0 && c > 0) atomicMax(reinterpret_cast<unsigned long long*>(max_count), (unsigned long long)c);
}

__device__ __forceinline__ void cswap(uint64_t& a, uint64_t& b) {
    const uint64_t lo = a < b ? a : b, hi = a < b ? b : a;
    a = lo;
    b = hi;
}

// One CTA sorts one tile's list of n <= NT * VT entries.  Shared-memory slots are padded by one per VT entries
// so that the per-thread runs (VT consecutive entries) start in different banks.
template <int NT, int VT>
__device__ __forceinline__ void sort_one_tile(uint64_t* s_e, const int tile, const uint64_t* __restrict__ entries,
                                              const int32_t* __restrict__ ranges, int32_t* __restrict__ sorted_values,
                                              uint64_t* __restrict__ sorted_keys, int lo, int hi, int pass_longer) {
    const int r0 = ranges[tile * 2];
    const int n = ranges[tile * 2 + 1] - r0;
    const int t = threadIdx.x;
    if (n > hi && pass_longer) {
        // The largest instance launched, and this list is longer than the caller expected when it chose the
        // instances: hand the indices on in emission order, so that whatever is queued behind reads valid indices;
        // the caller sees the true length afterwards and repeats the sort.
        for (int p = t; p < n; p += NT) sorted_values[r0 + p] = (int32_t)(uint32_t)entries[r0 + p];
        return;
    }
    if (n <= lo || n > hi) return;     // another instance (or nobody, n == 0) handles this tile
    auto slot = [](int p) { return p + p / VT; };
#pragma unroll
    for (int k = 0; k < VT; ++k) {
        const int p = k * NT + t;
        s_e[slot(p)] = p < n ? entries[r0 + p] : kPadEntry;
    }
    __syncthreads();
    uint64_t key[VT];
#pragma unroll
    for (int k = 0; k < VT; ++k) key[k] = s_e[slot(t * VT + k)];
    // odd-even transposition network over the thread's VT entries
#pragma unroll
    for (int round = 0; round < VT; ++round) {
#pragma unroll
        for (int k = round & 1; k + 1 < VT; k += 2) cswap(key[k], key[k + 1]);
    }
    const bool active = t * VT < n;    // threads past the end hold only padding, which is already in place
    for (int width = VT; width < n; width <<= 1) {
        __syncthreads();               // every thread has taken the previous pass's inputs
#pragma unroll
        for (int k = 0; k < VT; ++k) s_e[slot(t * VT + k)] = key[k];
        __syncthreads();
        if (active) {
            const int a0 = (t * VT) & ~(2 * width - 1), b0 = a0 + width;
            const int d = t * VT - a0;
            // merge path: how many of the first d outputs come from run A (ties: A first)
            int lo_i = max(0, d - width), hi_i = min(d, width);
            while (lo_i < hi_i) {
                const int mid = (lo_i + hi_i) >> 1;
                if (s_e[slot(a0 + mid)] <= s_e[slot(b0 + d - 1 - mid)]) lo_i = mid + 1;
                else hi_i = mid;
            }
            int ia = lo_i, ib = d - lo_i;
            uint64_t ka = ia < width ? s_e[slot(a0 + ia)] : kPadEntry;
            uint64_t kb = ib < width ? s_e[slot(b0 + ib)] : kPadEntry;
#pragma unroll
            for (int k = 0; k < VT; ++k) {
                const bool take_a = ib >= width || (ia < width && ka <= kb);
                key[k] = take_a ? ka : kb;
                if (take_a) {
                    ++ia;
                    ka = ia < width ? s_e[slot(a0 + ia)] : kPadEntry;
                } else {
                    ++ib;
                    kb = ib < width ? s_e[slot(b0 + ib)] : kPadEntry;
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < VT; ++k) s_e[slot(t * VT + k)] = key[k];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < VT; ++k) {
        const int p = k * NT + t;
        if (p < n) {
            const uint64_t e = s_e[slot(p)];
            sorted_values[r0 + p] = (int32_t)(uint32_t)e;
            if (sorted_keys != nullptr) sorted_keys[r0 + p] = ((uint64_t)(uint32_t)tile << 32) | (e >> 32);
        }
    }
}

// The grid may be smaller than the number of tiles: a CTA then takes every gridDim.x-th tile.  The instance for the
// longest lists holds 136 KB of shared memory, one CTA per SM; launched with one CTA per tile it spent 33 us on a
// scene where no list needed it (8160 CTAs that leave at once, 148 at a time), so it gets two CTAs per SM's worth.
template <int NT, int VT>
__global__ void __launch_bounds__(NT)
tile_sort_kernel(const uint64_t* __restrict__ entries, const int32_t* __restrict__ ranges, int num_tiles,
                 int32_t* __restrict__ sorted_values, uint64_t* __restrict__ sorted_keys, int lo, int hi, int pass_longer) {
    extern __shared__ __align__(16) uint64_t s_e[];
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        sort_one_tile<NT, VT>(s_e, tile, entries, ranges, sorted_values, sorted_keys, lo, hi, pass_longer);
        __syncthreads();      // the next tile reuses the shared memory
    }
}

template <int NT, int VT>
int32_t launch_sort(const uint64_t* entries, const int32_t* ranges, int64_t num_tiles, int32_t* sorted_values,
                    uint64_t* sorted_keys, int lo, int hi, bool pass_longer, cudaStream_t s) {
    const size_t smem = (size_t)(NT * VT + NT) * sizeof(uint64_t);
    if (smem > 48 * 1024)
        D3GS_CUDA(cudaFuncSetAttribute(tile_sort_kernel<NT, VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t grid = num_tiles;
    if (NT >= 1024) {
        int dev = 0, sms = 0;
        D3GS_CUDA(cudaGetDevice(&dev));
        D3GS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        grid = grid < 2 * (int64_t)sms ? grid : 2 * (int64_t)sms;
    }
    tile_sort_kernel<NT, VT><<<(unsigned)grid, NT, smem, s>>>(entries, ranges, (int)num_tiles, sorted_values, sorted_keys,
                                                              lo, hi, pass_longer ? 1 : 0);
    D3GS_LAUNCH_CHECK("tile_sort_kernel");
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" int64_t d3gs_bucket_sort_capacity(void) { return kSortCapacity; }

extern "C" int32_t d3gs_bucket_prepare(const int32_t* tile_counts, const int32_t* tile_scan, int64_t num_tiles,
                                       int32_t* ranges, int32_t* cursor, int64_t* max_count, int64_t pair_capacity,
                                       void* stream) {
    D3GS_REQUIRE(num_tiles >= 0 && num_tiles < ((int64_t)1 << 31), "tile count out of range");
    D3GS_REQUIRE(max_count != nullptr, "max_count is NULL");
    cudaStream_t s = (cudaStream_t)stream;
    D3GS_CUDA(cudaMemsetAsync(max_count, 0, sizeof(int64_t), s));
    if (num_tiles == 0) return D3GS_OK;
    D3GS_REQUIRE(tile_counts && tile_scan && ranges && cursor, "NULL argument");
    bucket_prepare_kernel<<<(unsigned)div_up64(num_tiles, 256), 256, 0, s>>>(tile_counts, tile_scan, num_tiles, ranges,
                                                                            cursor, max_count, pair_capacity);
    D3GS_LAUNCH_CHECK("bucket_prepare_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_bucket_sort(const uint64_t* entries, const int32_t* ranges, int64_t num_tiles, int64_t max_count,
                                    int32_t* sorted_values, uint64_t* sorted_keys, void* stream) {
    D3GS_REQUIRE(num_tiles >= 0 && num_tiles < ((int64_t)1 << 31), "tile count out of range");
    D3GS_REQUIRE(max_count >= 0, "negative max_count");
    if (max_count > kSortCapacity) {
        set_error("d3gs_bucket_sort holds at most %d entries per tile in shared memory; the longest list has %lld -- "
                  "use d3gs_duplicate_keys + d3gs_sort_pairs + d3gs_tile_ranges",
                  kSortCapacity, (long long)max_count);
        return D3GS_ERR_UNSUPPORTED;
    }
    if (num_tiles == 0 || max_count == 0) return D3GS_OK;
    D3GS_REQUIRE(entries && ranges && sorted_values, "NULL argument");
    cudaStream_t s = (cudaStream_t)stream;
    // three instances by list length; an instance is launched only when some list can fall into its class
    // (the largest one launched also passes through, unsorted, any list longer than max_count promised)
    int32_t rc = launch_sort<128, 4>(entries, ranges, num_tiles, sorted_values, sorted_keys, 0, 512, max_count <= 512, s);
    if (rc != D3GS_OK) return rc;
    if (max_count > 512) {
        rc = launch_sort<256, 8>(entries, ranges, num_tiles, sorted_values, sorted_keys, 512, 2048, max_count <= 2048, s);
        if (rc != D3GS_OK) return rc;
    }
    if (max_count > 2048) {
        rc = launch_sort<1024, 16>(entries, ranges, num_tiles, sorted_values, sorted_keys, 2048, kSortCapacity, true, s);
        if (rc != D3GS_OK) return rc;
    }
    return D3GS_OK;
}
