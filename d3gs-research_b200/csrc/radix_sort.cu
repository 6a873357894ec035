// K4: stable LSD radix sort of (uint64 key, int32 value) pairs on a bit range -- a hand-written
// "onesweep" (one read + one write of the pairs per 8-bit digit, chained-scan look-back between
// tiles), replacing the reference's cub::DeviceRadixSort::SortPairs call
// (d3sim/csrc/devsort.py:74-127, call site d3sim/algos/d3gs/render.py:845-887).
//
// Phases per call:
//   1. one histogram kernel builds the 256-bin digit histograms of ALL passes (one read of keys);
//   2. one tiny kernel turns each histogram into exclusive digit offsets;
//   3. per pass, one onesweep kernel: a tile of 8192 pairs is ranked stably inside the CTA
//      (warp match-any multi-split), the per-digit tile counts are published, each digit's
//      global offset is obtained by looking back over the predecessor tiles, and the tile is
//      written out through shared memory in digit-sorted runs.
// Every wait on another CTA's flag is bounded; when it gives up it raises
// D3GS_STATUS_SORT_TIMEOUT in the caller's status word and the kernel finishes without hanging.
#include "common.cuh"

namespace d3gs {
namespace {

// Digits are 8 bits wide, or 9 when that saves a pass (45 key bits: 5 passes instead of 6); the kernels are
// templated on the width.  Tables on the host side are sized for the wider digit.
constexpr int kMaxRadixBits = 9;
constexpr int kMaxRadix = 1 << kMaxRadixBits;
// 8192 pairs per CTA as 1024 threads x 8 items, one CTA per SM.  The ranking below is a chain of dependent
// rounds, one per item, so few items per thread keep a tile's lifetime short (at a few million pairs the
// sort is bound by latency, not by bytes), and a large tile amortises the per-tile phases (digit totals,
// look-back, barriers).  Measured at 4.3 M pairs, 45 key bits: 256x16 0.435 ms, 512x8 0.393, 1024x4 0.438,
// 512x4 0.457, 1024x8 0.371.
constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortItems = 8;
constexpr int kSortTile = kSortThreads * kSortItems;   // 8192 pairs per CTA
constexpr int kMaxPasses = 8;

constexpr uint32_t kLbAggregate = 1u << 30;
constexpr uint32_t kLbPrefix = 2u << 30;
constexpr uint32_t kLbFlagMask = 3u << 30;
constexpr uint32_t kLbValueMask = ~kLbFlagMask;

struct PassTable {
    int32_t shift[kMaxPasses];
    uint32_t mask[kMaxPasses];
    int32_t num_passes;
};

template <int BITS>
__global__ void __launch_bounds__(256)
histogram_kernel(const uint64_t* __restrict__ keys, int64_t n, const __grid_constant__ PassTable pt,
                 uint32_t* __restrict__ hist /* [passes][radix] */) {
    constexpr int kRadix = 1 << BITS;
    __shared__ uint32_t s_hist[kMaxPasses * kRadix];
    for (int k = threadIdx.x; k < pt.num_passes * kRadix; k += 256) s_hist[k] = 0;
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const uint64_t key = keys[i];
#pragma unroll
        for (int p = 0; p < kMaxPasses; ++p) {
            if (p < pt.num_passes) atomicAdd(&s_hist[p * kRadix + (uint32_t)((key >> pt.shift[p]) & pt.mask[p])], 1u);
        }
    }
    __syncthreads();
    for (int k = threadIdx.x; k < pt.num_passes * kRadix; k += 256) {
        const uint32_t c = s_hist[k];
        if (c) atomicAdd(&hist[k], c);
    }
}

// exclusive scan of each pass's bins, in place; one CTA of one thread per bin per pass
template <int BITS>
__global__ void __launch_bounds__(1 << BITS) digit_offsets_kernel(uint32_t* __restrict__ hist) {
    constexpr int kRadix = 1 << BITS;
    __shared__ uint32_t s_w[kRadix / 32];
    uint32_t* h = hist + (size_t)blockIdx.x * kRadix;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t c = h[t];
    uint32_t inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t y = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += y;
    }
    if (lane == 31) s_w[warp] = inc;
    __syncthreads();
    uint32_t off = 0;
    for (int w = 0; w < warp; ++w) off += s_w[w];
    h[t] = off + inc - c;
}

// Slots of the staging arrays are padded (one extra slot per 16 keys / per 32 values).  With uniformly
// distributed digits every digit's run in the sorted tile is ~16 long, so the 32 lanes of a warp -- which
// hold 32 different digits at similar ranks -- would all hit positions 16 apart: the same bank.
__device__ __forceinline__ int key_slot(int pos) { return pos + (pos >> 4); }
__device__ __forceinline__ int val_slot(int pos) { return pos + (pos >> 5); }

// Lanes of the warp that hold the same (BITS+1)-bit value (digit, or the radix for "no item"): one ballot per
// bit.  __match_any_sync gives the same mask, but its latency grows with the number of distinct values in
// the warp, and with uniformly distributed digits (the low depth bits) all 32 lanes differ.
template <int BITS>
__device__ __forceinline__ uint32_t same_bin_lanes(uint32_t bin) {
    uint32_t peers = 0xffffffffu;
#pragma unroll
    for (int b = 0; b <= BITS; ++b) {
        const bool bit = (bin >> b) & 1u;
        const uint32_t vote = __ballot_sync(0xffffffffu, bit);
        peers &= bit ? vote : ~vote;
    }
    return peers;
}

template <int BITS>
struct SweepSmem {
    static constexpr int kRadix = 1 << BITS;
    uint64_t keys[kSortTile + kSortTile / 16];
    int32_t vals[kSortTile + kSortTile / 32];
    uint32_t warp_hist[kSortWarps][kRadix + 1];
    uint32_t digit_off[kRadix + 1];
    int64_t global_base[kRadix];
    uint32_t scan_tmp[kRadix / 32];
    uint32_t tile;
};

template <int BITS>
__global__ void __launch_bounds__(kSortThreads, 1)
onesweep_kernel(const uint64_t* __restrict__ keys_in, uint64_t* __restrict__ keys_out,
                const int32_t* __restrict__ vals_in, int32_t* __restrict__ vals_out, int64_t n, int shift,
                uint32_t mask, const uint32_t* __restrict__ digit_base, uint32_t* __restrict__ ticket,
                uint32_t* __restrict__ lookback /* [tiles][radix] */, uint32_t* __restrict__ status,
                const TestHooks hooks) {
    constexpr int kRadix = 1 << BITS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SweepSmem<BITS>& sm = *reinterpret_cast<SweepSmem<BITS>*>(smem_raw);
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (t == 0) sm.tile = atomicAdd(ticket, 1u);
    for (int k = t; k < kSortWarps * (kRadix + 1); k += kSortThreads) (&sm.warp_hist[0][0])[k] = 0;
    __syncthreads();
    const uint32_t tile = sm.tile;
    const int64_t tile_base = (int64_t)tile * kSortTile;
    const int count = (int)min((int64_t)kSortTile, n - tile_base);

    // ---- load (warp-striped: index = warp*512 + item*32 + lane) and rank ------------------------
    uint64_t key[kSortItems];
    int32_t val[kSortItems];
    uint16_t rank[kSortItems];
    const uint32_t lanemask_lt = (1u << lane) - 1u;
#pragma unroll
    for (int i = 0; i < kSortItems; ++i) {
        const int local = warp * (32 * kSortItems) + i * 32 + lane;
        const bool valid = local < count;
        key[i] = valid ? keys_in[tile_base + local] : ~0ull;
        val[i] = valid ? vals_in[tile_base + local] : 0;
    }
#pragma unroll
    for (int i = 0; i < kSortItems; ++i) {
        const int local = warp * (32 * kSortItems) + i * 32 + lane;
        const uint32_t bin = (local < count) ? (uint32_t)((key[i] >> shift) & mask) : (uint32_t)kRadix;
        const uint32_t peers = same_bin_lanes<BITS>(bin);
        const uint32_t pre = sm.warp_hist[warp][bin];
        __syncwarp();
        if (lane == __ffs(peers) - 1) sm.warp_hist[warp][bin] = pre + __popc(peers);
        __syncwarp();
        rank[i] = (uint16_t)(pre + __popc(peers & lanemask_lt));
    }
    __syncthreads();

    // ---- per-digit tile counts, publish, look back ---------------------------------------------
    const int d = t;   // the first `radix` threads own one digit each
    uint32_t tot = 0, inc = 0;
    uint32_t* my = lookback + (size_t)tile * kRadix + (d < kRadix ? d : 0);
    if (d < kRadix) {
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const uint32_t c = sm.warp_hist[w][d];
            sm.warp_hist[w][d] = tot;   // exclusive offset of this warp inside the digit's run
            tot += c;
        }
        if ((int)tile != hooks.hold) {      // test hook: this tile never publishes its counts
            if (tile == 0) atomicExch(my, kLbPrefix | tot);
            else atomicExch(my, kLbAggregate | tot);
        }
        // block-wide exclusive scan over digits -> position of the digit's run in the sorted tile
        inc = tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            uint32_t y = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += y;
        }
        if (lane == 31) sm.scan_tmp[warp] = inc;
    }
    __syncthreads();
    if (d < kRadix) {
        uint32_t off = 0;
        for (int w = 0; w < warp; ++w) off += sm.scan_tmp[w];
        const uint32_t dig_off = off + inc - tot;
        sm.digit_off[d] = dig_off;
        // look-back: sum the counts of all predecessor tiles for this digit
        uint32_t excl = 0;
        if (tile > 0) {
            // Predecessors are read eight at a time (independent loads, one memory latency per batch) and
            // consumed in order; the walk stops at the first inclusive prefix and waits, bounded, at the
            // first tile that has not published yet.  (Batches of 32 measured slower than 8.)
            constexpr int kLook = 8;
            int64_t look = (int64_t)tile - 1;
            bool gave_up = false, done = false;
            int spins = 0;
            while (look >= 0 && !done && !gave_up) {
                uint32_t st[kLook];
#pragma unroll
                for (int k = 0; k < kLook; ++k) {
                    const int64_t idx = look - k;
                    st[k] = idx >= 0 ? *((const volatile uint32_t*)(lookback + (size_t)idx * kRadix + d)) : kLbPrefix;
                }
                int consumed = 0;
                bool blocked = false;
#pragma unroll
                for (int k = 0; k < kLook; ++k) {
                    if (!done && !blocked) {
                        if ((st[k] & kLbFlagMask) == 0) {
                            blocked = true;
                        } else {
                            excl += st[k] & kLbValueMask;
                            ++consumed;
                            if ((st[k] & kLbFlagMask) == kLbPrefix) done = true;
                        }
                    }
                }
                look -= consumed;
                if (blocked) {
                    if (++spins > (hooks.poll_limit != 0 ? (int)hooks.poll_limit : (1 << 20))) gave_up = true;
                    __nanosleep(20);
                } else {
                    spins = 0;
                }
            }
            if (gave_up) atomicOr(status, D3GS_STATUS_SORT_TIMEOUT);
            if ((int)tile != hooks.hold) atomicExch(my, kLbPrefix | ((excl + tot) & kLbValueMask));
        }
        sm.global_base[d] = (int64_t)digit_base[d] + (int64_t)excl - (int64_t)dig_off;
    }
    __syncthreads();

    // ---- scatter into shared memory in digit-sorted order, then coalesced write-out --------------
#pragma unroll
    for (int i = 0; i < kSortItems; ++i) {
        const int local = warp * (32 * kSortItems) + i * 32 + lane;
        if (local < count) {
            const uint32_t bin = (uint32_t)((key[i] >> shift) & mask);
            const uint32_t pos = sm.digit_off[bin] + sm.warp_hist[warp][bin] + rank[i];
            sm.keys[key_slot(pos)] = key[i];
            sm.vals[val_slot(pos)] = val[i];
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kSortItems; ++i) {
        const int pos = i * kSortThreads + t;
        if (pos < count) {
            const uint64_t k = sm.keys[key_slot(pos)];
            const uint32_t bin = (uint32_t)((k >> shift) & mask);
            const int64_t g = sm.global_base[bin] + pos;
            keys_out[g] = k;
            vals_out[g] = sm.vals[val_slot(pos)];
        }
    }
}

struct SortLayout {
    size_t hist_off, ticket_off, lookback_off, total;
    int64_t tiles;
};

SortLayout sort_layout(int64_t n) {
    SortLayout L;
    L.tiles = div_up64(n > 0 ? n : 1, kSortTile);
    L.hist_off = 0;
    L.ticket_off = L.hist_off + sizeof(uint32_t) * kMaxPasses * kMaxRadix;
    L.lookback_off = L.ticket_off + 256;
    // one look-back table per pass, all cleared by the single memset at the start: no memset node between
    // two passes' kernels
    L.total = L.lookback_off + (size_t)kMaxPasses * L.tiles * kMaxRadix * sizeof(uint32_t);
    return L;
}

}  // namespace
}  // namespace d3gs

namespace d3gs {
namespace {

// 9-bit digits when they save a pass, 8-bit digits otherwise
int digit_bits(int key_bits) {
    return (key_bits + 8) / 9 < (key_bits + 7) / 8 ? 9 : 8;
}

template <int BITS>
int32_t run_sort(uint64_t* keys, uint64_t* keys_alt, int32_t* values, int32_t* values_alt, int64_t n, int begin_bit,
                 int end_bit, int passes, const SortLayout& L, char* ws, uint32_t* status, cudaStream_t s) {
    constexpr int kRadix = 1 << BITS;
    uint32_t* hist = reinterpret_cast<uint32_t*>(ws + L.hist_off);
    uint32_t* tickets = reinterpret_cast<uint32_t*>(ws + L.ticket_off);
    uint32_t* lookback = reinterpret_cast<uint32_t*>(ws + L.lookback_off);
    PassTable pt;
    pt.num_passes = passes;
    for (int p = 0; p < kMaxPasses; ++p) {
        const int sh = begin_bit + p * BITS;
        const int bits = p < passes ? (end_bit - sh < BITS ? end_bit - sh : BITS) : 0;
        pt.shift[p] = p < passes ? sh : 0;
        pt.mask[p] = bits > 0 ? ((1u << bits) - 1u) : 0u;
    }
    D3GS_CUDA(cudaFuncSetAttribute(onesweep_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)sizeof(SweepSmem<BITS>)));
    const size_t lb_pass = (size_t)L.tiles * kRadix;         // look-back words per pass
    D3GS_CUDA(cudaMemsetAsync(ws, 0, L.lookback_off + (size_t)passes * lb_pass * sizeof(uint32_t), s));
    int hist_blocks = (int)(L.tiles < 148 * 8 ? L.tiles : 148 * 8);
    histogram_kernel<BITS><<<hist_blocks, 256, 0, s>>>(keys, n, pt, hist);
    D3GS_LAUNCH_CHECK("histogram_kernel");
    digit_offsets_kernel<BITS><<<passes, kRadix, 0, s>>>(hist);
    D3GS_LAUNCH_CHECK("digit_offsets_kernel");
    uint64_t* kin = keys;
    uint64_t* kout = keys_alt;
    int32_t* vin = values;
    int32_t* vout = values_alt;
    for (int p = 0; p < passes; ++p) {
        onesweep_kernel<BITS><<<(unsigned)L.tiles, kSortThreads, sizeof(SweepSmem<BITS>), s>>>(
            kin, kout, vin, vout, n, pt.shift[p], pt.mask[p], hist + (size_t)p * kRadix, tickets + p,
            lookback + (size_t)p * lb_pass, status, test_hooks());
        D3GS_LAUNCH_CHECK("onesweep_kernel");
        uint64_t* tk = kin; kin = kout; kout = tk;
        int32_t* tv = vin; vin = vout; vout = tv;
    }
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" size_t d3gs_sort_workspace_bytes(int64_t n, int32_t begin_bit, int32_t end_bit) {
    (void)begin_bit;
    (void)end_bit;
    return sort_layout(n).total;
}

extern "C" int32_t d3gs_sort_pairs(uint64_t* keys, uint64_t* keys_alt, int32_t* values, int32_t* values_alt, int64_t n,
                                   int32_t begin_bit, int32_t end_bit, void* workspace, size_t workspace_bytes,
                                   int32_t* result_in_alt, uint32_t* status, void* stream) {
    D3GS_REQUIRE(n >= 0, "negative pair count");
    D3GS_REQUIRE(begin_bit >= 0 && end_bit <= 64 && begin_bit <= end_bit, "bad bit range [%d,%d)", begin_bit, end_bit);
    D3GS_REQUIRE(result_in_alt != nullptr && status != nullptr, "result_in_alt/status is NULL");
    const int bits = digit_bits(end_bit - begin_bit);
    const int passes = (end_bit - begin_bit + bits - 1) / bits;
    *result_in_alt = passes & 1;
    if (n == 0 || passes == 0) {
        *result_in_alt = 0;
        return D3GS_OK;
    }
    D3GS_REQUIRE(keys && keys_alt && values && values_alt && workspace, "NULL buffer");
    D3GS_REQUIRE(n < ((int64_t)1 << 30), "pair count %lld exceeds the 2^30 limit of the look-back counters", (long long)n);
    const SortLayout L = sort_layout(n);
    D3GS_REQUIRE(workspace_bytes >= L.total, "sort workspace too small: %zu < %zu", workspace_bytes, L.total);
    D3GS_REQUIRE(((uintptr_t)workspace & 15) == 0, "sort workspace must be 16-byte aligned");
    char* ws = reinterpret_cast<char*>(workspace);
    if (bits == 9)
        return run_sort<9>(keys, keys_alt, values, values_alt, n, begin_bit, end_bit, passes, L, ws, status,
                           (cudaStream_t)stream);
    return run_sort<8>(keys, keys_alt, values, values_alt, n, begin_bit, end_bit, passes, L, ws, status,
                       (cudaStream_t)stream);
}
