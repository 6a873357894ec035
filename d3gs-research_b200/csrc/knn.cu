// Exact k-nearest-neighbour distances of a point cloud (d3sim/algos/d3gs/ops.py:14-183 simple_knn), used to
// initialise the Gaussians' scales from SfM points (origin/model.py:26-28, tools.py:65-67).
//
// The reference: Morton codes -> argsort -> boxes of 256 consecutive sorted points with their bounds -> one
// thread per point, which first takes the k-th distance among its 2k neighbours in sorted order as a bound
// and then walks ALL boxes, skipping those farther away than the bound.  The result is the exact set of the k
// smallest distances (self excluded by position, so a duplicate point counts with distance 0).
//
// Here: the same codes, this library's radix sort, and one CTA per box.  The CTA culls the box list once for all
// its 256 points (a box can matter to some point of the CTA only if it is within the largest bound of the CTA's
// own bounds), stages every surviving box's points in shared memory with coalesced loads, and each thread applies
// the reference's per-point box test before it scans the staged points.  (N/256)^2 box tests instead of
// N * N/256.  Distances are evaluated with round-to-nearest operations in a fixed order, so a host program
// reproduces every bit.
#include <cfloat>

#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kBox = 256;
constexpr int kMaxK = 8;
constexpr int kChunk = 1024;      // boxes culled per round

struct KnnArgs {
    const float* points;
    int64_t stride;        // floats between consecutive points
    int64_t n;
    const float* pmin;     // [3] on the device
    const float* pmax;     // [3]
    int bits;              // Morton bits per axis: 10 or 21
    uint64_t* keys;
    int32_t* values;
    const int32_t* sorted;     // point index at every sorted position
    float4* sorted_pts;        // x, y, z, bit pattern of the point index
    float* boxes;              // [num_box, 6] min xyz, max xyz
    float* out;                // [n, k] ascending distances
    int64_t num_box;
};

__device__ __forceinline__ uint64_t spread3(uint64_t v) {   // every bit of a 21-bit value to every third position
    v &= 0x1fffffull;
    v = (v | v << 32) & 0x1f00000000ffffull;
    v = (v | v << 16) & 0x1f0000ff0000ffull;
    v = (v | v << 8) & 0x100f00f00f00f00full;
    v = (v | v << 4) & 0x10c30c30c30c30c3ull;
    v = (v | v << 2) & 0x1249249249249249ull;
    return v;
}

__global__ void __launch_bounds__(256) morton_kernel(const KnnArgs a) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= a.n) return;
    const float* p = a.points + i * a.stride;
    const float scale = (float)((1u << a.bits) - 1u);
    uint64_t code = 0;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        const float ext = f_sub(a.pmax[c], a.pmin[c]);
        // ops.py:37-38: (point - min) / (max - min) * (2^bits - 1), truncated; a flat axis gives 0
        const float rel = ext > 0.0f ? f_mul(f_div(f_sub(p[c], a.pmin[c]), ext), scale) : 0.0f;
        code |= spread3((uint64_t)fminf(fmaxf(rel, 0.0f), scale)) << c;
    }
    a.keys[i] = code;
    a.values[i] = (int32_t)i;
}

// sorted order -> compact float4 rows, and every box's bounds (ops.py:45-122)
__global__ void __launch_bounds__(kBox) gather_box_kernel(const KnnArgs a) {
    const int t = threadIdx.x;
    const int64_t i = (int64_t)blockIdx.x * kBox + t;
    float lo[3] = {FLT_MAX, FLT_MAX, FLT_MAX}, hi[3] = {-FLT_MAX, -FLT_MAX, -FLT_MAX};
    if (i < a.n) {
        const int32_t idx = a.sorted[i];
        const float* p = a.points + (int64_t)idx * a.stride;
        const float x = p[0], y = p[1], z = p[2];
        a.sorted_pts[i] = make_float4(x, y, z, __int_as_float(idx));
        lo[0] = hi[0] = x; lo[1] = hi[1] = y; lo[2] = hi[2] = z;
    }
    __shared__ float s_red[kBox / 32][6];
#pragma unroll
    for (int c = 0; c < 3; ++c) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo[c] = fminf(lo[c], __shfl_xor_sync(0xffffffffu, lo[c], o));
            hi[c] = fmaxf(hi[c], __shfl_xor_sync(0xffffffffu, hi[c], o));
        }
    }
    if ((t & 31) == 0) {
#pragma unroll
        for (int c = 0; c < 3; ++c) { s_red[t >> 5][c] = lo[c]; s_red[t >> 5][3 + c] = hi[c]; }
    }
    __syncthreads();
    if (t < 6) {
        float v = s_red[0][t];
        for (int w = 1; w < kBox / 32; ++w) v = t < 3 ? fminf(v, s_red[w][t]) : fmaxf(v, s_red[w][t]);
        a.boxes[(int64_t)blockIdx.x * 6 + t] = v;
    }
}

__device__ __forceinline__ float dist2(const float4& p, float x, float y, float z) {
    const float dx = f_sub(x, p.x), dy = f_sub(y, p.y), dz = f_sub(z, p.z);
    return f_add(f_add(f_mul(dx, dx), f_mul(dy, dy)), f_mul(dz, dz));
}

template <int K>
__device__ __forceinline__ void insert(float (&best)[K], float d) {   // ops.py:135-141: keeps best ascending
#pragma unroll
    for (int k = 0; k < K; ++k) {
        if (best[k] > d) {
            const float tmp = best[k];
            best[k] = d;
            d = tmp;
        }
    }
}

// squared distance from a point to an axis-aligned box as the reference measures it (ops.py:147-154): per axis
// the distance to the nearer face when outside, else 0
__device__ __forceinline__ float box_dist2(const float4& p, const float* bx) {
    float d[3] = {0.0f, 0.0f, 0.0f};
    const float c[3] = {p.x, p.y, p.z};
#pragma unroll
    for (int k = 0; k < 3; ++k)
        if (c[k] < bx[k] || c[k] > bx[3 + k]) d[k] = fminf(fabsf(f_sub(c[k], bx[k])), fabsf(f_sub(c[k], bx[3 + k])));
    return f_add(f_add(f_mul(d[0], d[0]), f_mul(d[1], d[1])), f_mul(d[2], d[2]));
}

template <int K>
__global__ void __launch_bounds__(kBox) knn_kernel(const KnnArgs a) {
    __shared__ float4 s_pts[kBox];
    __shared__ float s_box[6];
    __shared__ float s_red[kBox / 32];
    __shared__ int s_list[kChunk];
    __shared__ int s_count;
    const int t = threadIdx.x;
    const int64_t i = (int64_t)blockIdx.x * kBox + t;
    const bool valid = i < a.n;
    const float4 p = valid ? a.sorted_pts[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float best[K];
#pragma unroll
    for (int k = 0; k < K; ++k) best[k] = FLT_MAX;
    // ops.py:128-143: the k-th distance among the 2k neighbours in sorted order bounds the true k-th distance
    if (valid) {
        const int64_t j0 = i - K < 0 ? 0 : i - K, j1 = i + K > a.n - 1 ? a.n - 1 : i + K;
        for (int64_t j = j0; j <= j1; ++j) {
            if (j == i) continue;
            const float4 q = a.sorted_pts[j];
            insert<K>(best, dist2(p, q.x, q.y, q.z));
        }
    }
    const float reject = best[K - 1];
#pragma unroll
    for (int k = 0; k < K; ++k) best[k] = FLT_MAX;
    // the largest bound of the CTA: a box farther than that from the CTA's own bounds matters to none of its points
    float r = valid ? reject : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
    if ((t & 31) == 0) s_red[t >> 5] = r;
    if (t < 6) s_box[t] = a.boxes[(int64_t)blockIdx.x * 6 + t];
    __syncthreads();
    float radius2 = s_red[0];
    for (int w = 1; w < kBox / 32; ++w) radius2 = fmaxf(radius2, s_red[w]);
    float own[6];
#pragma unroll
    for (int k = 0; k < 6; ++k) own[k] = s_box[k];

    for (int64_t c0 = 0; c0 < a.num_box; c0 += kChunk) {
        if (t == 0) s_count = 0;
        __syncthreads();
        for (int64_t b = c0 + t; b < a.num_box && b < c0 + kChunk; b += kBox) {
            const float* bx = a.boxes + b * 6;
            // gap between the two boxes per axis; its square norm never exceeds the distance of any pair of points
            float g2 = 0.0f;
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float gap = fmaxf(fmaxf(bx[k] - own[3 + k], own[k] - bx[3 + k]), 0.0f);
                g2 = fmaf(gap, gap, g2);
            }
            // g2 is rounded, so keep a margin: a box is dropped only when it is clearly out of reach
            if (!(g2 * 0.999f > radius2)) s_list[atomicAdd(&s_count, 1)] = (int)(b - c0);
        }
        __syncthreads();
        const int cnt = s_count;
        for (int e = 0; e < cnt; ++e) {
            const int64_t b = c0 + s_list[e];
            const int64_t j = b * kBox + t;
            __syncthreads();        // the previous box's points are no longer read
            if (j < a.n) s_pts[t] = a.sorted_pts[j];
            __syncthreads();
            if (!valid) continue;
            const float bd = box_dist2(p, a.boxes + b * 6);
            if (bd > reject || bd > best[K - 1]) continue;       // ops.py:156
            const int m = (int)min((int64_t)kBox, a.n - b * kBox);
            const int self = b == blockIdx.x ? t : -1;
            for (int q = 0; q < m; ++q) {
                if (q == self) continue;
                const float4 c = s_pts[q];
                insert<K>(best, dist2(p, c.x, c.y, c.z));
            }
        }
        __syncthreads();
    }
    if (valid) {
        float* dst = a.out + (int64_t)__float_as_int(p.w) * K;
#pragma unroll
        for (int k = 0; k < K; ++k) dst[k] = f_sqrt(best[k]);     // ops.py:170
    }
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Layout {
    size_t keys, keys_alt, vals, vals_alt, pts, boxes, sort, total;
};

Layout layout(int64_t n, int bits) {
    Layout l;
    size_t o = 0;
    l.keys = o; o += align256((size_t)n * 8);
    l.keys_alt = o; o += align256((size_t)n * 8);
    l.vals = o; o += align256((size_t)n * 4);
    l.vals_alt = o; o += align256((size_t)n * 4);
    l.pts = o; o += align256((size_t)n * 16);
    l.boxes = o; o += align256((size_t)div_up64(n, kBox) * 6 * 4);
    l.sort = o; o += align256(d3gs_sort_workspace_bytes(n, 0, bits * 3));
    l.total = o;
    return l;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" size_t d3gs_simple_knn_workspace_bytes(int64_t n, int32_t morton_bits) {
    if (n <= 0 || (morton_bits != 10 && morton_bits != 21)) return 0;
    return layout(n, morton_bits).total;
}

extern "C" int32_t d3gs_simple_knn(const float* points, int64_t point_stride, int64_t n, int32_t k, int32_t morton_bits,
                                   const float* points_min, const float* points_max, float* out, void* workspace,
                                   size_t workspace_bytes, uint32_t* status, void* stream) {
    D3GS_REQUIRE(n >= 0 && n < ((int64_t)1 << 31), "point count out of range");
    D3GS_REQUIRE(k >= 1 && k <= kMaxK, "k must be in [1, %d] (got %d)", kMaxK, k);
    D3GS_REQUIRE(morton_bits == 10 || morton_bits == 21, "morton_bits must be 10 or 21");
    D3GS_REQUIRE(point_stride >= 3, "point_stride must be at least 3 floats");
    if (n == 0) return D3GS_OK;
    D3GS_REQUIRE(points && points_min && points_max && out && workspace && status, "NULL argument");
    const Layout l = layout(n, morton_bits);
    D3GS_REQUIRE(workspace_bytes >= l.total, "workspace too small: %zu < %zu", workspace_bytes, l.total);
    D3GS_REQUIRE(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    char* ws = static_cast<char*>(workspace);
    KnnArgs a = {};
    a.points = points;
    a.stride = point_stride;
    a.n = n;
    a.pmin = points_min;
    a.pmax = points_max;
    a.bits = morton_bits;
    a.keys = reinterpret_cast<uint64_t*>(ws + l.keys);
    a.values = reinterpret_cast<int32_t*>(ws + l.vals);
    a.sorted_pts = reinterpret_cast<float4*>(ws + l.pts);
    a.boxes = reinterpret_cast<float*>(ws + l.boxes);
    a.out = out;
    a.num_box = div_up64(n, kBox);
    morton_kernel<<<(unsigned)div_up64(n, 256), 256, 0, s>>>(a);
    D3GS_LAUNCH_CHECK("morton_kernel");
    int32_t in_alt = 0;
    int32_t rc = d3gs_sort_pairs(a.keys, reinterpret_cast<uint64_t*>(ws + l.keys_alt), a.values,
                                 reinterpret_cast<int32_t*>(ws + l.vals_alt), n, 0, morton_bits * 3, ws + l.sort,
                                 l.total - l.sort, &in_alt, status, stream);
    if (rc != D3GS_OK) return rc;
    a.sorted = in_alt ? reinterpret_cast<int32_t*>(ws + l.vals_alt) : a.values;
    gather_box_kernel<<<(unsigned)a.num_box, kBox, 0, s>>>(a);
    D3GS_LAUNCH_CHECK("gather_box_kernel");
    switch (k) {
#define D3GS_KNN_CASE(K) \
    case K: knn_kernel<K><<<(unsigned)a.num_box, kBox, 0, s>>>(a); break;
        D3GS_KNN_CASE(1) D3GS_KNN_CASE(2) D3GS_KNN_CASE(3) D3GS_KNN_CASE(4)
        D3GS_KNN_CASE(5) D3GS_KNN_CASE(6) D3GS_KNN_CASE(7) D3GS_KNN_CASE(8)
#undef D3GS_KNN_CASE
    }
    D3GS_LAUNCH_CHECK("knn_kernel");
    return D3GS_OK;
}
