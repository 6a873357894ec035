// sparse_mode (d3sim/algos/d3gs/config_def.py:119; render.py:235-238, 478-499, 622-637, 2860-2903): the
// per-(view, Gaussian) tensors the forward keeps for the backward hold the VISIBLE items only, with two index lists
// that say which Gaussian and which view every kept item is.
//
// The reference compacts inside its preprocess kernel with an atomic counter (items land in arrival order) after a
// first pass that only counts.  Here the preprocess runs once, dense, and the kept items are compacted afterwards
// in flat-index order (a scan of the visibility flags gives every item its row): deterministic, and the relative
// order of the items -- which breaks depth ties in the sort -- is the dense one, so the sorted lists are the dense
// lists with the indices renumbered.  For the backward the compact rows are spread out again over zero-filled
// dense arrays of what the preprocess backward reads (16 + 48 bytes per item); what is held between forward and
// backward is compact.
#include "common.cuh"

namespace d3gs {
namespace {

// flags[i] = item i is kept.  views > 1 with per_gaussian: flags[g] = some view keeps Gaussian g.
__global__ void __launch_bounds__(256) sparse_flags_kernel(const int32_t* __restrict__ radii, int64_t count, int64_t num,
                                                           int views, int per_gaussian, int32_t* __restrict__ flags) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= count) return;
    int f = 0;
    if (per_gaussian) {
        for (int b = 0; b < views; ++b) f |= radii[(int64_t)b * num + i] != 0;
    } else {
        f = radii[i] != 0;
    }
    flags[i] = f;
}

struct CompactArgs {
    D3gsSplatContext dense, compact;
    const int32_t* scan;        // inclusive scan of the flags
    int64_t count, num;
    int32_t* gaussian_ids;
    int32_t* batch_ids;
};

__global__ void __launch_bounds__(256) sparse_compact_kernel(const CompactArgs a) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= a.count) return;
    const int32_t r = a.dense.radii[i];
    if (r == 0) return;
    const int64_t p = (int64_t)a.scan[i] - 1;
    const int64_t b = i / a.num;
    a.gaussian_ids[p] = (int32_t)(i - b * a.num);
    a.batch_ids[p] = (int32_t)b;
    a.compact.radii[p] = r;
    a.compact.depths[p] = a.dense.depths[i];
    *reinterpret_cast<float2*>(a.compact.uvs + p * 2) = *reinterpret_cast<const float2*>(a.dense.uvs + i * 2);
    *reinterpret_cast<float4*>(a.compact.conic_opacity + p * 4) = *reinterpret_cast<const float4*>(a.dense.conic_opacity + i * 4);
#pragma unroll
    for (int k = 0; k < 3; ++k) a.compact.rgb_gaussian[p * 3 + k] = a.dense.rgb_gaussian[i * 3 + k];
    if (a.dense.cov2d_vecs != nullptr) {
#pragma unroll
        for (int k = 0; k < 3; ++k) a.compact.cov2d_vecs[p * 3 + k] = a.dense.cov2d_vecs[i * 3 + k];
    }
    if (a.dense.sh_to_rgb_ne_0 != nullptr) a.compact.sh_to_rgb_ne_0[p] = a.dense.sh_to_rgb_ne_0[i];
    if (a.dense.records != nullptr) {
        const float4* s = reinterpret_cast<const float4*>(a.dense.records + i * D3GS_SPLAT_RECORD_FLOATS);
        float4* d = reinterpret_cast<float4*>(a.compact.records + p * D3GS_SPLAT_RECORD_FLOATS);
        d[0] = s[0]; d[1] = s[1]; d[2] = s[2];
    }
}

__global__ void __launch_bounds__(256) sparse_remap_kernel(int32_t* __restrict__ ids, int64_t n, const int32_t* __restrict__ scan) {
    const int64_t k = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (k < n) ids[k] = scan[ids[k]] - 1;
}

struct ExpandArgs {
    int64_t kept, num;
    const int32_t* gaussian_ids;
    const int32_t* batch_ids;
    const int32_t* radii;
    const float* cov2d;
    const uint8_t* ne0;
    const float* packed;
    int32_t* d_radii;
    float* d_cov2d;
    uint8_t* d_ne0;
    float* d_packed;
};

__global__ void __launch_bounds__(256) sparse_expand_kernel(const ExpandArgs a) {
    const int64_t p = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (p >= a.kept) return;
    const int64_t i = (int64_t)a.batch_ids[p] * a.num + a.gaussian_ids[p];
    a.d_radii[i] = a.radii[p];
#pragma unroll
    for (int k = 0; k < 3; ++k) a.d_cov2d[i * 3 + k] = a.cov2d[p * 3 + k];
    a.d_ne0[i] = a.ne0[p];
    const float4* s = reinterpret_cast<const float4*>(a.packed + p * D3GS_SPLAT_GRAD_FLOATS);
    float4* d = reinterpret_cast<float4*>(a.d_packed + i * D3GS_SPLAT_GRAD_FLOATS);
    d[0] = s[0]; d[1] = s[1]; d[2] = s[2];
}

// dst row p = src row index[p]; or, with flags + scan, the list of the flagged indices itself (src == NULL)
__global__ void __launch_bounds__(256) gather_rows_kernel(const float* __restrict__ src, int row_floats,
                                                          const int32_t* __restrict__ index, int64_t rows,
                                                          float* __restrict__ dst) {
    const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (e >= rows * row_floats) return;
    const int64_t p = e / row_floats;
    dst[e] = src[(int64_t)index[p] * row_floats + (e - p * row_floats)];
}

__global__ void __launch_bounds__(256) flagged_indices_kernel(const int32_t* __restrict__ flags, const int32_t* __restrict__ scan,
                                                              int64_t count, int32_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i < count && flags[i] != 0) out[scan[i] - 1] = (int32_t)i;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" int32_t d3gs_sparse_flags(const int32_t* radii, int64_t num, int32_t views, int32_t per_gaussian,
                                     int32_t* flags, void* stream) {
    D3GS_REQUIRE(num >= 0 && views >= 1, "bad sizes");
    const int64_t count = per_gaussian ? num : num * views;
    if (count == 0) return D3GS_OK;
    D3GS_REQUIRE(radii && flags, "NULL argument");
    sparse_flags_kernel<<<(unsigned)div_up64(count, 256), 256, 0, (cudaStream_t)stream>>>(radii, count, num, views,
                                                                                         per_gaussian, flags);
    D3GS_LAUNCH_CHECK("sparse_flags_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_sparse_compact(const D3gsSplatContext* dense, int64_t num, int32_t views, const int32_t* scan,
                                       const D3gsSplatContext* compact, int32_t* gaussian_ids, int32_t* batch_ids,
                                       void* stream) {
    D3GS_REQUIRE(dense && compact && scan && gaussian_ids && batch_ids, "NULL argument");
    D3GS_REQUIRE(dense->radii && dense->depths && dense->uvs && dense->conic_opacity && dense->rgb_gaussian,
                 "dense context tensor pointer is NULL");
    D3GS_REQUIRE(compact->radii && compact->depths && compact->uvs && compact->conic_opacity && compact->rgb_gaussian,
                 "compact context tensor pointer is NULL");
    D3GS_REQUIRE((dense->cov2d_vecs == nullptr) == (compact->cov2d_vecs == nullptr) &&
                     (dense->sh_to_rgb_ne_0 == nullptr) == (compact->sh_to_rgb_ne_0 == nullptr) &&
                     (dense->records == nullptr) == (compact->records == nullptr),
                 "dense and compact contexts must hold the same optional tensors");
    CompactArgs a;
    a.dense = *dense;
    a.compact = *compact;
    a.scan = scan;
    a.num = num;
    a.count = num * views;
    a.gaussian_ids = gaussian_ids;
    a.batch_ids = batch_ids;
    if (a.count == 0) return D3GS_OK;
    sparse_compact_kernel<<<(unsigned)div_up64(a.count, 256), 256, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("sparse_compact_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_sparse_remap(int32_t* sorted_values, int64_t n, const int32_t* scan, void* stream) {
    if (n == 0) return D3GS_OK;
    D3GS_REQUIRE(sorted_values && scan && n > 0, "NULL argument");
    sparse_remap_kernel<<<(unsigned)div_up64(n, 256), 256, 0, (cudaStream_t)stream>>>(sorted_values, n, scan);
    D3GS_LAUNCH_CHECK("sparse_remap_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_sparse_expand(int64_t kept, int64_t num, int32_t views, const int32_t* gaussian_ids,
                                      const int32_t* batch_ids, const int32_t* radii, const float* cov2d_vecs,
                                      const uint8_t* sh_to_rgb_ne_0, const float* splat_grads, int32_t* dense_radii,
                                      float* dense_cov2d_vecs, uint8_t* dense_sh_to_rgb_ne_0, float* dense_splat_grads,
                                      void* stream) {
    D3GS_REQUIRE(kept >= 0 && num >= 0 && views >= 1, "bad sizes");
    D3GS_REQUIRE(dense_radii && dense_cov2d_vecs && dense_sh_to_rgb_ne_0 && dense_splat_grads, "NULL dense argument");
    cudaStream_t s = (cudaStream_t)stream;
    // only the radii need clearing: the backward reads the other arrays where the radius is non-zero
    D3GS_CUDA(cudaMemsetAsync(dense_radii, 0, (size_t)num * views * sizeof(int32_t), s));
    if (kept == 0) return D3GS_OK;
    D3GS_REQUIRE(gaussian_ids && batch_ids && radii && cov2d_vecs && sh_to_rgb_ne_0 && splat_grads, "NULL compact argument");
    D3GS_REQUIRE((((uintptr_t)splat_grads | (uintptr_t)dense_splat_grads) & 15) == 0, "splat_grads must be 16-byte aligned");
    ExpandArgs a = {kept, num, gaussian_ids, batch_ids, radii, cov2d_vecs, sh_to_rgb_ne_0, splat_grads,
                    dense_radii, dense_cov2d_vecs, dense_sh_to_rgb_ne_0, dense_splat_grads};
    sparse_expand_kernel<<<(unsigned)div_up64(kept, 256), 256, 0, s>>>(a);
    D3GS_LAUNCH_CHECK("sparse_expand_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_gather_rows(const float* src, int32_t row_floats, const int32_t* index, int64_t rows, float* dst,
                                    void* stream) {
    D3GS_REQUIRE(rows >= 0 && row_floats >= 1, "bad sizes");
    if (rows == 0) return D3GS_OK;
    D3GS_REQUIRE(src && index && dst, "NULL argument");
    gather_rows_kernel<<<(unsigned)div_up64(rows * row_floats, 256), 256, 0, (cudaStream_t)stream>>>(src, row_floats, index,
                                                                                                   rows, dst);
    D3GS_LAUNCH_CHECK("gather_rows_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_flagged_indices(const int32_t* flags, const int32_t* scan, int64_t count, int32_t* out,
                                        void* stream) {
    if (count == 0) return D3GS_OK;
    D3GS_REQUIRE(flags && scan && out && count > 0, "NULL argument");
    flagged_indices_kernel<<<(unsigned)div_up64(count, 256), 256, 0, (cudaStream_t)stream>>>(flags, scan, count, out);
    D3GS_LAUNCH_CHECK("flagged_indices_kernel");
    return D3GS_OK;
}
