// K11 + K12: one launch that applies Adam to every parameter tensor of the Gaussian model and
// accumulates the densification statistics.
//
// Reference semantics: d3sim/ops/optim/adam.py:32-148 (fused_adam_single_tensor_step, launched
// once per tensor from GaussianAdam.step, 382-418 -- six launches per iteration), scalar update
// d3sim/csrc/optim.py:22-49, statistics kernel d3sim/algos/d3gs/origin/strategy.py:93-122.
// Here all tensors are "segments" of one grid: CTA -> (segment, chunk) by a prefix table in the
// kernel arguments; the statistics are a further segment of the same grid.
#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kMaxSegments = 8;
constexpr int kAdamThreads = 256;
constexpr int kAdamVec = 4;
constexpr int kAdamUnroll = 4;
constexpr int kAdamChunk = kAdamThreads * kAdamVec * kAdamUnroll;   // 4096 floats per CTA

struct AdamArgs {
    D3gsAdamSegment seg[kMaxSegments];
    int64_t block_start[kMaxSegments + 2];   // first CTA of each segment; [num_segments] = stats; last = end
    int32_t num_segments;
    int32_t has_stats;
    D3gsDensifyStats stats;
};

// csrc/optim.py:22-49 (weight decay 0 / plain Adam path kept as in the reference)
__device__ __forceinline__ void adam_update(float g, float& p, float& m, float& v, const D3gsAdamSegment& s) {
    g = g / s.grad_scale;
    if (s.weight_decay != 0.0f) g += p * s.weight_decay;
    m = g * (1.0f - s.beta1) + m * s.beta1;            // mix(grad, exp_avg, beta1)
    v = (g * g) * (1.0f - s.beta2) + v * s.beta2;
    const float step_size = s.lr / s.bias_correction1;
    const float denom = sqrtf(v) / s.bias_correction2_sqrt + s.eps;
    p = p - step_size * m / denom;
}

__device__ __forceinline__ void stats_update(const D3gsDensifyStats& st, int64_t i) {
    float la = 0.0f, ca = 0.0f, mr = st.need_max_radii ? st.max_radii[i] : 0.0f;
    const float lb = (float)(st.loss_batch > 0 ? st.loss_batch : st.batch);
    const float sx = 0.5f * (float)st.width * lb, sy = 0.5f * (float)st.height * lb;
    const float mwh = (float)max(st.width, st.height);
    for (int j = 0; j < st.batch; ++j) {
        const int64_t k = (int64_t)j * st.num + i;
        const float2 d = *reinterpret_cast<const float2*>(st.duv + k * 2);
        const float a = d.x * sx, b = d.y * sy;
        const float len = sqrtf(a * a + b * b);
        const int r = st.radii[k];
        if (r > 0) {
            la += len;
            ca += 1.0f;
            if (st.need_max_radii) mr = fmaxf(mr, (float)r / mwh);
        }
    }
    st.duv_ndc_length[i] += la;
    st.count[i] += ca;
    if (st.need_max_radii) st.max_radii[i] = mr;
}

__global__ void __launch_bounds__(kAdamThreads) adam_stats_kernel(const __grid_constant__ AdamArgs a) {
    const int64_t blk = blockIdx.x;
    int si = 0;
#pragma unroll
    for (int k = 1; k <= kMaxSegments; ++k)
        if (k <= a.num_segments && blk >= a.block_start[k]) si = k;
    if (si == a.num_segments) {   // statistics segment
        const int64_t i = (blk - a.block_start[si]) * kAdamThreads + threadIdx.x;
        if (a.has_stats && i < a.stats.num) stats_update(a.stats, i);
        return;
    }
    const D3gsAdamSegment& s = a.seg[si];
    const int64_t base = (blk - a.block_start[si]) * kAdamChunk;
    const bool vec_ok = (((uintptr_t)s.param | (uintptr_t)s.grad | (uintptr_t)s.exp_avg | (uintptr_t)s.exp_avg_sq) & 15) == 0;
    if (vec_ok && base + kAdamChunk <= s.count) {
        float4 p[kAdamUnroll], g[kAdamUnroll], m[kAdamUnroll], v[kAdamUnroll];
#pragma unroll
        for (int u = 0; u < kAdamUnroll; ++u) {
            const int64_t o = base / 4 + u * kAdamThreads + threadIdx.x;
            p[u] = reinterpret_cast<const float4*>(s.param)[o];
            g[u] = __ldcs(reinterpret_cast<const float4*>(s.grad) + o);
            m[u] = reinterpret_cast<const float4*>(s.exp_avg)[o];
            v[u] = reinterpret_cast<const float4*>(s.exp_avg_sq)[o];
        }
#pragma unroll
        for (int u = 0; u < kAdamUnroll; ++u) {
            adam_update(g[u].x, p[u].x, m[u].x, v[u].x, s);
            adam_update(g[u].y, p[u].y, m[u].y, v[u].y, s);
            adam_update(g[u].z, p[u].z, m[u].z, v[u].z, s);
            adam_update(g[u].w, p[u].w, m[u].w, v[u].w, s);
        }
#pragma unroll
        for (int u = 0; u < kAdamUnroll; ++u) {
            const int64_t o = base / 4 + u * kAdamThreads + threadIdx.x;
            reinterpret_cast<float4*>(s.param)[o] = p[u];
            reinterpret_cast<float4*>(s.exp_avg)[o] = m[u];
            reinterpret_cast<float4*>(s.exp_avg_sq)[o] = v[u];
        }
    } else {
        for (int64_t o = base + threadIdx.x; o < min(base + (int64_t)kAdamChunk, s.count); o += kAdamThreads) {
            float p = s.param[o], m = s.exp_avg[o], v = s.exp_avg_sq[o];
            adam_update(s.grad[o], p, m, v, s);
            s.param[o] = p;
            s.exp_avg[o] = m;
            s.exp_avg_sq[o] = v;
        }
    }
}

int32_t check_stats(const D3gsDensifyStats* st) {
    D3GS_REQUIRE(st->num >= 0 && st->batch >= 1, "bad stats shape");
    D3GS_REQUIRE(st->duv && st->radii && st->duv_ndc_length && st->count, "NULL stats tensor");
    D3GS_REQUIRE(!st->need_max_radii || st->max_radii, "max_radii is NULL");
    D3GS_REQUIRE(((uintptr_t)st->duv & 7) == 0, "duv must be 8-byte aligned");
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" int32_t d3gs_adam_stats_step(const D3gsAdamSegment* segments, int32_t num_segments,
                                        const D3gsDensifyStats* stats, void* stream) {
    D3GS_REQUIRE(num_segments >= 0 && num_segments <= kMaxSegments, "num_segments %d outside [0,%d]", num_segments,
                 kMaxSegments);
    D3GS_REQUIRE(num_segments == 0 || segments != nullptr, "segments is NULL");
    AdamArgs a = {};
    a.num_segments = num_segments;
    int64_t blocks = 0;
    for (int k = 0; k < num_segments; ++k) {
        const D3gsAdamSegment& s = segments[k];
        D3GS_REQUIRE(s.count >= 0, "segment %d: negative count", k);
        D3GS_REQUIRE(s.count == 0 || (s.param && s.grad && s.exp_avg && s.exp_avg_sq), "segment %d: NULL tensor", k);
        D3GS_REQUIRE(s.grad_scale != 0.0f && s.bias_correction1 != 0.0f && s.bias_correction2_sqrt != 0.0f,
                     "segment %d: zero grad_scale / bias correction", k);
        a.seg[k] = s;
        a.block_start[k] = blocks;
        blocks += div_up64(s.count, kAdamChunk);
    }
    a.block_start[num_segments] = blocks;
    a.has_stats = 0;
    if (stats != nullptr) {
        int32_t rc = check_stats(stats);
        if (rc != D3GS_OK) return rc;
        a.has_stats = 1;
        a.stats = *stats;
        blocks += div_up64(stats->num, kAdamThreads);
    }
    for (int k = num_segments + 1; k < kMaxSegments + 2; ++k) a.block_start[k] = blocks;
    if (blocks == 0) return D3GS_OK;
    D3GS_REQUIRE(blocks < ((int64_t)1 << 31), "too many CTAs");
    adam_stats_kernel<<<(unsigned)blocks, kAdamThreads, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("adam_stats_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_densify_stats(const D3gsDensifyStats* stats, void* stream) {
    D3GS_REQUIRE(stats != nullptr, "stats is NULL");
    return d3gs_adam_stats_step(nullptr, 0, stats, stream);
}
