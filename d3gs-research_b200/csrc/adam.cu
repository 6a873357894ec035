// K11 + K12: one launch that applies Adam to every parameter tensor of the Gaussian model and
// accumulates the densification statistics.
//
// Reference semantics: d3sim/ops/optim/adam.py:32-148 (fused_adam_single_tensor_step, launched
// once per tensor from GaussianAdam.step, 382-418 -- six launches per iteration), scalar update
// d3sim/csrc/optim.py:22-49, statistics kernel d3sim/algos/d3gs/origin/strategy.py:93-122.
// Here all tensors are "segments" of one grid: CTA -> (segment, chunk) by a prefix table in the
// kernel arguments; the statistics are a further segment of the same grid.
//
// Data-parallel variant (adam_peers_kernel): the gradient of an element is the sum, in rank order, of
// that element in every rank's gradient buffer, read through NVLink peer mappings, and the updated
// parameter is stored into every rank's parameter buffer.  A rank runs it over its own slice only, so
// the reduce-scatter, the update and the all-gather of a sharded optimizer are one pass in which
// gradients arrive and parameters leave over the two directions of the links at the same time.
// A load over NVLink takes several times as long as one from local HBM; to keep ~100 KB per SM in
// flight without spending registers, each CTA stages its chunk of every rank's gradients in shared
// memory with bulk async copies (64 KB per CTA, three CTAs per SM).
#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kMaxSegments = 8;
constexpr int kAdamThreads = 256;
constexpr int kAdamVec = 4;
constexpr int kAdamUnroll = 2;
constexpr int kAdamChunk = kAdamThreads * kAdamVec * kAdamUnroll;   // 2048 floats per CTA

struct AdamArgs {
    D3gsAdamSegment seg[kMaxSegments];
    SegConst sc[kMaxSegments];
    int64_t block_start[kMaxSegments + 2];   // first CTA of each segment; [num_segments] = stats; last = end
    int32_t num_segments;
    int32_t has_stats;
    D3gsDensifyStats stats;
    // peer variant: floats per CTA and rank, element offsets of each segment inside the flat buffers, and
    // the buffers of every rank
    int64_t chunk;
    int64_t param_off[kMaxSegments], grad_off[kMaxSegments];
    D3gsPeerSet peers;
};

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
    const SegConst c = a.sc[si];
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
            adam_update(g[u].x, p[u].x, m[u].x, v[u].x, c);
            adam_update(g[u].y, p[u].y, m[u].y, v[u].y, c);
            adam_update(g[u].z, p[u].z, m[u].z, v[u].z, c);
            adam_update(g[u].w, p[u].w, m[u].w, v[u].w, c);
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
            adam_update(s.grad[o], p, m, v, c);
            s.param[o] = p;
            s.exp_avg[o] = m;
            s.exp_avg_sq[o] = v;
        }
    }
}

constexpr int kPeerSmemBytes = 64 * 1024;

__device__ __forceinline__ void add4(float4& a, const float4 b) {
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
}

__global__ void __launch_bounds__(kAdamThreads) adam_peers_kernel(const __grid_constant__ AdamArgs a) {
    extern __shared__ __align__(128) unsigned char s_raw[];
    __shared__ __align__(8) uint64_t s_bar;
    const int64_t blk = blockIdx.x;
    const int tid = threadIdx.x;
    int si = 0;
#pragma unroll
    for (int k = 1; k <= kMaxSegments; ++k)
        if (k <= a.num_segments && blk >= a.block_start[k]) si = k;
    if (si == a.num_segments) {   // statistics segment
        const int64_t i = (blk - a.block_start[si]) * kAdamThreads + tid;
        if (a.has_stats && i < a.stats.num) stats_update(a.stats, i);
        return;
    }
    const D3gsAdamSegment& s = a.seg[si];
    const SegConst c = a.sc[si];
    const int world = a.peers.world;
    const int64_t chunk = a.chunk;
    const int64_t base = (blk - a.block_start[si]) * chunk;
    const int64_t goff = a.grad_off[si] + base, poff = a.param_off[si] + base;
    uintptr_t bits = (uintptr_t)(s.param + base) | (uintptr_t)(s.exp_avg + base) | (uintptr_t)(s.exp_avg_sq + base);
    for (int q = 0; q < world; ++q) bits |= (uintptr_t)(a.peers.grad[q] + goff) | (uintptr_t)(a.peers.param[q] + poff);
    if ((bits & 15) == 0 && base + chunk <= s.count) {
        float4* s_g = reinterpret_cast<float4*>(s_raw);     // [world][chunk / 4]
        const int64_t chunk4 = chunk / 4;
        if (tid == 0) {
            mbar_init(&s_bar, 1);
            fence_mbar_init();
        }
        __syncthreads();
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)(chunk * sizeof(float));
            mbar_arrive_expect_tx(&s_bar, bytes * (uint32_t)world);
            for (int q = 0; q < world; ++q) bulk_copy_g2s(s_g + q * chunk4, a.peers.grad[q] + goff, bytes, &s_bar);
        }
        bool arrived = mbar_wait_bounded(&s_bar, 0);
        if (__syncthreads_or(!arrived)) {
            // give the copies one more bounded wait before the shared memory is released, flag, and leave
            // this chunk unchanged
            if (!arrived) mbar_wait_bounded(&s_bar, 0);
            if (tid == 0 && a.peers.status != nullptr) atomicOr(a.peers.status, D3GS_STATUS_COPY_TIMEOUT);
            return;
        }
        for (int64_t st = 0; st < chunk4; st += kAdamUnroll * kAdamThreads) {
            float4 p[kAdamUnroll], g[kAdamUnroll], m[kAdamUnroll], v[kAdamUnroll];
#pragma unroll
            for (int u = 0; u < kAdamUnroll; ++u) {
                const int64_t o = st + u * kAdamThreads + tid;
                p[u] = reinterpret_cast<const float4*>(s.param + base)[o];
                m[u] = reinterpret_cast<const float4*>(s.exp_avg + base)[o];
                v[u] = reinterpret_cast<const float4*>(s.exp_avg_sq + base)[o];
                g[u] = s_g[o];
                // the sum runs in rank order on every rank: all replicas of an element come from the same bits
                for (int q = 1; q < world; ++q) add4(g[u], s_g[q * chunk4 + o]);
            }
#pragma unroll
            for (int u = 0; u < kAdamUnroll; ++u) {
                adam_update(g[u].x, p[u].x, m[u].x, v[u].x, c);
                adam_update(g[u].y, p[u].y, m[u].y, v[u].y, c);
                adam_update(g[u].z, p[u].z, m[u].z, v[u].z, c);
                adam_update(g[u].w, p[u].w, m[u].w, v[u].w, c);
            }
#pragma unroll
            for (int u = 0; u < kAdamUnroll; ++u) {
                const int64_t o = st + u * kAdamThreads + tid;
                for (int q = 0; q < world; ++q) reinterpret_cast<float4*>(a.peers.param[q] + poff)[o] = p[u];
                reinterpret_cast<float4*>(s.exp_avg + base)[o] = m[u];
                reinterpret_cast<float4*>(s.exp_avg_sq + base)[o] = v[u];
            }
        }
    } else {
        for (int64_t o = base + tid; o < min(base + chunk, s.count); o += kAdamThreads) {
            float p = s.param[o], m = s.exp_avg[o], v = s.exp_avg_sq[o];
            float g = __ldcg(a.peers.grad[0] + a.grad_off[si] + o);
            for (int q = 1; q < world; ++q) g += __ldcg(a.peers.grad[q] + a.grad_off[si] + o);
            adam_update(g, p, m, v, c);
            for (int q = 0; q < world; ++q) a.peers.param[q][a.param_off[si] + o] = p;
            s.exp_avg[o] = m;
            s.exp_avg_sq[o] = v;
        }
    }
}

int32_t check_stats(const D3gsDensifyStats* st) {
    D3GS_REQUIRE(st->num >= 0 && st->batch >= 1, "bad stats shape");
    D3GS_REQUIRE(st->duv && st->radii && st->duv_ndc_length && st->count, "NULL stats tensor");
    D3GS_REQUIRE(!st->need_max_radii || st->max_radii, "max_radii is NULL");
    D3GS_REQUIRE(((uintptr_t)st->duv & 7) == 0 && (st->duv_stride & 1) == 0, "duv must be 8-byte aligned, stride even");
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

static int32_t adam_launch(const D3gsAdamSegment* segments, int32_t num_segments, const D3gsDensifyStats* stats,
                           const D3gsPeerSet* peers, void* stream) {
    D3GS_REQUIRE(num_segments >= 0 && num_segments <= kMaxSegments, "num_segments %d outside [0,%d]", num_segments,
                 kMaxSegments);
    D3GS_REQUIRE(num_segments == 0 || segments != nullptr, "segments is NULL");
    AdamArgs a = {};
    a.num_segments = num_segments;
    a.chunk = kAdamChunk;
    if (peers != nullptr) {
        D3GS_REQUIRE(peers->world >= 1 && peers->world <= D3GS_MAX_PEERS, "world %d outside [1,%d]", peers->world,
                     D3GS_MAX_PEERS);
        D3GS_REQUIRE(peers->rank >= 0 && peers->rank < peers->world, "rank %d outside the world", peers->rank);
        for (int q = 0; q < peers->world; ++q)
            D3GS_REQUIRE(peers->grad[q] != nullptr && peers->param[q] != nullptr, "peer %d: NULL buffer", q);
        a.peers = *peers;
        // floats per CTA and rank: the largest power of two with world * chunk * 4 bytes <= 64 KB
        a.chunk = kPeerSmemBytes / 4 / 2;
        while (a.chunk * peers->world * 4 > kPeerSmemBytes) a.chunk /= 2;
    }
    int64_t blocks = 0;
    for (int k = 0; k < num_segments; ++k) {
        const D3gsAdamSegment& s = segments[k];
        D3GS_REQUIRE(s.count >= 0, "segment %d: negative count", k);
        D3GS_REQUIRE(s.count == 0 || (s.param && s.grad && s.exp_avg && s.exp_avg_sq), "segment %d: NULL tensor", k);
        D3GS_REQUIRE(s.grad_scale != 0.0f && s.bias_correction1 != 0.0f && s.bias_correction2_sqrt != 0.0f,
                     "segment %d: zero grad_scale / bias correction", k);
        a.seg[k] = s;
        if (peers != nullptr && s.count > 0) {
            a.param_off[k] = s.param - peers->param[peers->rank];
            a.grad_off[k] = s.grad - peers->grad[peers->rank];
            D3GS_REQUIRE(a.param_off[k] >= 0 && a.grad_off[k] >= 0,
                         "segment %d does not lie inside this rank's flat buffers", k);
        }
        a.sc[k] = make_seg_const(s);
        a.block_start[k] = blocks;
        blocks += div_up64(s.count, a.chunk);
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
    if (peers != nullptr) {
        D3GS_CUDA(cudaFuncSetAttribute(adam_peers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeerSmemBytes));
        adam_peers_kernel<<<(unsigned)blocks, kAdamThreads, kPeerSmemBytes, (cudaStream_t)stream>>>(a);
    } else {
        adam_stats_kernel<<<(unsigned)blocks, kAdamThreads, 0, (cudaStream_t)stream>>>(a);
    }
    D3GS_LAUNCH_CHECK("adam_stats_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_adam_stats_step(const D3gsAdamSegment* segments, int32_t num_segments,
                                        const D3gsDensifyStats* stats, void* stream) {
    return adam_launch(segments, num_segments, stats, nullptr, stream);
}

extern "C" int32_t d3gs_adam_stats_step_peers(const D3gsAdamSegment* segments, int32_t num_segments,
                                              const D3gsDensifyStats* stats, const D3gsPeerSet* peers,
                                              void* stream) {
    D3GS_REQUIRE(peers != nullptr, "peers is NULL");
    return adam_launch(segments, num_segments, stats, peers, stream);
}

extern "C" int32_t d3gs_densify_stats(const D3gsDensifyStats* stats, void* stream) {
    D3GS_REQUIRE(stats != nullptr, "stats is NULL");
    return d3gs_adam_stats_step(nullptr, 0, stats, stream);
}
