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
#include "exchange.cuh"

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
    int64_t total_blocks;   // chunks + statistics blocks; the exchange kernels walk them with a grid-sized stride
    int64_t chunk;
    int64_t param_off[kMaxSegments], grad_off[kMaxSegments];
    D3gsPeerSet peers;
    TestHooks hooks;
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
// a rank's share of one of the two staging buffers (64 KB / 2 / 4 B / world) must be a whole number of float4;
// the vector loop of adam_peers_kernel checks its index against the chunk, so any such size is safe
static_assert((kPeerSmemBytes / 2 / 4 / D3GS_MAX_PEERS) % 4 == 0 && kPeerSmemBytes / 2 / 4 / D3GS_MAX_PEERS >= 4,
              "a rank's share of a staging buffer must hold whole float4 vectors");

// ---- switch multicast (NVLink SHARP): one load returns the sum over all ranks' copies of an address, one store
// writes all ranks' copies.  The addresses come from a multicast mapping of the symmetric buffers.
__device__ __forceinline__ float4 multimem_ld_reduce_add_v4(const float* mc) {
    float4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(mc) : "memory");
    return r;
}
__device__ __forceinline__ float multimem_ld_reduce_add(const float* mc) {
    float r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];" : "=f"(r) : "l"(mc) : "memory");
    return r;
}
__device__ __forceinline__ void multimem_st_v4(float* mc, const float4 v) {
    asm volatile("multimem.st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void multimem_st(float* mc, float v) {
    asm volatile("multimem.st.global.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}

// The rank's slice through the switch: the gradient of an element is ONE multicast load (the switch adds the
// ranks' copies), the new parameter ONE multicast store.  Per GPU the links carry S/world + S in and out
// instead of 2 (world - 1) / world * S with plain peer accesses (S = bytes of the flat buffer).
// The grid is a few CTAs per SM and every CTA walks the chunks with a grid-sized stride: the launch-wide
// announcements at the start and the end (and the system-wide fence before the latter, which waits until the
// stores to the other GPUs have been acknowledged) are paid once per CTA, not once per chunk.
// Eight multicast loads (128 bytes) per thread are issued before the first result is used: a load through the switch
// takes several times as long as one from local HBM, and registers are the only place to keep them in flight.
constexpr int kMcUnroll = 8;
constexpr int kMcCtasPerSm = 3;
__global__ void __launch_bounds__(kAdamThreads, kMcCtasPerSm) adam_multimem_kernel(const __grid_constant__ AdamArgs a) {
    const int tid = threadIdx.x;
    const bool ready = exchange_begin(a.peers);
    for (int64_t blk = blockIdx.x; blk < a.total_blocks; blk += gridDim.x) {
        int si = 0;
#pragma unroll
        for (int k = 1; k <= kMaxSegments; ++k)
            if (k <= a.num_segments && blk >= a.block_start[k]) si = k;
        if (si == a.num_segments) {   // statistics segment
            const int64_t i = (blk - a.block_start[si]) * kAdamThreads + tid;
            if (a.has_stats && i < a.stats.num) stats_update(a.stats, i);
            continue;
        }
        if (!ready) continue;         // a rank never announced its gradients: leave the parameters alone
        const D3gsAdamSegment& s = a.seg[si];
        const SegConst c = a.sc[si];
        const int64_t base = (blk - a.block_start[si]) * a.chunk;
        const float* gmc = a.peers.grad_mc + a.grad_off[si] + base;
        float* pmc = a.peers.param_mc + a.param_off[si] + base;
        const uintptr_t bits = (uintptr_t)(s.param + base) | (uintptr_t)(s.exp_avg + base) |
                               (uintptr_t)(s.exp_avg_sq + base) | (uintptr_t)gmc | (uintptr_t)pmc;
        if ((bits & 15) == 0 && base + a.chunk <= s.count) {
            const int64_t chunk4 = a.chunk / 4;
            for (int64_t st = 0; st < chunk4; st += kMcUnroll * kAdamThreads) {
                float4 g[kMcUnroll];
#pragma unroll
                for (int u = 0; u < kMcUnroll; ++u) {
                    const int64_t o = st + u * kAdamThreads + tid;
                    if (o < chunk4) g[u] = multimem_ld_reduce_add_v4(gmc + o * 4);
                }
#pragma unroll
                for (int u = 0; u < kMcUnroll; ++u) {
                    const int64_t o = st + u * kAdamThreads + tid;
                    if (o < chunk4) {
                        float4 p = reinterpret_cast<const float4*>(s.param + base)[o];
                        float4 m = reinterpret_cast<const float4*>(s.exp_avg + base)[o];
                        float4 v = reinterpret_cast<const float4*>(s.exp_avg_sq + base)[o];
                        adam_update(g[u].x, p.x, m.x, v.x, c);
                        adam_update(g[u].y, p.y, m.y, v.y, c);
                        adam_update(g[u].z, p.z, m.z, v.z, c);
                        adam_update(g[u].w, p.w, m.w, v.w, c);
                        multimem_st_v4(pmc + o * 4, p);
                        reinterpret_cast<float4*>(s.exp_avg + base)[o] = m;
                        reinterpret_cast<float4*>(s.exp_avg_sq + base)[o] = v;
                    }
                }
            }
        } else {
            for (int64_t o = tid; o < min(a.chunk, s.count - base); o += kAdamThreads) {
                float p = s.param[base + o], m = s.exp_avg[base + o], v = s.exp_avg_sq[base + o];
                const float g = multimem_ld_reduce_add(gmc + o);
                adam_update(g, p, m, v, c);
                multimem_st(pmc + o, p);
                s.exp_avg[base + o] = m;
                s.exp_avg_sq[base + o] = v;
            }
        }
    }
    exchange_end(a.peers);
}

__device__ __forceinline__ void add4(float4& a, const float4 b) {
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
}

// What a CTA does with block `blk` of the launch: nothing to stage for a statistics block or a chunk that is not
// a full, 16-byte aligned span (those take scalar loads).
struct PeerChunk {
    int si;             // segment, or num_segments for a statistics block
    int64_t base;       // first element of the chunk inside the segment
    bool staged;        // the chunk's gradients of all ranks come through shared memory
};
__device__ __forceinline__ PeerChunk peer_chunk(const AdamArgs& a, int64_t blk) {
    PeerChunk ch;
    ch.si = 0;
#pragma unroll
    for (int k = 1; k <= kMaxSegments; ++k)
        if (k <= a.num_segments && blk >= a.block_start[k]) ch.si = k;
    ch.base = 0;
    ch.staged = false;
    if (ch.si < a.num_segments) {
        const D3gsAdamSegment& s = a.seg[ch.si];
        ch.base = (blk - a.block_start[ch.si]) * a.chunk;
        const int64_t goff = a.grad_off[ch.si] + ch.base, poff = a.param_off[ch.si] + ch.base;
        uintptr_t bits = (uintptr_t)(s.param + ch.base) | (uintptr_t)(s.exp_avg + ch.base) | (uintptr_t)(s.exp_avg_sq + ch.base);
        for (int q = 0; q < a.peers.world; ++q)
            bits |= (uintptr_t)(a.peers.grad[q] + goff) | (uintptr_t)(a.peers.param[q] + poff);
        ch.staged = (bits & 15) == 0 && ch.base + a.chunk <= s.count;
    }
    return ch;
}

// Every CTA walks the launch's blocks with a grid-sized stride (with flag ordering the grid is a few CTAs per SM,
// so that the announcements and the system-wide fence at the end are paid once per CTA; otherwise one CTA per
// block).  The gradients of the NEXT chunk travel into the second half of the staging buffer while the current
// chunk is summed, updated and stored: the links and the local memory work at the same time.
__global__ void __launch_bounds__(kAdamThreads, 3) adam_peers_kernel(const __grid_constant__ AdamArgs a) {
    extern __shared__ __align__(128) unsigned char s_raw[];
    __shared__ __align__(8) uint64_t s_bar[2];
    const int tid = threadIdx.x;
    const int world = a.peers.world;
    const int64_t chunk = a.chunk, chunk4 = chunk / 4;
    float4* const s_all = reinterpret_cast<float4*>(s_raw);
    auto buf_ptr = [&](int b) { return s_all + (int64_t)b * world * chunk4; };
    if (tid == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        fence_mbar_init();
    }
    const bool ready = exchange_begin(a.peers);      // (contains a barrier when flags are in use)
    if (a.peers.flags[0] == nullptr) __syncthreads();
    auto issue = [&](const PeerChunk& ch, int buf) {   // thread 0: start the copies of a staged chunk
        const uint32_t bytes = (uint32_t)(chunk * sizeof(float));
        const int64_t goff = a.grad_off[ch.si] + ch.base;
        mbar_arrive_expect_tx(&s_bar[buf], bytes * (uint32_t)world);
        if ((int)blockIdx.x == a.hooks.hold) return;      // test hook: this CTA's copies are never issued
        for (int q = 0; q < world; ++q) bulk_copy_g2s(buf_ptr(buf) + q * chunk4, a.peers.grad[q] + goff, bytes, &s_bar[buf]);
    };
    bool copy_failed = false;
    uint32_t phases = 0u;                             // bit b: parity of staging barrier b
    int cur = 0;
    if (ready && blockIdx.x < a.total_blocks) {
        const PeerChunk first = peer_chunk(a, blockIdx.x);
        if (first.staged && tid == 0) issue(first, 0);
    }
    for (int64_t blk = blockIdx.x; blk < a.total_blocks; blk += gridDim.x) {
        const PeerChunk ch = peer_chunk(a, blk);
        // the next block's copies go into the other buffer, whose last reader finished before the barrier below
        __syncthreads();
        bool next_in_flight = false;
        if (ready && !copy_failed && blk + gridDim.x < a.total_blocks) {
            const PeerChunk nx = peer_chunk(a, blk + gridDim.x);
            if (nx.staged) {
                if (tid == 0) issue(nx, cur ^ 1);
                next_in_flight = true;
            }
        }
        if (ch.si == a.num_segments) {   // statistics block
            const int64_t i = (blk - a.block_start[ch.si]) * kAdamThreads + tid;
            if (a.has_stats && i < a.stats.num) stats_update(a.stats, i);
        } else if (ready && !copy_failed) {
            const D3gsAdamSegment& s = a.seg[ch.si];
            const SegConst c = a.sc[ch.si];
            const int64_t base = ch.base;
            const int64_t poff = a.param_off[ch.si] + base;
            if (ch.staged) {
                bool arrived = mbar_wait_bounded(&s_bar[cur], (phases >> cur) & 1u, a.hooks.poll_limit);
                if (__syncthreads_or(!arrived)) {
                    // give the copies one more bounded wait before the shared memory can be released, flag, and
                    // leave this and the CTA's remaining chunks unchanged
                    if (!arrived) mbar_wait_bounded(&s_bar[cur], (phases >> cur) & 1u, a.hooks.poll_limit);
                    if (tid == 0 && a.peers.status != nullptr) atomicOr(a.peers.status, D3GS_STATUS_COPY_TIMEOUT);
                    copy_failed = true;
                } else {
                    phases ^= 1u << cur;
                    const float4* s_g = buf_ptr(cur);
                    for (int64_t st = 0; st < chunk4; st += kAdamUnroll * kAdamThreads) {
                        float4 p[kAdamUnroll], g[kAdamUnroll], m[kAdamUnroll], v[kAdamUnroll];
#pragma unroll
                        for (int u = 0; u < kAdamUnroll; ++u) {
                            const int64_t o = st + u * kAdamThreads + tid;
                            if (o < chunk4) {       // a chunk of many ranks is shorter than one step of this loop
                                p[u] = reinterpret_cast<const float4*>(s.param + base)[o];
                                m[u] = reinterpret_cast<const float4*>(s.exp_avg + base)[o];
                                v[u] = reinterpret_cast<const float4*>(s.exp_avg_sq + base)[o];
                                g[u] = s_g[o];
                                // the sum runs in rank order on every rank: all replicas of an element come from the same bits
                                for (int q = 1; q < world; ++q) add4(g[u], s_g[q * chunk4 + o]);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < kAdamUnroll; ++u) {
                            const int64_t o = st + u * kAdamThreads + tid;
                            if (o < chunk4) {
                                adam_update(g[u].x, p[u].x, m[u].x, v[u].x, c);
                                adam_update(g[u].y, p[u].y, m[u].y, v[u].y, c);
                                adam_update(g[u].z, p[u].z, m[u].z, v[u].z, c);
                                adam_update(g[u].w, p[u].w, m[u].w, v[u].w, c);
                                for (int q = 0; q < world; ++q) reinterpret_cast<float4*>(a.peers.param[q] + poff)[o] = p[u];
                                reinterpret_cast<float4*>(s.exp_avg + base)[o] = m[u];
                                reinterpret_cast<float4*>(s.exp_avg_sq + base)[o] = v[u];
                            }
                        }
                    }
                }
            } else {
                for (int64_t o = base + tid; o < min(base + chunk, s.count); o += kAdamThreads) {
                    float p = s.param[o], m = s.exp_avg[o], v = s.exp_avg_sq[o];
                    float g = __ldcg(a.peers.grad[0] + a.grad_off[ch.si] + o);
                    for (int q = 1; q < world; ++q) g += __ldcg(a.peers.grad[q] + a.grad_off[ch.si] + o);
                    adam_update(g, p, m, v, c);
                    for (int q = 0; q < world; ++q) a.peers.param[q][a.param_off[ch.si] + o] = p;
                    s.exp_avg[o] = m;
                    s.exp_avg_sq[o] = v;
                }
            }
        }
        if (next_in_flight) cur ^= 1;                  // the next block's gradients are on their way into the other buffer
        if (copy_failed && next_in_flight) {
            // the copies issued for the next block still land in shared memory: wait for them (bounded) before
            // the CTA may go on to its exit
            mbar_wait_bounded(&s_bar[cur], (phases >> cur) & 1u, a.hooks.poll_limit);
            next_in_flight = false;
        }
    }
    exchange_end(a.peers);      // a failure of this launch travels to every rank with the end-of-launch flags
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
        D3GS_REQUIRE((peers->grad_mc == nullptr) == (peers->param_mc == nullptr),
                     "grad_mc and param_mc must be given together");
        const bool with_flags = peers->flags[0] != nullptr;
        for (int q = 0; q < peers->world; ++q)
            D3GS_REQUIRE((peers->flags[q] != nullptr) == with_flags, "peer %d: flag blocks must be given for all ranks or none", q);
        D3GS_REQUIRE(!with_flags || peers->epoch != 0, "epoch must be positive when flag blocks are given");
        a.peers = *peers;
        for (int q = peers->world; q < D3GS_MAX_PEERS; ++q) a.peers.flags[q] = nullptr;
        if (peers->grad_mc != nullptr) {
            a.chunk = (int64_t)kMcUnroll * kAdamThreads * kAdamVec;    // one step of the multicast loop
        } else {
            // floats per CTA, rank and staging buffer (there are two): the largest power of two with
            // 2 * world * chunk * 4 bytes <= 64 KB
            a.chunk = kPeerSmemBytes / 4 / 4;
            while (2 * a.chunk * peers->world * 4 > kPeerSmemBytes) a.chunk /= 2;
        }
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
    a.total_blocks = blocks;
    a.hooks = test_hooks();
    if (blocks == 0) return D3GS_OK;
    D3GS_REQUIRE(blocks < ((int64_t)1 << 31), "too many CTAs");
    if (peers != nullptr) {
        // with flag ordering: a resident grid (CTAs per SM x SMs) that strides over the chunks
        int64_t grid = blocks;
        if (peers->flags[0] != nullptr) {
            int dev = 0, sms = 0;
            D3GS_CUDA(cudaGetDevice(&dev));
            D3GS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            const int per_sm = peers->grad_mc != nullptr ? kMcCtasPerSm : 3;
            grid = blocks < (int64_t)sms * per_sm ? blocks : (int64_t)sms * per_sm;
        }
        if (peers->grad_mc != nullptr) {
            adam_multimem_kernel<<<(unsigned)grid, kAdamThreads, 0, (cudaStream_t)stream>>>(a);
        } else {
            D3GS_CUDA(cudaFuncSetAttribute(adam_peers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeerSmemBytes));
            adam_peers_kernel<<<(unsigned)grid, kAdamThreads, kPeerSmemBytes, (cudaStream_t)stream>>>(a);
        }
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
