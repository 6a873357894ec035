// K6 raster forward and K7 raster backward: per-tile front-to-back alpha blending.
//
// Reference semantics: d3sim/algos/d3gs/render.py:1329-2316 (forward is_bwd=False; backward
// 1589-1676 + 1774-2210).  One CTA per 16x16 tile like the reference, but four warps of 8x8 pixels with TWO
// pixels per lane instead of eight warps of 8x4 pixels with one (render.py:1503-1512).
//
// What is different from the reference's kernel, and why:
//  * The tile's sorted list of 48-byte splat records is staged through shared memory in batches, double
//    buffered, either with one bulk async copy per batch (cp.async.bulk + mbarrier) when the records were
//    packed per (tile, splat) pair beforehand, or with per-thread 16-byte async gathers by sorted id from the
//    per-Gaussian record table the preprocess writes (render.py:1699-1716 gathers per thread, synchronously).
//  * Both kernels were instruction-issue bound when every warp walked every record.  The 32 lanes of a warp
//    first test 32 records at once (each record carries a conservative bounding box of its
//    alpha >= 1/255 region) against the eight 4x2 sub-blocks of the warp's 8x8 pixel block, ballot, and
//    append the survivors of every sub-block to a compact index list in shared memory.  Then every GROUP
//    of four lanes walks only the list of its own sub-block, front to back: one pass of the instruction
//    stream serves up to eight records.  The pass bodies are branch free (selects and predicates), which
//    is cheaper than votes and divergent branches when nearly every pass has a contributing pixel.
//  * A lane owns two horizontally adjacent pixels and uses the packed fp32 instructions of sm_100 (see below).
//  * Backward: the nine per-splat partial sums are reduced inside each group with a transposing butterfly
//    (8 shuffles for eight records instead of 45 for one).  Then either (a) they are accumulated per CTA in
//    shared memory and leave the CTA as three vector atomic adds per (tile, splat), or (b) the four lanes of
//    the group add them to global memory at once (four 8-byte and one 4-byte atomic per group and record).
//    (b) has no shared-memory atomics, no flush and one barrier less per batch and is faster while a splat is
//    seen by one or two groups of a tile (small splats: 0.89 -> 0.77 ms at 3 M Gaussians, 1080p); (a) wins when
//    splats cover many 4x2 sub-blocks.  The reference issues nine scalar atomics per warp (render.py:2061-2148).
//
// The arithmetic that decides n_contrib -- power, exp, alpha, the transmittance product and the
// three threshold compares -- is written with explicit round-to-nearest intrinsics so that its
// bits are defined (see common.cuh); skipping a record by its bounding box or by `power < thr`
// never changes a result because both imply alpha < alpha_eps.
#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kRecFloat4 = 3;                      // 48 bytes: [u v hx hy][ha nb hc o][r g b thr]
constexpr uint32_t kRecBytes = kRecFloat4 * 16;
constexpr int kGradFloats = D3GS_SPLAT_GRAD_FLOATS;   // 12: [dconic a b c, dopacity][dcolor r g b, 0][duv x y, 0 0]

struct RasterArgs {
    int width, height, tiles_x, tiles_y;
    float alpha_eps, t_eps;
    float bg[3];
    int training;
    const int32_t* ranges;
    const int32_t* tile_order;   // optional: CTA k handles tile tile_order[k] (longest lists first)
    const float4* records;
    const int32_t* sorted_ids;
    uint32_t* status;
    // forward outputs / backward inputs
    float* color;
    float* final_T;
    int32_t* n_contrib;
    // backward
    const float* drgb;
    const float* dT;
    float* splat_grads;
    unsigned long long* atomic_counts;   // instrumented backward only: [0] groups of global adds, [1] warp passes
    TestHooks hooks;
};

// The tile a CTA works on.  The grid is one-dimensional; with an order table the CTAs take the tiles by
// decreasing list length, so that the last CTAs to start are the cheapest and the grid ends without a tail.
struct TileId {
    int x, y, view, tile;
};
__device__ __forceinline__ TileId tile_of_cta(const RasterArgs& a) {
    TileId t;
    t.tile = a.tile_order != nullptr ? a.tile_order[blockIdx.x] : (int)blockIdx.x;
    const int per_view = a.tiles_x * a.tiles_y;
    t.view = t.tile / per_view;
    const int r = t.tile - t.view * per_view;
    t.y = r / a.tiles_x;
    t.x = r - t.y * a.tiles_x;
    return t;
}

__device__ __forceinline__ float shfl_x(float v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }

__device__ __forceinline__ void red_add_v4(float* addr, float x, float y, float z, float w) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ void red_add_v2(float* addr, float x, float y) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(x), "f"(y) : "memory");
}

// ---- two pixels per lane, packed fp32 arithmetic ---------------------------------------------------------
// sm_100 executes add/mul/fma on pairs of fp32 values held in a 64-bit register pair as ONE instruction
// (each half rounded to nearest like the scalar operation, so no result changes).  Both raster kernels are
// bound by instruction issue, so here a lane owns two horizontally adjacent pixels: everything that depends
// on the splat alone (record loads, list walk, dy-only terms) is done once for both, and the arithmetic on
// values that already come in pairs (the exp polynomial, transmittance, gradient moments) is packed.
// Operations that mix a per-splat scalar with a pair stay scalar: duplicating the scalar into a register
// pair costs what the packing saves, and staging duplicated records in shared memory cost more
// shared-memory bandwidth than it saved issue slots.  A warp covers an 8x8 pixel block, a CTA of four warps
// the 16x16 tile.  A group of FOUR lanes covers a 4x2 sub-block (the culling granularity) and walks its own
// survivor list, so one pass of the instruction stream serves up to eight records.
using f2 = float2;
__device__ __forceinline__ f2 f2_add(f2 a, f2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ f2 f2_mul(f2 a, f2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ f2 f2_fma(f2 a, f2 b, f2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ f2 f2_dup(float x) { return make_float2(x, x); }

// blend_exp on both halves: the same operations in the same order as the scalar version
__device__ __forceinline__ f2 blend_exp2(f2 power) {
    f2 t = f2_mul(power, f2_dup(1.44269504088896341f));
    t.x = fminf(fmaxf(t.x, -125.0f), 125.0f);
    t.y = fminf(fmaxf(t.y, -125.0f), 125.0f);
    const f2 m = f2_add(t, f2_dup(12582912.0f));
    const f2 n = f2_add(m, f2_dup(-12582912.0f));
    const f2 f = f2_fma(n, f2_dup(-1.0f), t);           // t - n
    f2 p = f2_dup(0.001327647129073739f);
    p = f2_fma(p, f, f2_dup(0.009675540961325169f));
    p = f2_fma(p, f, f2_dup(0.05550713092088699f));
    p = f2_fma(p, f, f2_dup(0.24022120237350464f));
    p = f2_fma(p, f, f2_dup(0.6931469440460205f));
    p = f2_fma(p, f, f2_dup(1.0f));
    p.x = __uint_as_float(__float_as_uint(p.x) + (__float_as_uint(m.x) << 23));
    p.y = __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(m.y) << 23));
    return p;
}

// Adds (x, y) to two adjacent floats in shared memory (8-byte aligned) with one 64-bit compare-and-swap loop:
// a float atomic add on shared memory is a compare-and-swap loop as well, so the pair costs one loop, not two.
__device__ __forceinline__ void smem_add_pair(float* addr, float x, float y) {
    unsigned long long* p = reinterpret_cast<unsigned long long*>(addr);
    unsigned long long seen = *p, assumed;
    do {
        assumed = seen;
        const f2 sum = f2_add(make_float2(__uint_as_float((uint32_t)assumed), __uint_as_float((uint32_t)(assumed >> 32))),
                              make_float2(x, y));
        const unsigned long long next =
            (unsigned long long)__float_as_uint(sum.x) | ((unsigned long long)__float_as_uint(sum.y) << 32);
        seen = atomicCAS(p, assumed, next);
    } while (seen != assumed);
}

constexpr int kBatch = 128;                // records per staged batch
constexpr int kListStride = kBatch + 8;    // bytes per group list (padded: the walk reads one entry ahead)

__device__ __forceinline__ void issue_batch(const RasterArgs& a, float4* buf, uint64_t* bar, int r0, int n, int batch) {
    const int cnt = min(kBatch, n - batch * kBatch);
    const uint32_t bytes = (uint32_t)cnt * kRecBytes;
    mbar_arrive_expect_tx(bar, bytes);
    if ((int)blockIdx.x != a.hooks.hold)      // test hook: this CTA's copies are never issued
        bulk_copy_g2s(buf, a.records + (int64_t)(r0 + batch * kBatch) * kRecFloat4, bytes, bar);
}

// Gather staging: thread t of the CTA fetches record `id` of the per-Gaussian table into slot t of a batch
// buffer with three 16-byte asynchronous copies (the thread waits for its own copies with cp.async.wait_all
// before the batch's barrier).  Used when the records are not packed per (tile, splat) pair beforehand.
__device__ __forceinline__ void gather_record(const RasterArgs& a, float4* buf, int slot, int32_t id) {
    if (id < 0) return;
    const float4* src = a.records + (int64_t)id * kRecFloat4;
    cp_async16(buf + slot * 3, src);
    cp_async16(buf + slot * 3 + 1, src + 1);
    cp_async16(buf + slot * 3 + 2, src + 2);
}
// id of the record that thread t stages for batch `batch` of a list of n records starting at r0 (-1: none)
__device__ __forceinline__ int32_t staged_id(const RasterArgs& a, int r0, int n, int batch, int t) {
    const int k = batch * kBatch + t;
    return k < n ? a.sorted_ids[r0 + k] : -1;
}

// The 32 lanes test the records [g*32, g*32+32) of the staged batch, one per lane, against the eight 4x2
// sub-blocks of the warp's 8x8 pixel block (columns at -+2 from the block centre, rows at -3, -1, +1, +3)
// and append every survivor of sub-block k to lists[k] (in list order).
// The record's (hx, hy) include the half size (3.5, 1.5) of an 8x4 block; a 4x2 sub-block is 2.0 / 1.0 smaller.
__device__ __forceinline__ void cull_to_lists(const float4* raw, int g, int limit, float wcx, float wcy,
                                              uint8_t* lists, int (&c)[8]) {
    const int lane = threadIdx.x & 31;
    const int j = g * 32 + lane;
    bool bx[2] = {false, false}, by[4] = {false, false, false, false};
    if (j < limit) {
        const float4 q0 = raw[j * 3];
        const float ddx = q0.x - wcx, ddy = q0.y - wcy, hxq = q0.z - 2.0f, hyq = q0.w - 1.0f;
        bx[0] = fabsf(ddx + 2.0f) <= hxq;
        bx[1] = fabsf(ddx - 2.0f) <= hxq;
        by[0] = fabsf(ddy + 3.0f) <= hyq;
        by[1] = fabsf(ddy + 1.0f) <= hyq;
        by[2] = fabsf(ddy - 1.0f) <= hyq;
        by[3] = fabsf(ddy - 3.0f) <= hyq;
    }
    const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const bool in = bx[k & 1] && by[k >> 1];
        const uint32_t m = __ballot_sync(0xffffffffu, in);
        if (in) lists[k * kListStride + c[k] + __popc(m & lt)] = (uint8_t)j;
        c[k] += __popc(m);
    }
}

// power = dx*(ha*dx + nb*dy) + (hc*dy)*dy for two pixels of one row (blend_power's operations and order)
__device__ __forceinline__ f2 blend_power2(const float4& q1, f2 dx, float dy) {
    const float t0 = f_fma(q1.y, dy, f_mul(q1.x, dx.x)), t1 = f_fma(q1.y, dy, f_mul(q1.x, dx.y));
    const float uu = f_mul(f_mul(q1.z, dy), dy);
    return make_float2(f_fma(t0, dx.x, uu), f_fma(t1, dx.y, uu));
}

__device__ __forceinline__ int pick8(const int (&c)[8], int k) {
    int v = c[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) v = k == i ? c[i] : v;
    return v;
}

// 8 CTAs per SM (64 registers): measured faster than 10 or 12 CTAs with 48 / 40 registers and than 6 with 72
template <bool GATHER>
__global__ void __launch_bounds__(128, 8) raster_forward_kernel(const __grid_constant__ RasterArgs a) {
    __shared__ __align__(128) float4 s_raw[2][kBatch * kRecFloat4];
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ uint8_t s_list[4][8 * kListStride];   // per warp: the eight groups' survivor lists
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, group = lane >> 2;
    const TileId tl = tile_of_cta(a);
    const int tile = tl.tile;
    const int r0 = a.ranges[tile * 2], r1 = a.ranges[tile * 2 + 1];
    const int n = r1 - r0;
    const int nb = (n + kBatch - 1) / kBatch;
    if (t == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        fence_mbar_init();
    }
    __syncthreads();
    int32_t id_next = -1;   // GATHER: the id this thread stages for the batch after the one in flight
    if (GATHER) {
        gather_record(a, s_raw[0], t, staged_id(a, r0, n, 0, t));
        id_next = staged_id(a, r0, n, 1, t);
    } else if (t == 0 && nb > 0) {
        issue_batch(a, s_raw[0], &s_bar[0], r0, n, 0);
    }

    // pixel A = (px, py), pixel B = (px + 1, py)
    const int bx0 = tl.x * 16 + (warp & 1) * 8, by0 = tl.y * 16 + (warp >> 1) * 8;
    const int px = bx0 + (group & 1) * 4 + (lane & 1) * 2;
    const int py = by0 + (group >> 1) * 2 + ((lane >> 1) & 1);
    const bool insideA = px < a.width && py < a.height, insideB = px + 1 < a.width && py < a.height;
    const float fpxA = (float)px, fpxB = (float)(px + 1), fpy = (float)py;
    const float wcx = (float)bx0 + 3.5f, wcy = (float)by0 + 3.5f;
    bool doneA = !insideA, doneB = !insideB;
    f2 T = f2_dup(1.0f), C0 = f2_dup(0.0f), C1 = f2_dup(0.0f), C2 = f2_dup(0.0f);
    int contribA = 0, contribB = 0;
    bool copy_failed = false;

    for (int b = 0; b < nb; ++b) {
        const int cur = b & 1;
        if (GATHER) cp_async_wait_all();
        else if (!mbar_wait_bounded(&s_bar[cur], (uint32_t)((b >> 1) & 1), a.hooks.poll_limit)) copy_failed = true;
        // The one barrier of a batch: batch b has arrived for everybody, everybody has finished batch b-1
        // (so the other buffer may be refilled), and the whole-tile early exit is decided
        // (render.py:1691-1694).  No copy is in flight here: the next is issued below.
        const int num_done = __syncthreads_count((doneA && doneB) || copy_failed);
        if (num_done == 128) break;
        if (GATHER) {
            if (b + 1 < nb) {
                gather_record(a, s_raw[cur ^ 1], t, id_next);
                id_next = staged_id(a, r0, n, b + 2, t);
            }
        } else if (t == 0 && b + 1 < nb) {
            issue_batch(a, s_raw[cur ^ 1], &s_bar[cur ^ 1], r0, n, b + 1);
        }
        const int cnt = min(kBatch, n - b * kBatch);
        const int ng = (cnt + 31) >> 5;
        const float4* rec = s_raw[cur];
        if (!__all_sync(0xffffffffu, doneA && doneB)) {
            int c[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int g = 0; g < ng; ++g) cull_to_lists(rec, g, cnt, wcx, wcy, s_list[warp], c);
            __syncwarp();
            const int mine = pick8(c, group);
            const uint8_t* lst = &s_list[warp][group * kListStride];
            const int base = b * kBatch;
            // The list index of a pass is loaded one pass ahead (the lists are padded, so reading one past the
            // end is in bounds).  Past the end of its list a group replays record 0 (always staged, finite);
            // `live` masks the result.
            int jn = 0 < mine ? (int)lst[0] : 0;
            for (int i = 0;; ++i) {
                const bool live = i < mine && !(doneA && doneB);
                if (!__any_sync(0xffffffffu, live)) break;
                const int j = jn;
                jn = i + 1 < mine ? (int)lst[i + 1] : 0;
                const float2 uv = *reinterpret_cast<const float2*>(rec + j * 3);   // u, v
                const float4 q1 = rec[j * 3 + 1];                                  // ha, nb, hc, opacity
                const float4 q2 = rec[j * 3 + 2];                                  // r, g, b, thr
                const f2 dx = make_float2(f_sub(uv.x, fpxA), f_sub(uv.x, fpxB));
                const float dy = f_sub(uv.y, fpy);
                const f2 power = blend_power2(q1, dx, dy);
                const f2 G = blend_exp2(power);
                const f2 alpha = make_float2(fminf(0.99f, f_mul(q1.w, G.x)), fminf(0.99f, f_mul(q1.w, G.y)));
                const f2 oma = f2_fma(alpha, f2_dup(-1.0f), f2_dup(1.0f));   // 1 - alpha
                const f2 nT = f2_mul(T, oma);
                f2 w = f2_mul(alpha, T);
                const float thr = q2.w;
                // power < thr  =>  alpha < alpha_eps: the pixel skips this splat (render.py:1796-1798)
                const bool okA = live && !doneA && power.x >= thr && alpha.x >= a.alpha_eps;
                const bool okB = live && !doneB && power.y >= thr && alpha.y >= a.alpha_eps;
                const bool sdA = nT.x < a.t_eps, sdB = nT.y < a.t_eps;
                // render.py:1803-1807: a splat with power > 0 or one that would end the pixel is not blended
                const bool updA = okA && !(power.x > 0.0f) && !sdA;
                const bool updB = okB && !(power.y > 0.0f) && !sdB;
                doneA = doneA || (okA && sdA);
                doneB = doneB || (okB && sdB);
                T.x = updA ? nT.x : T.x;
                T.y = updB ? nT.y : T.y;
                contribA = updA ? base + j : contribA;   // render.py:1836
                contribB = updB ? base + j : contribB;
                w.x = updA ? w.x : 0.0f;                 // a zero weight leaves the colour sums unchanged
                w.y = updB ? w.y : 0.0f;
                C0 = make_float2(f_fma(w.x, q2.x, C0.x), f_fma(w.y, q2.x, C0.y));
                C1 = make_float2(f_fma(w.x, q2.y, C1.x), f_fma(w.y, q2.y, C1.y));
                C2 = make_float2(f_fma(w.x, q2.z, C2.x), f_fma(w.y, q2.z, C2.y));
            }
        }
    }
    if (copy_failed && t == 0) atomicOr(a.status, D3GS_STATUS_COPY_TIMEOUT);
    const int64_t pix = ((int64_t)tl.view * a.height + py) * a.width + px;
    if (insideA) {
        float c0 = C0.x, c1 = C1.x, c2 = C2.x;
        a.final_T[pix] = T.x;
        a.n_contrib[pix] = contribA;
        if (!a.training) {   // render.py:2259-2263: composite the background and clamp at inference
            c0 = fminf(fmaxf(f_add(c0, f_mul(T.x, a.bg[0])), 0.0f), 1.0f);
            c1 = fminf(fmaxf(f_add(c1, f_mul(T.x, a.bg[1])), 0.0f), 1.0f);
            c2 = fminf(fmaxf(f_add(c2, f_mul(T.x, a.bg[2])), 0.0f), 1.0f);
        }
        a.color[pix * 3] = c0; a.color[pix * 3 + 1] = c1; a.color[pix * 3 + 2] = c2;
    }
    if (insideB) {
        float c0 = C0.y, c1 = C1.y, c2 = C2.y;
        a.final_T[pix + 1] = T.y;
        a.n_contrib[pix + 1] = contribB;
        if (!a.training) {
            c0 = fminf(fmaxf(f_add(c0, f_mul(T.y, a.bg[0])), 0.0f), 1.0f);
            c1 = fminf(fmaxf(f_add(c1, f_mul(T.y, a.bg[1])), 0.0f), 1.0f);
            c2 = fminf(fmaxf(f_add(c2, f_mul(T.y, a.bg[2])), 0.0f), 1.0f);
        }
        a.color[pix * 3 + 3] = c0; a.color[pix * 3 + 4] = c1; a.color[pix * 3 + 5] = c2;
    }
}

// Backward with two pixels per lane.  Per pass a lane adds its two pixels' nine moment values, then the
// four lanes of a group reduce them with a transposing butterfly (8 shuffles) and every lane adds the two
// components it ends up holding to the record's row in shared memory.
// 8 CTAs per SM (64 registers): measured faster than 9 / 10 CTAs (56 / 48 registers) and than 6 / 5 (72 / 77)
// COUNT (instrumentation, config_def.py:134 measure_atomic_add_count): a.atomic_counts[0] += groups of global adds
// issued (one per Gaussian a lane group / a tile flush adds to), [1] += warp passes with a valid pixel.
template <bool GATHER, bool DIRECT, bool COUNT>
__global__ void __launch_bounds__(128, 8) raster_backward_kernel(const __grid_constant__ RasterArgs a) {
    __shared__ __align__(128) float4 s_raw[2][kBatch * kRecFloat4];
    __shared__ __align__(8) uint64_t s_bar[2];
    // per record: sum m dx^2, m dx dy, m dy^2, m, dcolor r g b, m dx, m dy, (pad: rows stay 8-byte aligned)
    __shared__ __align__(8) float s_acc[DIRECT ? 1 : kBatch][10];
    __shared__ int32_t s_ids[2][DIRECT ? kBatch : 1];   // DIRECT: sorted id of every staged record
    __shared__ int s_max[4];
    __shared__ uint8_t s_list[4][8 * kListStride];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, group = lane >> 2;
    const TileId tl = tile_of_cta(a);
    const int tile = tl.tile;
    const int r0 = a.ranges[tile * 2], r1 = a.ranges[tile * 2 + 1];
    const int n = r1 - r0;
    const int bx0 = tl.x * 16 + (warp & 1) * 8, by0 = tl.y * 16 + (warp >> 1) * 8;
    const int px = bx0 + (group & 1) * 4 + (lane & 1) * 2;
    const int py = by0 + (group >> 1) * 2 + ((lane >> 1) & 1);
    const bool insideA = px < a.width && py < a.height, insideB = px + 1 < a.width && py < a.height;
    const int64_t pix = ((int64_t)tl.view * a.height + py) * a.width + px;
    // render.py:1594: list positions [0, n_contrib] took part in the forward blend
    int contribA = 0, contribB = 0;
    // nr = -(colour suffix): starts at -final colour and gains w*c per blended splat (render.py:1868-1895)
    f2 nr0 = f2_dup(0.0f), nr1 = nr0, nr2 = nr0, dr0 = nr0, dr1 = nr0, dr2 = nr0, ndTT = nr0;
    if (insideA && n > 0) {
        contribA = min(a.n_contrib[pix] + 1, n);
        nr0.x = -a.color[pix * 3]; nr1.x = -a.color[pix * 3 + 1]; nr2.x = -a.color[pix * 3 + 2];
        dr0.x = a.drgb[pix * 3]; dr1.x = a.drgb[pix * 3 + 1]; dr2.x = a.drgb[pix * 3 + 2];
        ndTT.x = a.dT != nullptr ? -(a.dT[pix] * a.final_T[pix]) : 0.0f;   // render.py:1935
    }
    if (insideB && n > 0) {
        contribB = min(a.n_contrib[pix + 1] + 1, n);
        nr0.y = -a.color[pix * 3 + 3]; nr1.y = -a.color[pix * 3 + 4]; nr2.y = -a.color[pix * 3 + 5];
        dr0.y = a.drgb[pix * 3 + 3]; dr1.y = a.drgb[pix * 3 + 4]; dr2.y = a.drgb[pix * 3 + 5];
        ndTT.y = a.dT != nullptr ? -(a.dT[pix + 1] * a.final_T[pix + 1]) : 0.0f;
    }
    int wmax = max(contribA, contribB);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
    if (lane == 0) s_max[warp] = wmax;
    if (t == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        fence_mbar_init();
    }
    __syncthreads();
    const int bmax = max(max(s_max[0], s_max[1]), max(s_max[2], s_max[3]));
    const int nb = (bmax + kBatch - 1) / kBatch;     // batches anybody in the tile still needs
    // GATHER: ids of the records this thread stages: of the current batch, the one in flight, the one after
    int32_t id_cur = -1, id_flight = -1, id_next = -1;
    if (GATHER) {
        id_cur = staged_id(a, r0, bmax, 0, t);
        gather_record(a, s_raw[0], t, id_cur);
        id_next = staged_id(a, r0, bmax, 1, t);
        if (DIRECT) s_ids[0][t] = id_cur;
    } else {
        if (t == 0 && nb > 0) issue_batch(a, s_raw[0], &s_bar[0], r0, bmax, 0);
        if (DIRECT) s_ids[0][t] = staged_id(a, r0, bmax, 0, t);
    }

    const float fpxA = (float)px, fpxB = (float)(px + 1), fpy = (float)py;
    const float wcx = (float)bx0 + 3.5f, wcy = (float)by0 + 3.5f;
    const bool h2 = (lane & 2) != 0, h1 = (lane & 1) != 0;
    // after the butterfly a lane holds the group's totals of components slot and slot + 1
    const int slot = (h2 ? 4 : 0) + (h1 ? 2 : 0);
    f2 T = f2_dup(1.0f);
    bool copy_failed = false;
    unsigned int n_groups = 0, n_passes = 0;    // COUNT only
    if (!DIRECT) {
#pragma unroll
        for (int k = 0; k < 9; ++k) s_acc[t][k] = 0.0f;   // row t is zeroed again by its owner after every flush
    }
    for (int b = 0; b < nb; ++b) {
        const int cur = b & 1;
        if (GATHER) cp_async_wait_all();
        else if (!mbar_wait_bounded(&s_bar[cur], (uint32_t)((b >> 1) & 1), a.hooks.poll_limit)) copy_failed = true;
        // First barrier of the batch: batch b has arrived for everybody and everybody has flushed and zeroed
        // its accumulator row of batch b-1, so the other record buffer may be refilled.  No copy is in flight.
        if (__syncthreads_or(copy_failed)) break;
        const int cnt = min(kBatch, bmax - b * kBatch);
        int32_t my_id = 0;
        if (GATHER) {
            if (b > 0) id_cur = id_flight;
            my_id = max(id_cur, 0);
            if (b + 1 < nb) {
                gather_record(a, s_raw[cur ^ 1], t, id_next);
                if (DIRECT) s_ids[cur ^ 1][t] = id_next;
                id_flight = id_next;
                id_next = staged_id(a, r0, bmax, b + 2, t);
            }
        } else {
            if (t == 0 && b + 1 < nb) issue_batch(a, s_raw[cur ^ 1], &s_bar[cur ^ 1], r0, bmax, b + 1);
            if (DIRECT) {
                if (b + 1 < nb) s_ids[cur ^ 1][t] = staged_id(a, r0, bmax, b + 1, t);
            } else if (t < cnt) {
                my_id = a.sorted_ids[r0 + b * kBatch + t];
            }
        }
        const float4* raw = s_raw[cur];
        const int wlim = min(cnt, wmax - b * kBatch);   // warp-uniform: nobody in the warp goes further
        const int ng = (wlim + 31) >> 5;
        if (ng > 0) {
            int c[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int g = 0; g < ng; ++g) cull_to_lists(raw, g, wlim, wcx, wcy, s_list[warp], c);
            __syncwarp();
            const int mine = pick8(c, group);
            const int maxc = max(max(max(c[0], c[1]), max(c[2], c[3])), max(max(c[4], c[5]), max(c[6], c[7])));
            const uint8_t* lst = &s_list[warp][group * kListStride];
            const int base = b * kBatch;
            // The list index of a pass is loaded one pass ahead (the lists are padded, so reading one past the
            // end is in bounds).  A group past the end of its list replays record 0 with zero weights: every
            // value below stays finite, so the branch-free selects cannot leak a NaN into T or the colour suffix.
            int jn = 0 < mine ? (int)lst[0] : 0;
            for (int i = 0; i < maxc; ++i) {
                const bool act = i < mine;
                const int j = jn;
                jn = i + 1 < mine ? (int)lst[i + 1] : 0;
                const float2 uv = *reinterpret_cast<const float2*>(raw + j * 3);   // u, v
                const float4 q1 = raw[j * 3 + 1];                                  // ha, nb, hc, opacity
                const float4 q2 = raw[j * 3 + 2];                                  // r, g, b, thr
                const f2 dx = make_float2(f_sub(uv.x, fpxA), f_sub(uv.x, fpxB));
                const float dy = f_sub(uv.y, fpy);
                const f2 power = blend_power2(q1, dx, dy);
                const f2 G = blend_exp2(power);
                const f2 alpha = make_float2(fminf(0.99f, f_mul(q1.w, G.x)), fminf(0.99f, f_mul(q1.w, G.y)));
                const float thr = q2.w;
                // render.py:1777: valid = power <= 0 && alpha >= alpha_eps && position < contributor
                const bool validA = act && (base + j < contribA) && power.x >= thr && power.x <= 0.0f &&
                                    alpha.x >= a.alpha_eps;
                const bool validB = act && (base + j < contribB) && power.y >= thr && power.y <= 0.0f &&
                                    alpha.y >= a.alpha_eps;
                const f2 oma = f2_fma(alpha, f2_dup(-1.0f), f2_dup(1.0f));
                f2 w = f2_mul(alpha, T);
                const f2 nT = f2_mul(T, oma);
                w.x = validA ? w.x : 0.0f;
                w.y = validB ? w.y : 0.0f;
                T.x = validA ? nT.x : T.x;
                T.y = validB ? nT.y : T.y;
                nr0 = make_float2(fmaf(w.x, q2.x, nr0.x), fmaf(w.y, q2.x, nr0.y));
                nr1 = make_float2(fmaf(w.x, q2.y, nr1.x), fmaf(w.y, q2.y, nr1.y));
                nr2 = make_float2(fmaf(w.x, q2.z, nr2.x), fmaf(w.y, q2.z, nr2.y));
                f2 dl = f2_mul(dr0, make_float2(fmaf(T.x, q2.x, nr0.x), fmaf(T.y, q2.x, nr0.y)));
                dl = f2_fma(dr1, make_float2(fmaf(T.x, q2.y, nr1.x), fmaf(T.y, q2.y, nr1.y)), dl);
                dl = f2_fma(dr2, make_float2(fmaf(T.x, q2.z, nr2.x), fmaf(T.y, q2.z, nr2.y)), dl);
                dl = f2_add(dl, ndTT);
                // m = dL/dalpha * G (render.py:1957, 2018).  The per-splat sums are kept as moments of m over
                // the pixels; the record's constants (opacity, conic) are applied once when the batch is
                // flushed: dL/dG * G = opacity * m (render.py:1995).
                f2 m;
                m.x = validA ? __fdividef(dl.x, oma.x) : 0.0f;
                m.y = validB ? __fdividef(dl.y, oma.y) : 0.0f;
                m = f2_mul(m, G);
                const f2 dy2 = f2_dup(dy);
                const f2 mx = f2_mul(m, dx), my = f2_mul(m, dy2);
                const f2 pxx = f2_mul(mx, dx), pxy = f2_mul(mx, dy2), pyy = f2_mul(my, dy2);
                const f2 pc0 = f2_mul(w, dr0), pc1 = f2_mul(w, dr1), pc2 = f2_mul(w, dr2);
                const uint32_t vmask = __ballot_sync(0xffffffffu, validA || validB);
                if (vmask == 0) continue;
                const float v0 = pxx.x + pxx.y, v1 = pxy.x + pxy.y, v2 = pyy.x + pyy.y, v3 = m.x + m.y;
                const float v4 = pc0.x + pc0.y, v5 = pc1.x + pc1.y, v6 = pc2.x + pc2.y, v7 = mx.x + mx.y;
                float v8 = my.x + my.y;
                // transposing butterfly inside each group of four lanes: 8 components in 6 shuffles, the ninth in 2
                const f2 a01 = f2_add(make_float2(h2 ? v4 : v0, h2 ? v5 : v1),
                                      make_float2(shfl_x(h2 ? v0 : v4, 2), shfl_x(h2 ? v1 : v5, 2)));
                const f2 a23 = f2_add(make_float2(h2 ? v6 : v2, h2 ? v7 : v3),
                                      make_float2(shfl_x(h2 ? v2 : v6, 2), shfl_x(h2 ? v3 : v7, 2)));
                const f2 b01 = f2_add(make_float2(h1 ? a23.x : a01.x, h1 ? a23.y : a01.y),
                                      make_float2(shfl_x(h1 ? a01.x : a23.x, 1), shfl_x(h1 ? a01.y : a23.y, 1)));
                v8 += shfl_x(v8, 2);
                v8 += shfl_x(v8, 1);
                const bool gvalid = ((vmask >> (group * 4)) & 0xfu) != 0;
                if (COUNT) {
                    n_passes += lane == 0;
                    if (DIRECT) n_groups += gvalid && (lane & 3) == 0;
                }
                if (DIRECT) {
                    // No accumulation in shared memory: a record is touched by one or two groups of the tile on
                    // average, so the group's totals leave as they are.  The four lanes hold (sxx, sxy),
                    // (syy, s0), (dcolor r, g), (dcolor b, sx); sy is on every lane.  The record's conic and
                    // opacity are applied here (see the flush of the other variant for the formulas).
                    if (gvalid) {
                        float* dst = a.splat_grads + (int64_t)s_ids[cur][j] * kGradFloats;
                        const float o = q1.w;
                        const float sx = b01.y, sy = v8;
                        const float gu = o * fmaf(2.0f * q1.x, sx, q1.y * sy), gv = o * fmaf(2.0f * q1.z, sy, q1.y * sx);
                        const float x = h2 ? (h1 ? gu : b01.x) : -0.5f * o * b01.x;
                        const float y = h2 ? (h1 ? gv : b01.y) : (h1 ? b01.y : -o * b01.y);
                        red_add_v2(dst + (h2 ? (h1 ? 8 : 4) : (h1 ? 2 : 0)), x, y);
                        if (h2 && h1) atomicAdd(dst + 6, b01.x);
                    }
                } else if (gvalid) {
                    smem_add_pair(&s_acc[j][slot], b01.x, b01.y);
                    if ((lane & 3) == 0) atomicAdd(&s_acc[j][8], v8);
                }
            }
        }
        if (DIRECT) continue;
        __syncthreads();
        if (t < cnt) {
            const float* acc = s_acc[t];
            const float sxx = acc[0], sxy = acc[1], syy = acc[2], s0 = acc[3], g4 = acc[4], g5 = acc[5], g6 = acc[6],
                        sx = acc[7], sy = acc[8];
            const bool any = (sxx != 0.f) | (sxy != 0.f) | (syy != 0.f) | (s0 != 0.f) | (g4 != 0.f) | (g5 != 0.f) |
                             (g6 != 0.f) | (sx != 0.f) | (sy != 0.f);
            // conic = (-2 ha, -nb, -2 hc), render.py:2001-2017: d/dconic = -0.5 o sxx, -o sxy, -0.5 o syy;
            // d/duv = o (2 ha sx + nb sy, 2 hc sy + nb sx); d/dopacity = s0
            const float4 k1 = raw[t * 3 + 1];   // ha, nb, hc, opacity
            const float g0 = -0.5f * k1.w * sxx, g1 = -k1.w * sxy, g2 = -0.5f * k1.w * syy, g3 = s0;
            const float g7 = k1.w * fmaf(2.0f * k1.x, sx, k1.y * sy);
            const float g8 = k1.w * fmaf(2.0f * k1.z, sy, k1.y * sx);
            if (any) {
                if (COUNT) ++n_groups;
                float* dst = a.splat_grads + (int64_t)my_id * kGradFloats;
                red_add_v4(dst, g0, g1, g2, g3);
                red_add_v4(dst + 4, g4, g5, g6, 0.0f);
                red_add_v2(dst + 8, g7, g8);
#pragma unroll
                for (int k = 0; k < 9; ++k) s_acc[t][k] = 0.0f;
            }
        }
    }
    if (copy_failed && t == 0) atomicOr(a.status, D3GS_STATUS_COPY_TIMEOUT);
    if (COUNT) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            n_groups += __shfl_xor_sync(0xffffffffu, n_groups, o);
            n_passes += __shfl_xor_sync(0xffffffffu, n_passes, o);
        }
        if (lane == 0) {
            atomicAdd(a.atomic_counts, (unsigned long long)n_groups);
            atomicAdd(a.atomic_counts + 1, (unsigned long long)n_passes);
        }
    }
}

int32_t fill_args(const D3gsOpConfig* cfg, RasterArgs& a) {
    D3GS_REQUIRE(cfg != nullptr, "cfg is NULL");
    D3GS_REQUIRE(cfg->tile_x == 16 && cfg->tile_y == 16, "only 16x16 tiles are supported");
    D3GS_REQUIRE(cfg->width > 0 && cfg->height > 0, "bad image size");
    D3GS_REQUIRE(cfg->num_views >= 1 && cfg->num_views <= 65535, "num_views out of range");
    a.width = cfg->width;
    a.height = cfg->height;
    a.tiles_x = (cfg->width + 15) / 16;
    a.tiles_y = (cfg->height + 15) / 16;
    a.alpha_eps = cfg->alpha_eps;
    a.t_eps = cfg->transmittance_eps;
    a.bg[0] = cfg->bg_color[0]; a.bg[1] = cfg->bg_color[1]; a.bg[2] = cfg->bg_color[2];
    a.training = cfg->training;
    a.hooks = test_hooks();
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" int32_t d3gs_raster_forward(const D3gsOpConfig* cfg, const int32_t* ranges, const int32_t* tile_order,
                                       const float* records, const int32_t* sorted_values, float* color,
                                       float* final_T, int32_t* n_contrib, uint32_t* status, void* stream) {
    RasterArgs a = {};
    int32_t rc = fill_args(cfg, a);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(ranges && color && final_T && n_contrib && status, "NULL argument");
    D3GS_REQUIRE(((uintptr_t)records & 15) == 0, "records must be 16-byte aligned");
    a.ranges = ranges;
    a.tile_order = tile_order;
    a.records = reinterpret_cast<const float4*>(records);
    a.status = status;
    a.color = color;
    a.final_T = final_T;
    a.n_contrib = n_contrib;
    const unsigned grid = (unsigned)(a.tiles_x * a.tiles_y * cfg->num_views);
    if (sorted_values != nullptr) {   // records are the per-Gaussian table: gather by sorted id
        a.sorted_ids = sorted_values;
        raster_forward_kernel<true><<<grid, 128, 0, (cudaStream_t)stream>>>(a);
    } else {                          // records are packed per (tile, splat) pair, in list order
        raster_forward_kernel<false><<<grid, 128, 0, (cudaStream_t)stream>>>(a);
    }
    D3GS_LAUNCH_CHECK("raster_forward_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_raster_backward(const D3gsOpConfig* cfg, int64_t num, const int32_t* ranges,
                                        const int32_t* tile_order, const float* records, int32_t mode,
                                        const int32_t* sorted_values, const float* color,
                                        const float* final_T, const int32_t* n_contrib, const float* drgb,
                                        const float* dT, float* splat_grads, uint64_t* atomic_counts,
                                        uint32_t* status, void* stream) {
    RasterArgs a = {};
    int32_t rc = fill_args(cfg, a);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(ranges && sorted_values && color && final_T && n_contrib && drgb && status, "NULL argument");
    D3GS_REQUIRE(splat_grads != nullptr, "NULL gradient output");
    D3GS_REQUIRE(((uintptr_t)records & 15) == 0, "records must be 16-byte aligned");
    D3GS_REQUIRE(((uintptr_t)splat_grads & 15) == 0, "splat_grads must be 16-byte aligned");
    D3GS_REQUIRE(num >= 0, "negative Gaussian count");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t bn = (size_t)num * cfg->num_views;
    D3GS_CUDA(cudaMemsetAsync(splat_grads, 0, bn * kGradFloats * sizeof(float), s));
    a.ranges = ranges;
    a.tile_order = tile_order;
    a.records = reinterpret_cast<const float4*>(records);
    a.sorted_ids = sorted_values;
    a.status = status;
    a.color = const_cast<float*>(color);
    a.final_T = const_cast<float*>(final_T);
    a.n_contrib = const_cast<int32_t*>(n_contrib);
    a.drgb = drgb;
    a.dT = dT;
    a.splat_grads = splat_grads;
    const unsigned grid = (unsigned)(a.tiles_x * a.tiles_y * cfg->num_views);
    a.atomic_counts = reinterpret_cast<unsigned long long*>(atomic_counts);
    const bool records_by_id = (mode & D3GS_RASTER_RECORDS_BY_ID) != 0;
    const bool direct = (mode & D3GS_RASTER_DIRECT_ATOMICS) != 0;
    if (atomic_counts != nullptr) {     // the instrumented instances: same arithmetic, plus the two counters
        if (direct) {
            if (records_by_id) raster_backward_kernel<true, true, true><<<grid, 128, 0, s>>>(a);
            else raster_backward_kernel<false, true, true><<<grid, 128, 0, s>>>(a);
        } else {
            if (records_by_id) raster_backward_kernel<true, false, true><<<grid, 128, 0, s>>>(a);
            else raster_backward_kernel<false, false, true><<<grid, 128, 0, s>>>(a);
        }
    } else if (direct) {
        if (records_by_id) raster_backward_kernel<true, true, false><<<grid, 128, 0, s>>>(a);
        else raster_backward_kernel<false, true, false><<<grid, 128, 0, s>>>(a);
    } else {
        if (records_by_id) raster_backward_kernel<true, false, false><<<grid, 128, 0, s>>>(a);
        else raster_backward_kernel<false, false, false><<<grid, 128, 0, s>>>(a);
    }
    D3GS_LAUNCH_CHECK("raster_backward_kernel");
    return D3GS_OK;
}
