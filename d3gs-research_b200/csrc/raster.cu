// K6 raster forward and K7 raster backward: per-tile front-to-back alpha blending.
//
// Reference semantics: d3sim/algos/d3gs/render.py:1329-2316 (forward is_bwd=False; backward
// 1589-1676 + 1774-2210).  One CTA of 256 threads per 16x16 tile, one pixel per thread, pixels laid
// out 8x4 per warp (render.py:1503-1512).
//
// What is different from the reference's kernel, and why:
//  * The tile's sorted list of 48-byte splat records is streamed through shared memory with bulk
//    async copies (cp.async.bulk + mbarrier, double buffered) instead of per-thread gathers
//    (render.py:1699-1716).
//  * Both kernels were instruction-issue bound when every warp walked every record.  Now the 32
//    lanes of a warp first test 32 records at once (each record carries a conservative bounding
//    box of its alpha >= 1/255 region) against the four 4x2 sub-blocks of the warp's 8x4 pixel
//    block, ballot, and append the survivors of every sub-block to a compact index list in shared
//    memory.  Then every QUARTER of the warp walks only the list of its own sub-block, front to
//    back: one pass of the instruction stream serves up to four records.  The forward pass body is
//    branch free (selects and predicates), which is cheaper than votes and divergent branches
//    when nearly every pass has a contributing pixel.
//  * Backward: the nine per-splat partial derivatives are reduced inside each quarter with a
//    transposing butterfly (10 shuffles for four records instead of 45 for one), accumulated per
//    CTA in shared memory, and leave the CTA as three vector atomic adds per (tile, splat) instead
//    of the reference's nine scalar atomics per warp (render.py:2061-2148).
//
// The arithmetic that decides n_contrib -- power, exp, alpha, the transmittance product and the
// three threshold compares -- is written with explicit round-to-nearest intrinsics so that its
// bits are defined (see common.cuh); skipping a record by its bounding box or by `power < thr`
// never changes a result because both imply alpha < alpha_eps.
#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kBatch = 256;                        // records per staged batch
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
};

struct PixelCoord {
    int px, py;
    bool inside;
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

// Pixel of a thread.  A warp covers an 8x4 pixel block of the tile (render.py:1503-1512 uses the same
// block per warp); inside it every QUARTER of the warp (8 lanes) covers a 4x2 sub-block:
//   quarter q = lane>>3: x half (q&1)*4, y half (q>>1)*2; inside the quarter lane&3 -> x, (lane>>2)&1 -> y.
// Results do not depend on which thread owns which pixel.
__device__ __forceinline__ PixelCoord pixel_of_thread(const RasterArgs& a, const TileId& tl) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = lane >> 3;
    PixelCoord p;
    p.px = tl.x * 16 + (warp & 1) * 8 + (q & 1) * 4 + (lane & 3);
    p.py = tl.y * 16 + (warp >> 1) * 4 + (q >> 1) * 2 + ((lane >> 2) & 1);
    p.inside = p.px < a.width && p.py < a.height;
    return p;
}

// Producer side of the staging pipeline (thread 0 only).
__device__ __forceinline__ void issue_batch(const RasterArgs& a, float4* buf, uint64_t* bar, int r0, int n, int batch) {
    const int cnt = min(kBatch, n - batch * kBatch);
    const uint32_t bytes = (uint32_t)cnt * kRecBytes;
    mbar_arrive_expect_tx(bar, bytes);
    bulk_copy_g2s(buf, a.records + (int64_t)(r0 + batch * kBatch) * kRecFloat4, bytes, bar);
}

constexpr int kListStride = kBatch + 8;   // bytes per quarter list; +8 keeps the four lists on different banks

// The 32 lanes test the records [g*32, g*32+32) of the staged batch, one record per lane, against the
// four 4x2 sub-blocks of this warp's pixel block and append the index of every record that touches
// sub-block q to lists[q] (in list order); c[q] is the running length, the same in all lanes.
// The record's (hx, hy) already include the half size of the 8x4 block (3.5, 1.5); a sub-block is
// 2.0 / 1.0 smaller and its centre sits at (+-2, +-1) from the block centre (wcx, wcy).
__device__ __forceinline__ void cull_to_lists(const float4* rec, int g, int limit, float wcx, float wcy,
                                              uint8_t* lists, int& c0, int& c1, int& c2, int& c3) {
    const int lane = threadIdx.x & 31;
    const int j = g * 32 + lane;
    bool left = false, right = false, top = false, bottom = false;
    if (j < limit) {
        const float4 q0 = rec[j * 3];
        const float ddx = q0.x - wcx, ddy = q0.y - wcy, hxq = q0.z - 2.0f, hyq = q0.w - 1.0f;
        left = fabsf(ddx + 2.0f) <= hxq;
        right = fabsf(ddx - 2.0f) <= hxq;
        top = fabsf(ddy + 1.0f) <= hyq;
        bottom = fabsf(ddy - 1.0f) <= hyq;
    }
    const uint32_t lt = (1u << lane) - 1u;
    const uint32_t m0 = __ballot_sync(0xffffffffu, left && top);
    const uint32_t m1 = __ballot_sync(0xffffffffu, right && top);
    const uint32_t m2 = __ballot_sync(0xffffffffu, left && bottom);
    const uint32_t m3 = __ballot_sync(0xffffffffu, right && bottom);
    if (left && top) lists[c0 + __popc(m0 & lt)] = (uint8_t)j;
    if (right && top) lists[kListStride + c1 + __popc(m1 & lt)] = (uint8_t)j;
    if (left && bottom) lists[2 * kListStride + c2 + __popc(m2 & lt)] = (uint8_t)j;
    if (right && bottom) lists[3 * kListStride + c3 + __popc(m3 & lt)] = (uint8_t)j;
    c0 += __popc(m0);
    c1 += __popc(m1);
    c2 += __popc(m2);
    c3 += __popc(m3);
}

__global__ void __launch_bounds__(256) raster_forward_kernel(const __grid_constant__ RasterArgs a) {
    __shared__ __align__(128) float4 s_rec[2][kBatch * kRecFloat4];
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ uint8_t s_list[8][4 * kListStride];   // per warp: the four quarters' survivor lists
    const int t = threadIdx.x;
    const TileId tl = tile_of_cta(a);
    const PixelCoord pc = pixel_of_thread(a, tl);
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
    if (t == 0 && nb > 0) issue_batch(a, s_rec[0], &s_bar[0], r0, n, 0);

    const float fpx = (float)pc.px, fpy = (float)pc.py;
    const float wcx = (float)(tl.x * 16 + ((t >> 5) & 1) * 8) + 3.5f;
    const float wcy = (float)(tl.y * 16 + (t >> 6) * 4) + 1.5f;
    const int quarter = (t & 31) >> 3, warp = t >> 5;
    bool done = !pc.inside;
    float T = 1.0f, C0 = 0.0f, C1 = 0.0f, C2 = 0.0f;
    int contributor = 0;
    bool copy_failed = false;

    for (int b = 0; b < nb; ++b) {
        const int cur = b & 1;
        if (!mbar_wait_bounded(&s_bar[cur], (uint32_t)((b >> 1) & 1))) copy_failed = true;
        // The one barrier of a batch: batch b has arrived for everybody, everybody has finished batch b-1
        // (so the other buffer may be refilled), and the whole-tile early exit is decided (render.py:1691-1694).
        // No copy is in flight here: the next one is issued below.
        const int num_done = __syncthreads_count(done || copy_failed);
        if (num_done == 256) break;
        if (t == 0 && b + 1 < nb) issue_batch(a, s_rec[cur ^ 1], &s_bar[cur ^ 1], r0, n, b + 1);
        const int cnt = min(kBatch, n - b * kBatch);
        const float4* rec = s_rec[cur];
        // Cull the whole batch first, then every quarter (8 lanes, a 4x2 pixel sub-block) walks its own
        // survivor list front to back, independently of the other quarters: one pass of the instruction
        // stream serves up to four different records.
        const int ng = (cnt + 31) >> 5;
        if (!__all_sync(0xffffffffu, done)) {
            int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
            for (int g = 0; g < ng; ++g) cull_to_lists(rec, g, cnt, wcx, wcy, s_list[warp], c0, c1, c2, c3);
            __syncwarp();
            const int mine = quarter == 0 ? c0 : (quarter == 1 ? c1 : (quarter == 2 ? c2 : c3));
            const uint8_t* lst = &s_list[warp][quarter * kListStride];
            const int base = b * kBatch;
            for (int i = 0;; ++i) {
                const bool live = i < mine && !done;
                if (!__any_sync(0xffffffffu, live)) break;
                // past the end of its list a quarter reads a stale index (< kBatch); `live` masks the result
                const int j = lst[i];
                const float4 q0 = rec[j * 3];       // u, v, hx, hy
                const float4 q1 = rec[j * 3 + 1];   // ha, nb, hc, opacity
                const float4 q2 = rec[j * 3 + 2];   // r, g, b, thr
                const float dx = f_sub(q0.x, fpx), dy = f_sub(q0.y, fpy);
                const float power = blend_power(q1.x, q1.y, q1.z, dx, dy);
                const float G = blend_exp(power);
                const float alpha = fminf(0.99f, f_mul(q1.w, G));
                const float nT = f_mul(T, f_sub(1.0f, alpha));
                // power < thr  =>  alpha < alpha_eps: the pixel skips this splat (render.py:1796-1798)
                const bool ok = live && power >= q2.w && alpha >= a.alpha_eps;
                const bool should_done = nT < a.t_eps;
                // render.py:1803-1807: a splat with power > 0 or one that would end the pixel is not blended
                const bool upd = ok && !(power > 0.0f) && !should_done;
                done = done || (ok && should_done);
                const float w = f_mul(alpha, T);
                T = upd ? nT : T;
                contributor = upd ? base + j : contributor;   // render.py:1836
                C0 = upd ? f_fma(w, q2.x, C0) : C0;
                C1 = upd ? f_fma(w, q2.y, C1) : C1;
                C2 = upd ? f_fma(w, q2.z, C2) : C2;
            }
        }
    }
    if (copy_failed && t == 0) atomicOr(a.status, D3GS_STATUS_COPY_TIMEOUT);
    if (pc.inside) {
        const int64_t pix = ((int64_t)tl.view * a.height + pc.py) * a.width + pc.px;
        a.final_T[pix] = T;
        a.n_contrib[pix] = contributor;
        if (!a.training) {   // render.py:2259-2263: composite the background and clamp at inference
            C0 = fminf(fmaxf(f_add(C0, f_mul(T, a.bg[0])), 0.0f), 1.0f);
            C1 = fminf(fmaxf(f_add(C1, f_mul(T, a.bg[1])), 0.0f), 1.0f);
            C2 = fminf(fmaxf(f_add(C2, f_mul(T, a.bg[2])), 0.0f), 1.0f);
        }
        a.color[pix * 3] = C0;
        a.color[pix * 3 + 1] = C1;
        a.color[pix * 3 + 2] = C2;
    }
}

__device__ __forceinline__ float shfl_x(float v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }

__device__ __forceinline__ void red_add_v4(float* addr, float x, float y, float z, float w) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ void red_add_v2(float* addr, float x, float y) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(x), "f"(y) : "memory");
}

// Backward.  Per pixel the blend is replayed front to back (T from 1, colour suffix = final -
// prefix, render.py:1868-1895).
__global__ void __launch_bounds__(256) raster_backward_kernel(const __grid_constant__ RasterArgs a) {
    __shared__ __align__(128) float4 s_rec[2][kBatch * kRecFloat4];
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ float s_acc[kBatch][9];   // per record: dconic a b c, dopacity, dcolor r g b, duv x y
    __shared__ int s_max[8];
    __shared__ uint8_t s_list[8][4 * kListStride];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const TileId tl = tile_of_cta(a);
    const PixelCoord pc = pixel_of_thread(a, tl);
    const int tile = tl.tile;
    const int r0 = a.ranges[tile * 2], r1 = a.ranges[tile * 2 + 1];
    const int n = r1 - r0;
    const int64_t pix = ((int64_t)tl.view * a.height + pc.py) * a.width + pc.px;
    // render.py:1594: list positions [0, n_contrib] took part in the forward blend
    int contributor = 0;
    float rr0 = 0.0f, rr1 = 0.0f, rr2 = 0.0f, dr0 = 0.0f, dr1 = 0.0f, dr2 = 0.0f, dTT = 0.0f;
    if (pc.inside && n > 0) {
        contributor = min(a.n_contrib[pix] + 1, n);
        rr0 = a.color[pix * 3]; rr1 = a.color[pix * 3 + 1]; rr2 = a.color[pix * 3 + 2];
        dr0 = a.drgb[pix * 3]; dr1 = a.drgb[pix * 3 + 1]; dr2 = a.drgb[pix * 3 + 2];
        dTT = a.dT != nullptr ? a.dT[pix] * a.final_T[pix] : 0.0f;   // render.py:1935
    }
    int wmax = contributor;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
    if (lane == 0) s_max[warp] = wmax;
    if (t == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        fence_mbar_init();
    }
    __syncthreads();
    int bmax = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) bmax = max(bmax, s_max[w]);
    const int nb = (bmax + kBatch - 1) / kBatch;     // batches anybody in the tile still needs
    if (t == 0 && nb > 0) issue_batch(a, s_rec[0], &s_bar[0], r0, bmax, 0);

    const float fpx = (float)pc.px, fpy = (float)pc.py;
    const float wcx = (float)(tl.x * 16 + (warp & 1) * 8) + 3.5f;
    const float wcy = (float)(tl.y * 16 + (warp >> 1) * 4) + 1.5f;
    const int quarter = lane >> 3;
    const bool h4 = (lane & 4) != 0, h2 = (lane & 2) != 0, h1 = (lane & 1) != 0;
    // after the butterfly, lane k of a quarter holds the quarter's total of component `slot`
    const int slot = (h4 ? 4 : 0) + (h2 ? 2 : 0) + (h1 ? 1 : 0);
    float T = 1.0f;
    bool copy_failed = false;
#pragma unroll
    for (int k = 0; k < 9; ++k) s_acc[t][k] = 0.0f;   // row t is zeroed again by its owner after every flush
    for (int b = 0; b < nb; ++b) {
        const int cur = b & 1;
        if (!mbar_wait_bounded(&s_bar[cur], (uint32_t)((b >> 1) & 1))) copy_failed = true;
        // First barrier of the batch: batch b has arrived for everybody and everybody has flushed and zeroed
        // its accumulator row of batch b-1, so the other record buffer may be refilled.  No copy is in flight.
        if (__syncthreads_or(copy_failed)) break;
        if (t == 0 && b + 1 < nb) issue_batch(a, s_rec[cur ^ 1], &s_bar[cur ^ 1], r0, bmax, b + 1);
        const int cnt = min(kBatch, bmax - b * kBatch);
        int32_t my_id = 0;
        if (t < cnt) my_id = a.sorted_ids[r0 + b * kBatch + t];
        const float4* rec = s_rec[cur];
        const int wlim = min(cnt, wmax - b * kBatch);   // warp-uniform: nobody in the warp goes further
        const int ng = (wlim + 31) >> 5;
        if (ng > 0) {
            int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
            for (int g = 0; g < ng; ++g) cull_to_lists(rec, g, wlim, wcx, wcy, s_list[warp], c0, c1, c2, c3);
            __syncwarp();
            const int mine = quarter == 0 ? c0 : (quarter == 1 ? c1 : (quarter == 2 ? c2 : c3));
            const int maxc = max(max(c0, c1), max(c2, c3));
            const uint8_t* lst = &s_list[warp][quarter * kListStride];
            const int base = b * kBatch;
            // every quarter (8 lanes, 4x2 pixels) walks its own survivors; one pass serves up to four records
            for (int i = 0; i < maxc; ++i) {
                const bool act = i < mine;
                // a quarter past the end of its list replays record 0 with zero weights: every value below
                // stays finite, so the branch-free selects cannot leak a NaN into T or the colour suffix
                const int j = act ? (int)lst[i] : 0;
                const float4 q0 = rec[j * 3];
                const float4 q1 = rec[j * 3 + 1];
                const float4 q2 = rec[j * 3 + 2];
                const float dx = f_sub(q0.x, fpx), dy = f_sub(q0.y, fpy);
                const float power = blend_power(q1.x, q1.y, q1.z, dx, dy);
                const float G = blend_exp(power);
                const float alpha = fminf(0.99f, f_mul(q1.w, G));
                // render.py:1777: valid = power <= 0 && alpha >= alpha_eps && position < contributor
                const bool valid = act && (base + j < contributor) && power >= q2.w && power <= 0.0f &&
                                   alpha >= a.alpha_eps;
                const float oma = f_sub(1.0f, alpha);
                const float w = valid ? f_mul(alpha, T) : 0.0f;
                T = valid ? f_mul(T, oma) : T;
                rr0 = fmaf(-w, q2.x, rr0); rr1 = fmaf(-w, q2.y, rr1); rr2 = fmaf(-w, q2.z, rr2);
                float dl = dr0 * fmaf(T, q2.x, -rr0);
                dl = fmaf(dr1, fmaf(T, q2.y, -rr1), dl);
                dl = fmaf(dr2, fmaf(T, q2.z, -rr2), dl);
                dl -= dTT;
                // m = dL/dalpha * G (render.py:1957, 2018).  The per-splat sums are kept as moments of m over
                // the pixels; the record's constants (opacity, conic) are applied once when the batch is
                // flushed: dL/dG * G = opacity * m (render.py:1995).
                const float m = valid ? __fdividef(dl, oma) * G : 0.0f;
                const float mx = m * dx, my = m * dy;
                float v0 = mx * dx, v1 = mx * dy, v2 = my * dy, v3 = m;      // sum m dx^2, m dx dy, m dy^2, m
                float v4 = w * dr0, v5 = w * dr1, v6 = w * dr2;              // dcolor, render.py:1962
                float v7 = mx, v8 = my;                                      // sum m dx, m dy
                const uint32_t vmask = __ballot_sync(0xffffffffu, valid);
                if (vmask == 0) continue;
                // transposing butterfly inside each quarter: 8 components in 7 shuffles, the ninth in 3
                const float a0 = (h4 ? v4 : v0) + shfl_x(h4 ? v0 : v4, 4);
                const float a1 = (h4 ? v5 : v1) + shfl_x(h4 ? v1 : v5, 4);
                const float a2 = (h4 ? v6 : v2) + shfl_x(h4 ? v2 : v6, 4);
                const float a3 = (h4 ? v7 : v3) + shfl_x(h4 ? v3 : v7, 4);
                const float b0 = (h2 ? a2 : a0) + shfl_x(h2 ? a0 : a2, 2);
                const float b1 = (h2 ? a3 : a1) + shfl_x(h2 ? a1 : a3, 2);
                const float c = (h1 ? b1 : b0) + shfl_x(h1 ? b0 : b1, 1);
                v8 += shfl_x(v8, 4);
                v8 += shfl_x(v8, 2);
                v8 += shfl_x(v8, 1);
                // quarters with at least one valid lane add their nine sums: lane k adds component k,
                // the first lane of the quarter also the ninth
                const bool qvalid = ((vmask >> (quarter * 8)) & 0xffu) != 0;
                if (qvalid) {
                    atomicAdd(&s_acc[j][slot], c);
                    if ((lane & 7) == 0) atomicAdd(&s_acc[j][8], v8);
                }
            }
        }
        __syncthreads();
        if (t < cnt) {
            const float* acc = s_acc[t];
            const float sxx = acc[0], sxy = acc[1], syy = acc[2], s0 = acc[3], g4 = acc[4], g5 = acc[5], g6 = acc[6],
                        sx = acc[7], sy = acc[8];
            const bool any = (sxx != 0.f) | (sxy != 0.f) | (syy != 0.f) | (s0 != 0.f) | (g4 != 0.f) | (g5 != 0.f) |
                             (g6 != 0.f) | (sx != 0.f) | (sy != 0.f);
            // conic = (-2 ha, -nb, -2 hc), render.py:2001-2017: d/dconic = -0.5 o sxx, -o sxy, -0.5 o syy;
            // d/duv = o (2 ha sx + nb sy, 2 hc sy + nb sx); d/dopacity = s0
            const float4 k1 = rec[t * 3 + 1];   // ha, nb, hc, opacity
            const float g0 = -0.5f * k1.w * sxx, g1 = -k1.w * sxy, g2 = -0.5f * k1.w * syy, g3 = s0;
            const float g7 = k1.w * fmaf(2.0f * k1.x, sx, k1.y * sy);
            const float g8 = k1.w * fmaf(2.0f * k1.z, sy, k1.y * sx);
            if (any) {
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
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" int32_t d3gs_raster_forward(const D3gsOpConfig* cfg, const int32_t* ranges, const int32_t* tile_order,
                                       const float* records, float* color, float* final_T, int32_t* n_contrib,
                                       uint32_t* status, void* stream) {
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
    raster_forward_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("raster_forward_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_raster_backward(const D3gsOpConfig* cfg, int64_t num, const int32_t* ranges,
                                        const int32_t* tile_order, const float* records,
                                        const int32_t* sorted_values, const float* color,
                                        const float* final_T, const int32_t* n_contrib, const float* drgb,
                                        const float* dT, float* splat_grads, uint32_t* status, void* stream) {
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
    raster_backward_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("raster_backward_kernel");
    return D3GS_OK;
}
