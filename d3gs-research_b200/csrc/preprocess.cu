// K1 preprocess forward and K3 key duplication.
//
// This translation unit is compiled with -fmad=false: every float expression below is evaluated
// exactly as written (IEEE add/mul/div/sqrt, explicit fmaf only), because the integer outputs of
// these stages -- radii, tile rectangles, tiles_touched, culling decisions, and the depth bits
// inside the sort keys -- must be reproducible bit for bit by a host program.
//
// Reference semantics: d3sim/algos/d3gs/render.py:250-681 (proxy branch 421-476, 569-619),
// 739-840, 1017-1327; math from d3sim/csrc/gs3d.py and d3sim/csrc/camera.py:307-333.
#include <type_traits>

#include "common.cuh"

namespace d3gs {
namespace {

struct TileGeom {
    int tiles_x, tiles_y;
    float ts;
};

// x / ts for the tile size 16 (the only one the entry points accept): a division by a power of two and the
// multiplication by its reciprocal round to the same float, and the multiplication is one instruction
// instead of the ~10 of an IEEE division.
__device__ __forceinline__ float div_ts(float x, const TileGeom& tg) {
    return tg.ts == 16.0f ? x * 0.0625f : x / tg.ts;
}

__device__ __forceinline__ void tile_rect(const TileGeom& tg, float u, float v, float radius, int* rmin, int* rmax) {
    // render.py:472-473: clamp(int((uv -/+ r (+ 15)) / 16), 0, tiles); max is exclusive
    rmin[0] = clampi(f2i_sat(div_ts(u - radius, tg)), 0, tg.tiles_x);
    rmin[1] = clampi(f2i_sat(div_ts(v - radius, tg)), 0, tg.tiles_y);
    rmax[0] = clampi(f2i_sat(div_ts(u + radius + tg.ts - 1.0f, tg)), 0, tg.tiles_x);
    rmax[1] = clampi(f2i_sat(div_ts(v + radius + tg.ts - 1.0f, tg)), 0, tg.tiles_y);
}

struct Obb {
    float w, h, s, c;
};

// gs3d.py:710-742
__device__ __forceinline__ void ellipse_bound_aabb(float ca, float cb, float cc, float bound, float* half) {
    float det = ca * cc - cb * cb;
    float vx = (-bound * cc) * det, vy = (-bound * ca) * det;
    float sx = sqrtf(fmaxf(0.0f, vx)) / det, sy = sqrtf(fmaxf(0.0f, vy)) / det;
    half[0] = fabsf(vx > 0.0f ? sx : 0.0f);
    half[1] = fabsf(vy > 0.0f ? sy : 0.0f);
}

// gs3d.py:744-793, 968-989
__device__ __forceinline__ Obb ellipse_bound_obb(float ca, float cb, float cc, float bound) {
    float A = -ca / bound, C = -cc / bound, Bh = -cb / bound;
    float det = A * C - Bh * Bh;
    float mid = 0.5f * (A + C);
    float sq = sqrtf(fmaxf(0.0f, mid * mid - det));
    float e1 = mid + sq, e2 = mid - sq;
    float s1 = e1 > 0.0f ? 1.0f : -1.0f, s2 = e2 > 0.0f ? 1.0f : -1.0f;
    float vx = e2 - C, vy = Bh;
    float vn = sqrtf(vx * vx + vy * vy);
    vx = vx / vn;
    vy = vy / vn;
    float minor = 1.0f / sqrtf(e1 * s1), major = 1.0f / sqrtf(e2 * s2);
    float mx = vx * major, my = vy * major;
    float mn = sqrtf(mx * mx + my * my);
    Obb r;
    r.w = major * 2.0f;
    r.h = minor * 2.0f;
    r.s = my / mn;
    r.c = mx / mn;
    return r;
}

// gs3d.py:1254-1322: separating-axis test, touching boxes do not overlap
__device__ __forceinline__ bool aabb_overlap_obb(float minx, float miny, float maxx, float maxy, const Obb& o,
                                                 float cx, float cy) {
    float l1x = (maxx - minx) / 2.0f, l1y = (maxy - miny) / 2.0f;
    float l2x = o.w / 2.0f, l2y = o.h / 2.0f;
    float lx = (maxx + minx) / 2.0f - cx, ly = (maxy + miny) / 2.0f - cy;
    const float ax[4][2] = {{1.0f, 0.0f}, {0.0f, 1.0f}, {o.c, o.s}, {-o.s, o.c}};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float ux = ax[k][0], uy = ax[k][1];
        float r1 = l1x * fabsf(ax[0][0] * ux + ax[0][1] * uy);
        float r2 = l1y * fabsf(ax[1][0] * ux + ax[1][1] * uy);
        float r3 = l2x * fabsf(ax[2][0] * ux + ax[2][1] * uy);
        float r4 = l2y * fabsf(ax[3][0] * ux + ax[3][1] * uy);
        if (((r1 + r2) + r3) + r4 <= fabsf(lx * ux + ly * uy)) return false;
    }
    return true;
}

// The tiles that the early filter keeps (render.py:1017-1327) intersected with the 3-sigma rect
// (render.py:594, 814-817).  filter: 0 NONE, 1 AABB, 2 ELLIPSE, 3 OBB; OBB_DFVT (4) is mapped to OBB by the host (same
// tile set by construction of the traversal).  The walk covers the box [bmin, bmax) row by row: the rect
// itself for NONE, the bounding box of the alpha >= alpha_eps ellipse otherwise.
// ELL: the walk can also evaluate the exact ellipse test (filter 2); it then keeps the conic and the bound, four
// more live registers, which is why the kernels that never need it are instantiated without.
struct EllipseState {
    float cx, cy, cz, bound;
};
struct NoEllipseState {};

// gs3d.py:1149-1178, 1210-1229 (the _v2 forms, offsets taken relative to the centre): where the ellipse
// cx dx^2 + 2 cy dx dy + cz dy^2 = -bound crosses the horizontal line y (the two x) or the vertical line x (the two y);
// (-1, -1) when it does not
__device__ __forceinline__ void ellipse_cross_y(const EllipseState& e, float y, float u, float v, float* r) {
    y -= v;
    const float val = -e.bound * e.cx - e.cx * e.cz * y * y + e.cy * e.cy * y * y;
    const float sq = f_sqrt(fmaxf(0.0f, val));
    r[0] = val >= 0.0f ? u + (-e.cy * y - sq) / e.cx : -1.0f;
    r[1] = val >= 0.0f ? u + (-e.cy * y + sq) / e.cx : -1.0f;
}
__device__ __forceinline__ void ellipse_cross_x(const EllipseState& e, float x, float u, float v, float* r) {
    x -= u;
    const float val = -e.bound * e.cz - e.cx * e.cz * x * x + e.cy * e.cy * x * x;
    const float sq = f_sqrt(fmaxf(0.0f, val));
    r[0] = val >= 0.0f ? v + (-e.cy * x - sq) / e.cz : -1.0f;
    r[1] = val >= 0.0f ? v + (-e.cy * x + sq) / e.cz : -1.0f;
}
// gs3d.py:1078-1117: an edge of the box is crossed, or the ellipse covers the box, or the box holds the centre
__device__ __forceinline__ bool ellipse_overlaps_box(const EllipseState& e, float px0, float py0, float px1, float py1,
                                                     float u, float v) {
    float x0[2], x1[2], y0[2], y1[2];
    ellipse_cross_x(e, px0, u, v, x0);
    ellipse_cross_x(e, px1, u, v, x1);
    ellipse_cross_y(e, py0, u, v, y0);
    ellipse_cross_y(e, py1, u, v, y1);
    bool hit = (x0[0] >= py0 && x0[0] <= py1) || (x0[1] >= py0 && x0[1] <= py1);
    hit |= (x1[0] >= py0 && x1[0] <= py1) || (x1[1] >= py0 && x1[1] <= py1);
    hit |= (y0[0] >= px0 && y0[0] <= px1) || (y0[1] >= px0 && y0[1] <= px1);
    hit |= (y1[0] >= px0 && y1[0] <= px1) || (y1[1] >= px0 && y1[1] <= px1);
    bool cover = x0[0] <= py0 && x0[1] >= py1;
    cover &= x1[0] <= py0 && x1[1] >= py1;
    cover &= y0[0] <= px0 && y0[1] >= px1;
    cover &= y1[0] <= px0 && y1[1] >= px1;
    const bool centre = px0 <= u && px1 >= u && py0 <= v && py1 >= v;
    return hit || cover || centre;
}

template <bool ELL>
struct TileWalkT {
    int filter, tile_px;
    float ts;
    int rmin[2], rmax[2], bmin[2], bmax[2];
    float half[2], ox, oy;
    Obb obb;
    typename std::conditional<ELL, EllipseState, NoEllipseState>::type ell;

    __device__ __forceinline__ void init(int filter_, const TileGeom& tg, int tile_px_, float alpha_eps, float u, float v,
                                         float ca, float cb, float cc, float opacity, const int* rmin_, const int* rmax_) {
        filter = filter_;
        tile_px = tile_px_;
        ts = tg.ts;
        rmin[0] = rmin_[0]; rmin[1] = rmin_[1]; rmax[0] = rmax_[0]; rmax[1] = rmax_[1];
        if (filter == 0) {
            bmin[0] = rmin[0]; bmin[1] = rmin[1]; bmax[0] = rmax[0]; bmax[1] = rmax[1];
            return;
        }
        float bound = 2.0f * act_log(alpha_eps / opacity);
        ellipse_bound_aabb(ca, cb, cc, bound, half);
        bmin[0] = clampi(f2i_sat(div_ts(u - half[0], tg)), 0, tg.tiles_x);
        bmin[1] = clampi(f2i_sat(div_ts(v - half[1], tg)), 0, tg.tiles_y);
        bmax[0] = clampi(f2i_sat(ceilf(div_ts(u + half[0], tg))), 0, tg.tiles_x);
        bmax[1] = clampi(f2i_sat(ceilf(div_ts(v + half[1], tg))), 0, tg.tiles_y);
        ox = u - (float)bmin[0] * tg.ts;
        oy = v - (float)bmin[1] * tg.ts;
        if constexpr (ELL) {
            if (filter == 2) {
                ell.cx = ca; ell.cy = cb; ell.cz = cc; ell.bound = bound;
                return;
            }
        }
        obb = ellipse_bound_obb(ca, cb, cc, bound);
    }
    __device__ __forceinline__ int width() const { return max(bmax[0] - bmin[0], 0); }
    __device__ __forceinline__ int area() const { return width() * max(bmax[1] - bmin[1], 0); }
    __device__ __forceinline__ bool test(int x, int y) const {
        if (filter == 0) return true;
        float py0 = (float)((y - bmin[1]) * tile_px), py1 = py0 + ts;
        float px0 = (float)((x - bmin[0]) * tile_px), px1 = px0 + ts;
        bool ok;
        if (filter == 1) {
            bool xo = (ox - half[0]) <= px1 && (ox + half[0]) >= px0;
            bool yo = (oy - half[1]) <= py1 && (oy + half[1]) >= py0;
            ok = xo && yo;
        } else if (ELL && filter == 2) {
            if constexpr (ELL) ok = ellipse_overlaps_box(ell, px0, py0, px1, py1, ox, oy);   // render.py:1277-1297
            else ok = false;
        } else {
            ok = aabb_overlap_obb(px0, py0, px1, py1, obb, ox, oy);
        }
        return ok && x >= rmin[0] && x < rmax[0] && y >= rmin[1] && y < rmax[1];
    }
    // one thread visits all kept tiles, row-major
    template <class F>
    __device__ __forceinline__ void for_each(F fn) const {
        for (int y = bmin[1]; y < bmax[1]; ++y)
            for (int x = bmin[0]; x < bmax[0]; ++x)
                if (test(x, y)) fn(x, y);
    }
};

// A Gaussian whose walk covers more tiles than this is handled by its whole warp (32 tiles per step)
// instead of by its own thread: a few screen-filling Gaussians otherwise keep one lane busy for thousands
// of iterations while the other 31 wait (measured: preprocess 0.24 -> 0.60 ms and key duplication
// 0.15 -> 0.57 ms once training had grown a handful of such Gaussians).
constexpr int kCoopTiles = 64;

// what a warp needs to rebuild another lane's TileWalk
struct WalkSeed {
    float u, v, ca, cb, cc, opacity;
    int rmin0, rmin1, rmax0, rmax1;
};

__device__ __forceinline__ WalkSeed bcast_seed(const WalkSeed& s, int src) {
    WalkSeed r;
    r.u = __shfl_sync(0xffffffffu, s.u, src); r.v = __shfl_sync(0xffffffffu, s.v, src);
    r.ca = __shfl_sync(0xffffffffu, s.ca, src); r.cb = __shfl_sync(0xffffffffu, s.cb, src);
    r.cc = __shfl_sync(0xffffffffu, s.cc, src); r.opacity = __shfl_sync(0xffffffffu, s.opacity, src);
    r.rmin0 = __shfl_sync(0xffffffffu, s.rmin0, src); r.rmin1 = __shfl_sync(0xffffffffu, s.rmin1, src);
    r.rmax0 = __shfl_sync(0xffffffffu, s.rmax0, src); r.rmax1 = __shfl_sync(0xffffffffu, s.rmax1, src);
    return r;
}

__constant__ float kShC2[5] = {1.0925484305920792f, -1.0925484305920792f, 0.31539156525252005f,
                               -1.0925484305920792f, 0.5462742152960396f};
__constant__ float kShC3[7] = {-0.5900435899266435f, 2.890611442640554f, -0.4570457994644658f, 0.3731763325901154f,
                               -0.4570457994644658f, 1.445305721320277f,  -0.5900435899266435f};

// gs3d.py:151-201: basis values, bs[0] = C0
__device__ __forceinline__ void sh_basis(int deg, float x, float y, float z, float* bs) {
    const float C1 = 0.4886025119029199f;
    bs[0] = 0.28209479177387814f;
    if (deg > 0) {
        bs[1] = -C1 * y;
        bs[2] = C1 * z;
        bs[3] = -C1 * x;
        if (deg > 1) {
            float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
            bs[4] = kShC2[0] * xy;
            bs[5] = kShC2[1] * yz;
            bs[6] = kShC2[2] * (2.0f * zz - xx - yy);
            bs[7] = kShC2[3] * xz;
            bs[8] = kShC2[4] * (xx - yy);
            if (deg > 2) {
                bs[9] = kShC3[0] * y * (3.0f * xx - yy);
                bs[10] = kShC3[1] * xy * z;
                bs[11] = kShC3[2] * y * (4.0f * zz - xx - yy);
                bs[12] = kShC3[3] * z * (2.0f * zz - 3.0f * xx - 3.0f * yy);
                bs[13] = kShC3[4] * x * (4.0f * zz - xx - yy);
                bs[14] = kShC3[5] * z * (xx - yy);
                bs[15] = kShC3[6] * x * (xx - 3.0f * yy);
            }
        }
    }
}

struct PrepArgs {
    D3gsOpConfig cfg;
    D3gsModel model;
    D3gsSplatContext ctx;
    const uint8_t* mask;
    uint32_t* status;     // optional: D3GS_STATUS_COPY_TIMEOUT when a CTA's coefficient rows never arrived
    TestHooks hooks;
};

constexpr int kRow = 45;   // shared-memory row length in floats (odd: conflict-free per-thread rows)

// One CTA handles 256 consecutive (view, Gaussian) items.  Geometry first; the l>=1 SH coefficients of
// the SURVIVING Gaussians only (180 bytes each) are then brought into shared memory with coalesced
// loads and evaluated per thread from there: per-thread global loads with a 180-byte stride cost ~22
// sectors per request.
// 64 registers (4 CTAs of 256 threads per SM): with 78 the kernel lost a fifth of its throughput
// INST: instance rendering, a per-Gaussian camera (12 more live registers; an instantiation of its own)
template <int DEG, bool INST, bool ELL>
__global__ void __launch_bounds__(256, (INST || ELL) ? 3 : 4) preprocess_fwd_kernel(const __grid_constant__ PrepArgs a) {
    using TileWalk = TileWalkT<ELL>;
    constexpr int NB = (DEG + 1) * (DEG + 1);
    constexpr int NR3 = (NB - 1) * 3;
    __shared__ __align__(128) float s_rest[NR3 > 0 ? 256 * kRow : 4];
    __shared__ int32_t s_src[256];   // Gaussian index whose coefficients row t needs, -1 = none
    __shared__ __align__(8) uint64_t s_bar;
    const int64_t N = a.model.num;
    const int64_t total = N * a.cfg.num_views;
    const int t = threadIdx.x;
    const int64_t i0 = (int64_t)blockIdx.x * 256;
    const int64_t i = i0 + t;
    const D3gsOpConfig& cf = a.cfg;
    // Fast staging: when the CTA's 256 rows are one contiguous, 16-byte aligned span of the coefficient
    // array (degree-3 layout, rows inside one view), a single bulk async copy fetches them while the
    // threads do the geometry.  Otherwise the rows of the surviving Gaussians are gathered afterwards.
    bool bulk = false;
    if (NR3 > 0) {
        const int64_t g_first = i0 % N;
        const int rows = (int)min((int64_t)256, total - i0);
        bulk = a.model.sh_rest_stride == 45 && g_first + rows <= N && (rows & 3) == 0 &&
               ((uintptr_t)(a.model.sh_rest + g_first * 45) & 15) == 0;
        if (bulk) {
            if (t == 0) {
                mbar_init(&s_bar, 1);
                fence_mbar_init();
                mbar_arrive_expect_tx(&s_bar, (uint32_t)rows * 180u);
                if ((int)blockIdx.x != a.hooks.hold)      // test hook: this CTA's copy is never issued
                    bulk_copy_g2s(s_rest, a.model.sh_rest + g_first * 45, (uint32_t)rows * 180u, &s_bar);
            }
            __syncthreads();   // the barrier is initialised before anybody polls it
        }
    }
    bool valid = i < total;
    bool big = false;        // this Gaussian's tile walk is left to the warp
    WalkSeed seed = {};
    int64_t g = 0;
    float d0 = 0.f, d1 = 0.f, d2 = 0.f;
    if (valid) {
        const int b = (int)(i / N);
        g = i - (int64_t)b * N;
        const D3gsCamera& cam = cf.cameras[b];
        const float* Rt = cam.cam2world_T;   // Rt[k*3 + j]: k-th column of R_c2w
        float Ri[12];
        if constexpr (INST) {
            if (instance_camera(cf, b, g, Ri)) Rt = Ri;
        }
        TileGeom tg;
        tg.tiles_x = (cf.width + cf.tile_x - 1) / cf.tile_x;
        tg.tiles_y = (cf.height + cf.tile_y - 1) / cf.tile_y;
        tg.ts = (float)cf.tile_x;
        const float px = a.model.xyz[g * 3], py = a.model.xyz[g * 3 + 1], pz = a.model.xyz[g * 3 + 2];
        d0 = px - Rt[9]; d1 = py - Rt[10]; d2 = pz - Rt[11];
        const float pc0 = (Rt[0] * d0 + Rt[1] * d1) + Rt[2] * d2;
        const float pc1 = (Rt[3] * d0 + Rt[4] * d1) + Rt[5] * d2;
        const float z = (Rt[6] * d0 + Rt[7] * d1) + Rt[8] * d2;
        if (!(z >= cf.near_plane && z <= cf.far_plane)) valid = false;
        if (a.mask != nullptr && a.mask[i] != 0) valid = false;
        if (valid) {
            const float u = ((pc0 / z) * cam.fx + cam.cx) - 0.5f;
            const float v = ((pc1 / z) * cam.fy + cam.cy) - 0.5f;
            // fused activations
            const float4 qr = *reinterpret_cast<const float4*>(a.model.quaternion_xyzw + g * 4);
            const bool fused = cf.fused_activations != 0;
            const float qn = fused ? sqrtf(((qr.x * qr.x + qr.y * qr.y) + qr.z * qr.z) + qr.w * qr.w) : 1.0f;
            const float qx = qr.x / qn, qy = qr.y / qn, qz = qr.z / qn, qw = qr.w / qn;
            const float sg = cf.training ? 1.0f : cf.scale_global;
            const float r0 = a.model.scale[g * 3], r1 = a.model.scale[g * 3 + 1], r2 = a.model.scale[g * 3 + 2];
            const float s0 = (fused ? act_exp(r0) : r0) * sg, s1 = (fused ? act_exp(r1) : r1) * sg,
                        s2 = (fused ? act_exp(r2) : r2) * sg;
            const float oraw = a.model.opacity[g];
            const float opac = fused ? 1.0f / (1.0f + act_exp(-oraw)) : oraw;
            // rotation, M = R diag(s), Sigma = M M^T
            float R[3][3];
            {
                float xx = qx * qx, yy = qy * qy, zz = qz * qz, xy = qx * qy, xz = qx * qz, yz = qy * qz;
                float wx = qw * qx, wy = qw * qy, wz = qw * qz;
                R[0][0] = 1.0f - 2.0f * (yy + zz); R[0][1] = 2.0f * (xy - wz); R[0][2] = 2.0f * (xz + wy);
                R[1][0] = 2.0f * (xy + wz); R[1][1] = 1.0f - 2.0f * (xx + zz); R[1][2] = 2.0f * (yz - wx);
                R[2][0] = 2.0f * (xz - wy); R[2][1] = 2.0f * (yz + wx); R[2][2] = 1.0f - 2.0f * (xx + yy);
            }
            float M[3][3];
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                M[r][0] = R[r][0] * s0;
                M[r][1] = R[r][1] * s1;
                M[r][2] = R[r][2] * s2;
            }
            float Sg[3][3];
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int c = r; c < 3; ++c)
                    Sg[r][c] = Sg[c][r] = (M[r][0] * M[c][0] + M[r][1] * M[c][1]) + M[r][2] * M[c][2];
            // projection
            const float tanx = 0.5f * (float)cf.width / cam.fx, tany = 0.5f * (float)cf.height / cam.fy;
            const float limx = fabsf((tanx * cf.projected_clamp_factor) * z), limy = fabsf((tany * cf.projected_clamp_factor) * z);
            const float tx = fminf(limx, fmaxf(-limx, pc0)), ty = fminf(limy, fmaxf(-limy, pc1));
            const float z2 = z * z;
            const float J00 = cam.fx / z, J02 = -(tx * cam.fx) / z2, J11 = cam.fy / z, J12 = -(ty * cam.fy) / z2;
            float T0[3], T1[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                T0[j] = J00 * Rt[j] + J02 * Rt[6 + j];
                T1[j] = J11 * Rt[3 + j] + J12 * Rt[6 + j];
            }
            float U0[3], U1[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                U0[j] = (T0[0] * Sg[0][j] + T0[1] * Sg[1][j]) + T0[2] * Sg[2][j];
                U1[j] = (T1[0] * Sg[0][j] + T1[1] * Sg[1][j]) + T1[2] * Sg[2][j];
            }
            float ca = (U0[0] * T0[0] + U0[1] * T0[1]) + U0[2] * T0[2];
            float cb = (U0[0] * T1[0] + U0[1] * T1[1]) + U0[2] * T1[2];
            float cc = (U1[0] * T1[0] + U1[1] * T1[1]) + U1[2] * T1[2];
            ca += cf.gaussian_lowpass_filter;
            cc += cf.gaussian_lowpass_filter;
            float det = ca * cc - cb * cb;
            float k0, k1, k2, opq = opac;
            if (cf.anti_aliasing) {
                // gs3d.py:592-619, render.py:449-462: the conic inverts the low-passed covariance without the eps
                // guard, `det` becomes the determinant BEFORE the low-pass (it feeds the radius and the validity
                // test below, as in the reference), and the opacity is scaled by sqrt(det / det_lowpass)
                const float a0 = ca - cf.gaussian_lowpass_filter, c0 = cc - cf.gaussian_lowpass_filter;
                const float det_l = det;
                det = a0 * c0 - cb * cb;
                const float inv = 1.0f / det_l;
                k0 = cc * inv; k1 = -cb * inv; k2 = ca * inv;
                opq = opac * sqrtf(fmaxf(0.000025f, det / det_l));
            } else {
                const float det_inv = 1.0f / (det + cf.eps);
                k0 = cc * det_inv; k1 = -cb * det_inv; k2 = ca * det_inv;
            }
            const float mid = 0.5f * (ca + cc);
            const float sq = sqrtf(fmaxf(cf.cov2d_radii_eigen_eps, mid * mid - det));
            const float radius = ceilf(cf.gaussian_std_sigma * sqrtf(fmaxf(mid + sq, mid - sq)));
            int rmin[2], rmax[2];
            tile_rect(tg, u, v, radius, rmin, rmax);
            const int area = (rmax[0] - rmin[0]) * (rmax[1] - rmin[1]);
            if (det <= 0.0f || area == 0 || opq <= cf.alpha_eps) {
                valid = false;
            } else {
                int cnt = 0;
                // accepted tiles as a bit mask over the 3-sigma rect (row-major), so that the key
                // duplication does not have to repeat the overlap tests; rects above 64 tiles are re-walked
                uint64_t tmask = 0;
                const int rw = rmax[0] - rmin[0];
                const bool small_rect = area <= 64;
                TileWalk walk;
                walk.init(cf.early_filter_algo, tg, cf.tile_x, cf.alpha_eps, u, v, k0, k1, k2, opq, rmin, rmax);
                if (walk.area() > kCoopTiles && !small_rect) {   // a small rect keeps its bit mask: walked here
                    big = true;   // counted by the whole warp below
                    seed.u = u; seed.v = v; seed.ca = k0; seed.cb = k1; seed.cc = k2; seed.opacity = opq;
                    seed.rmin0 = rmin[0]; seed.rmin1 = rmin[1]; seed.rmax0 = rmax[0]; seed.rmax1 = rmax[1];
                } else {
                    int32_t* tcount = a.ctx.tile_counts != nullptr ? a.ctx.tile_counts + (int64_t)b * (tg.tiles_x * tg.tiles_y)
                                                                   : nullptr;
                    walk.for_each([&](int x, int y) {
                        ++cnt;
                        if (small_rect) tmask |= 1ull << ((y - rmin[1]) * rw + (x - rmin[0]));
                        if (tcount != nullptr) atomicAdd(tcount + (y * tg.tiles_x + x), 1);
                    });
                }
                if (a.ctx.tile_mask != nullptr) a.ctx.tile_mask[i] = tmask;
                a.ctx.tiles_touched[i] = cnt;
                a.ctx.radii[i] = (int)radius;
                a.ctx.depths[i] = cf.inv_depth ? 1.0f / z : z;   // render.py:582 (this array also feeds the sort keys)
                *reinterpret_cast<float2*>(a.ctx.uvs + i * 2) = make_float2(u, v);
                *reinterpret_cast<float4*>(a.ctx.conic_opacity + i * 4) = make_float4(k0, k1, k2, opq);
                if (a.ctx.cov2d_vecs != nullptr) {
                    a.ctx.cov2d_vecs[i * 3] = ca;
                    a.ctx.cov2d_vecs[i * 3 + 1] = cb;
                    a.ctx.cov2d_vecs[i * 3 + 2] = cc;
                }
            }
        }
        if (!valid) {
            a.ctx.tiles_touched[i] = 0;
            a.ctx.radii[i] = 0;
        }
    }
    {   // large walks, one after the other, 32 tiles per step (every lane of the warp takes part)
        uint32_t todo = __ballot_sync(0xffffffffu, big);
        if (todo) {
            TileGeom tg;
            tg.tiles_x = (cf.width + cf.tile_x - 1) / cf.tile_x;
            tg.tiles_y = (cf.height + cf.tile_y - 1) / cf.tile_y;
            tg.ts = (float)cf.tile_x;
            const int lane = t & 31;
            while (todo) {
                const int src = __ffs(todo) - 1;
                todo &= todo - 1;
                const WalkSeed sd = bcast_seed(seed, src);
                const int rmin[2] = {sd.rmin0, sd.rmin1}, rmax[2] = {sd.rmax0, sd.rmax1};
                TileWalk walk;
                walk.init(cf.early_filter_algo, tg, cf.tile_x, cf.alpha_eps, sd.u, sd.v, sd.ca, sd.cb, sd.cc, sd.opacity,
                          rmin, rmax);
                const int bw = walk.width(), n_tiles = walk.area();
                int32_t* tcount = nullptr;
                if (a.ctx.tile_counts != nullptr) {
                    const int64_t isrc = i0 + (t & ~31) + src;     // flat index of the lane whose walk this is
                    tcount = a.ctx.tile_counts + (isrc / N) * (int64_t)(tg.tiles_x * tg.tiles_y);
                }
                int cnt = 0;
                for (int q0 = 0; q0 < n_tiles; q0 += 32) {
                    const int q = q0 + lane;
                    const int x = walk.bmin[0] + q % bw, y = walk.bmin[1] + q / bw;
                    const bool ok = q < n_tiles && walk.test(x, y);
                    cnt += __popc(__ballot_sync(0xffffffffu, ok));
                    if (ok && tcount != nullptr) atomicAdd(tcount + (y * tg.tiles_x + x), 1);
                }
                if (lane == src) a.ctx.tiles_touched[i] = cnt;
            }
        }
    }
    if constexpr (NR3 > 0) {
        if (bulk) {
            if (!mbar_wait_bounded(&s_bar, 0, a.hooks.poll_limit)) {
                // The copy never landed: no colour and no raster record leave this CTA, and the caller learns of it
                // through the status word (tile counts of these Gaussians are already out: the launch's results
                // are invalid as a whole).
                valid = false;
                if (t == 0 && a.status != nullptr) atomicOr(a.status, D3GS_STATUS_COPY_TIMEOUT);
            }
        } else {
            s_src[t] = valid ? (int32_t)g : -1;
            __syncthreads();
            const float* src = a.model.sh_rest;
            const int64_t stride = a.model.sh_rest_stride;
            constexpr int kU = NR3 % 9 == 0 ? 9 : 3;   // loads of one round are issued back to back
            for (int f0 = t; f0 < 256 * NR3; f0 += 256 * kU) {
                float tmp[kU];
                int dst[kU];
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const int f = f0 + u * 256;
                    const int row = f / NR3, k = f - row * NR3;
                    const int32_t gs = f < 256 * NR3 ? s_src[row] : -1;
                    dst[u] = gs >= 0 ? row * kRow + k : -1;
                    tmp[u] = gs >= 0 ? src[(int64_t)gs * stride + k] : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < kU; ++u)
                    if (dst[u] >= 0) s_rest[dst[u]] = tmp[u];
            }
            __syncthreads();
        }
    }
    if (!valid) return;
    // colour: SH of the normalised world-space view direction (render.py:587, 605-611)
    const float dn = sqrtf((d0 * d0 + d1 * d1) + d2 * d2);
    float bs[16];
    sh_basis(DEG, d0 / dn, d1 / dn, d2 / dn, bs);
    const float* base = a.model.sh_base + g * a.model.sh_base_stride;
    const float* rest = s_rest + t * kRow;
    float c3[3];
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) c3[ch] = bs[0] * base[ch];
#pragma unroll
    for (int k = 1; k < NB; ++k) {
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) c3[ch] = c3[ch] + bs[k] * rest[(k - 1) * 3 + ch];
    }
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) c3[ch] = c3[ch] + 0.5f;
    if (a.ctx.sh_to_rgb_ne_0 != nullptr)
        a.ctx.sh_to_rgb_ne_0[i] = (uint8_t)(((c3[0] < 0.0f) << 2) | ((c3[1] < 0.0f) << 1) | (c3[2] < 0.0f));
    const float cr = fmaxf(c3[0], 0.0f), cg = fmaxf(c3[1], 0.0f), cb = fmaxf(c3[2], 0.0f);
    a.ctx.rgb_gaussian[i * 3] = cr;
    a.ctx.rgb_gaussian[i * 3 + 1] = cg;
    a.ctx.rgb_gaussian[i * 3 + 2] = cb;
    if (a.ctx.records != nullptr) {
        // the raster record of this Gaussian (this thread wrote uv and the conic above)
        const float2 uv = *reinterpret_cast<const float2*>(a.ctx.uvs + i * 2);
        const float4 co = *reinterpret_cast<const float4*>(a.ctx.conic_opacity + i * 4);
        float4 r0, r1, r2;
        make_splat_record(uv, co, cr, cg, cb, cf.alpha_eps, r0, r1, r2);
        float4* dst = reinterpret_cast<float4*>(a.ctx.records) + i * 3;
        dst[0] = r0; dst[1] = r1; dst[2] = r2;
    }
}

struct DupArgs {
    D3gsOpConfig cfg;
    D3gsSplatContext ctx;
    const int32_t* scan;
    uint64_t* keys;
    int32_t* values;
    int32_t* cursor;      // BUCKET: next free position of every tile's range
    uint64_t* entries;    // BUCKET: depth bits << 32 | flat index, one per pair, in the tile's range
    int64_t num;
    const int64_t* total_pairs;   // BUCKET, optional: the pair count on the device, checked against pair_capacity
    int64_t pair_capacity;
};

// BUCKET == false: key = tile << shift | depth bits and value = flat index at the Gaussian's scanned offset
// (render.py:739-840).  BUCKET == true: the pair becomes one 8-byte entry, depth bits << 32 | flat index, at a
// position drawn from the tile's cursor inside the tile's range.
template <bool BUCKET, bool ELL>
__global__ void __launch_bounds__(256) duplicate_keys_kernel(const __grid_constant__ DupArgs a) {
    using TileWalk = TileWalkT<ELL>;
    // entries sized before the pair count was known: write nothing when the pairs do not fit (the caller repeats)
    if (BUCKET && a.total_pairs != nullptr && *a.total_pairs > a.pair_capacity) return;
    const int64_t total = a.num * a.cfg.num_views;
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const D3gsOpConfig& cf = a.cfg;
    TileGeom tg;
    tg.tiles_x = (cf.width + cf.tile_x - 1) / cf.tile_x;
    tg.tiles_y = (cf.height + cf.tile_y - 1) / cf.tile_y;
    tg.ts = (float)cf.tile_x;
    const int shift = cf.key_shift_bits == 18 ? 18 : 32;
    const int r = i < total ? a.ctx.radii[i] : 0;
    bool big = false;        // emitted by the whole warp below
    WalkSeed seed = {};
    int64_t off = 0;
    uint32_t dbits = 0;
    uint64_t tile_base = 0;
    if (r > 0) {
        const int b = (int)(i / a.num);
        if (!BUCKET) off = i == 0 ? 0 : (int64_t)a.scan[i - 1];
        const float2 uv = *reinterpret_cast<const float2*>(a.ctx.uvs + i * 2);
        int rmin[2], rmax[2];
        tile_rect(tg, uv.x, uv.y, (float)r, rmin, rmax);
        // 64-bit keys carry the depth's bits (depth > 0: bit order = numeric order); 32-bit keys an 18-bit
        // quantised depth (render.py:767-773)
        dbits = shift == 32 ? __float_as_uint(a.ctx.depths[i])
                            : ((uint32_t)(a.ctx.depths[i] / cf.depth_32bit_prec) & 0x3FFFFu);
        tile_base = (uint64_t)b * (uint64_t)(tg.tiles_x * tg.tiles_y);
        const int rw = rmax[0] - rmin[0];
        if (a.ctx.tile_mask != nullptr && rw * (rmax[1] - rmin[1]) <= 64) {
            // the preprocess left the accepted tiles as a row-major bit mask over the 3-sigma rect
            uint64_t m = a.ctx.tile_mask[i];
            // bit / rw by one multiplication: exact for bit < 64 and rw <= 64
            const uint32_t rcp = (65536u + (uint32_t)max(rw, 1) - 1u) / (uint32_t)max(rw, 1);
            if (BUCKET) {
                // The position of an entry comes back from an atomic on its tile's cursor: four tiles at a time, so
                // that the four round trips to L2 overlap instead of following one another.
                const uint64_t e = ((uint64_t)dbits << 32) | (uint32_t)i;
                while (m) {
                    int32_t* cur[4];
                    int nt = 0;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        cur[u] = a.cursor;
                        if (m) {
                            const int bit = __ffsll((long long)m) - 1;
                            m &= m - 1;
                            const int by = (int)(((uint32_t)bit * rcp) >> 16);
                            cur[u] = a.cursor + (tile_base + (uint64_t)((rmin[1] + by) * tg.tiles_x + rmin[0] + (bit - by * rw)));
                            nt = u + 1;
                        }
                    }
                    int pos[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (u < nt) pos[u] = atomicAdd(cur[u], 1);
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (u < nt) a.entries[pos[u]] = e;
                }
            } else {
                while (m) {
                    const int bit = __ffsll((long long)m) - 1;
                    m &= m - 1;
                    const int by = (int)(((uint32_t)bit * rcp) >> 16);
                    const int y = rmin[1] + by, x = rmin[0] + (bit - by * rw);
                    const uint64_t key = tile_base + (uint64_t)(y * tg.tiles_x + x);
                    a.keys[off] = (key << shift) | dbits;
                    a.values[off] = (int32_t)i;
                    ++off;
                }
            }
        } else {
            const float4 co = *reinterpret_cast<const float4*>(a.ctx.conic_opacity + i * 4);
            TileWalk walk;
            walk.init(cf.early_filter_algo, tg, cf.tile_x, cf.alpha_eps, uv.x, uv.y, co.x, co.y, co.z, co.w, rmin, rmax);
            if (walk.area() > kCoopTiles) {
                big = true;
                seed.u = uv.x; seed.v = uv.y; seed.ca = co.x; seed.cb = co.y; seed.cc = co.z; seed.opacity = co.w;
                seed.rmin0 = rmin[0]; seed.rmin1 = rmin[1]; seed.rmax0 = rmax[0]; seed.rmax1 = rmax[1];
            } else {
                walk.for_each([&](int x, int y) {
                    uint64_t key = tile_base + (uint64_t)(y * tg.tiles_x + x);
                    if (BUCKET) {
                        a.entries[atomicAdd(a.cursor + key, 1)] = ((uint64_t)dbits << 32) | (uint32_t)i;
                    } else {
                        a.keys[off] = (key << shift) | dbits;
                        a.values[off] = (int32_t)i;
                        ++off;
                    }
                });
            }
        }
    }
    // large walks: the warp tests 32 tiles per step and emits the kept ones in row-major order
    uint32_t todo = __ballot_sync(0xffffffffu, big);
    const int lane = threadIdx.x & 31;
    while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        const WalkSeed sd = bcast_seed(seed, src);
        const int rmin[2] = {sd.rmin0, sd.rmin1}, rmax[2] = {sd.rmax0, sd.rmax1};
        int64_t o = __shfl_sync(0xffffffffu, off, src);
        const uint32_t db = __shfl_sync(0xffffffffu, dbits, src);
        const uint64_t tb = __shfl_sync(0xffffffffu, tile_base, src);
        const int32_t id = (int32_t)__shfl_sync(0xffffffffu, (int)i, src);
        TileWalk walk;
        walk.init(cf.early_filter_algo, tg, cf.tile_x, cf.alpha_eps, sd.u, sd.v, sd.ca, sd.cb, sd.cc, sd.opacity, rmin, rmax);
        const int bw = walk.width(), n_tiles = walk.area();
        for (int q0 = 0; q0 < n_tiles; q0 += 32) {
            const int q = q0 + lane;
            const int x = walk.bmin[0] + (bw > 0 ? q % bw : 0), y = walk.bmin[1] + (bw > 0 ? q / bw : 0);
            const bool ok = q < n_tiles && walk.test(x, y);
            const uint32_t m = __ballot_sync(0xffffffffu, ok);
            if (ok) {
                if (BUCKET) {
                    a.entries[atomicAdd(a.cursor + (tb + (uint64_t)(y * tg.tiles_x + x)), 1)] =
                        ((uint64_t)db << 32) | (uint32_t)id;
                } else {
                    const int64_t dst = o + __popc(m & ((1u << lane) - 1u));
                    a.keys[dst] = ((tb + (uint64_t)(y * tg.tiles_x + x)) << shift) | db;
                    a.values[dst] = id;
                }
            }
            o += __popc(m);
        }
    }
}

int32_t check_cfg(const D3gsOpConfig* cfg) {
    D3GS_REQUIRE(cfg != nullptr, "cfg is NULL");
    D3GS_REQUIRE(cfg->tile_x == 16 && cfg->tile_y == 16, "only 16x16 tiles are supported (got %dx%d)", cfg->tile_x,
                 cfg->tile_y);
    D3GS_REQUIRE(cfg->width > 0 && cfg->height > 0, "bad image size %dx%d", cfg->width, cfg->height);
    D3GS_REQUIRE(cfg->num_views >= 1 && cfg->num_views <= D3GS_MAX_VIEWS, "num_views %d outside [1,%d]",
                 cfg->num_views, D3GS_MAX_VIEWS);
    D3GS_REQUIRE(cfg->sh_degree >= 0 && cfg->sh_degree <= 3, "sh_degree %d outside [0,3]", cfg->sh_degree);
    D3GS_REQUIRE(cfg->early_filter_algo >= 0 && cfg->early_filter_algo <= 4,
                 "early_filter_algo %d unsupported (NONE=0, AABB=1, ELLIPSE=2, OBB=3, OBB_DFVT=4)", cfg->early_filter_algo);
    D3GS_REQUIRE(cfg->key_shift_bits == 0 || cfg->key_shift_bits == 32 || cfg->key_shift_bits == 18,
                 "key_shift_bits must be 32 (64-bit keys) or 18 (32-bit keys), got %d", cfg->key_shift_bits);
    if (cfg->key_shift_bits == 18) {
        const int64_t tiles = (int64_t)cfg->num_views * ((cfg->width + 15) / 16) * ((cfg->height + 15) / 16);
        D3GS_REQUIRE(tiles < (1 << 14), "32-bit sort keys hold 14 bits of tile index: %lld tiles", (long long)tiles);
        D3GS_REQUIRE(cfg->depth_32bit_prec > 0.0f, "depth_32bit_prec must be positive");
    }
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" int32_t d3gs_preprocess_forward(const D3gsOpConfig* cfg, const D3gsModel* model, const uint8_t* mask,
                                           const D3gsSplatContext* ctx, uint32_t* status, void* stream) {
    int32_t rc = check_cfg(cfg);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(model != nullptr && ctx != nullptr, "model/ctx is NULL");
    D3GS_REQUIRE(model->num >= 0, "negative Gaussian count");
    D3GS_REQUIRE(model->xyz && model->quaternion_xyzw && model->scale && model->opacity && model->sh_base,
                 "model tensor pointer is NULL");
    D3GS_REQUIRE(cfg->sh_degree == 0 || model->sh_rest != nullptr, "sh_rest is NULL with sh_degree > 0");
    D3GS_REQUIRE(((uintptr_t)model->quaternion_xyzw & 15) == 0, "quaternion_xyzw must be 16-byte aligned");
    D3GS_REQUIRE(ctx->tiles_touched && ctx->radii && ctx->depths && ctx->uvs && ctx->conic_opacity && ctx->rgb_gaussian,
                 "context tensor pointer is NULL");
    D3GS_REQUIRE(((uintptr_t)ctx->uvs & 7) == 0 && ((uintptr_t)ctx->conic_opacity & 15) == 0,
                 "uvs / conic_opacity must be 8 / 16-byte aligned");
    D3GS_REQUIRE(((uintptr_t)ctx->records & 15) == 0, "records must be 16-byte aligned");
    D3GS_REQUIRE(!cfg->training || (ctx->cov2d_vecs && ctx->sh_to_rgb_ne_0),
                 "training needs cov2d_vecs and sh_to_rgb_ne_0");
    const int64_t total = model->num * cfg->num_views;
    cudaStream_t s = (cudaStream_t)stream;
    if (ctx->tile_counts != nullptr) {
        const size_t tiles = (size_t)cfg->num_views * ((cfg->width + 15) / 16) * ((cfg->height + 15) / 16);
        D3GS_CUDA(cudaMemsetAsync(ctx->tile_counts, 0, tiles * sizeof(int32_t), s));
    }
    if (total == 0) return D3GS_OK;
    D3GS_REQUIRE(total < (int64_t)1 << 31, "B*N = %lld does not fit int32 indexing", (long long)total);
    PrepArgs a;
    a.cfg = *cfg;
    if (a.cfg.early_filter_algo == 4) a.cfg.early_filter_algo = 3;
    a.model = *model;
    a.ctx = *ctx;
    a.mask = mask;
    a.status = status;
    a.hooks = test_hooks();
    dim3 grid((unsigned)div_up64(total, 256));
    if (cfg->instance_id != nullptr)
        D3GS_REQUIRE(cfg->instance2world_T != nullptr && cfg->num_instance > 0, "instance rendering needs instance2world_T");
    // instances of their own for instance rendering and for the exact ellipse filter (both keep more state live)
#define D3GS_LAUNCH_PREP(DEG)                                                                           \
    do {                                                                                                \
        if (cfg->instance_id != nullptr) {                                                              \
            if (ellipse) preprocess_fwd_kernel<DEG, true, true><<<grid, 256, 0, s>>>(a);                \
            else preprocess_fwd_kernel<DEG, true, false><<<grid, 256, 0, s>>>(a);                       \
        } else {                                                                                        \
            if (ellipse) preprocess_fwd_kernel<DEG, false, true><<<grid, 256, 0, s>>>(a);               \
            else preprocess_fwd_kernel<DEG, false, false><<<grid, 256, 0, s>>>(a);                      \
        }                                                                                               \
    } while (0)
    const bool ellipse = a.cfg.early_filter_algo == 2;
    switch (cfg->sh_degree) {
        case 0: D3GS_LAUNCH_PREP(0); break;
        case 1: D3GS_LAUNCH_PREP(1); break;
        case 2: D3GS_LAUNCH_PREP(2); break;
        default: D3GS_LAUNCH_PREP(3); break;
    }
#undef D3GS_LAUNCH_PREP
    D3GS_LAUNCH_CHECK("preprocess_fwd_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_duplicate_keys(const D3gsOpConfig* cfg, int64_t num, const int32_t* scan,
                                       const D3gsSplatContext* ctx, uint64_t* keys, int32_t* values, void* stream) {
    int32_t rc = check_cfg(cfg);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(ctx != nullptr && scan != nullptr, "ctx/scan is NULL");
    const int64_t total = num * cfg->num_views;
    if (total == 0) return D3GS_OK;
    D3GS_REQUIRE(keys != nullptr && values != nullptr, "keys/values is NULL");
    DupArgs a;
    a.cfg = *cfg;
    if (a.cfg.early_filter_algo == 4) a.cfg.early_filter_algo = 3;
    a.ctx = *ctx;
    a.scan = scan;
    a.keys = keys;
    a.values = values;
    a.num = num;
    if (a.cfg.early_filter_algo == 2)
        duplicate_keys_kernel<false, true><<<(unsigned)div_up64(total, 256), 256, 0, (cudaStream_t)stream>>>(a);
    else
        duplicate_keys_kernel<false, false><<<(unsigned)div_up64(total, 256), 256, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("duplicate_keys_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_bucket_emit(const D3gsOpConfig* cfg, int64_t num, const D3gsSplatContext* ctx, int32_t* cursor,
                                    uint64_t* entries, const int64_t* total_pairs, int64_t pair_capacity, void* stream) {
    int32_t rc = check_cfg(cfg);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(cfg->key_shift_bits == 0 || cfg->key_shift_bits == 32,
                 "tile-bucket binning orders by the 32 depth bits (64-bit sort keys); got key_shift_bits %d",
                 cfg->key_shift_bits);
    D3GS_REQUIRE(ctx != nullptr, "ctx is NULL");
    const int64_t total = num * cfg->num_views;
    if (total == 0) return D3GS_OK;
    D3GS_REQUIRE(cursor != nullptr && entries != nullptr, "cursor/entries is NULL");
    D3GS_REQUIRE(ctx->radii && ctx->depths && ctx->uvs && ctx->conic_opacity, "context tensor pointer is NULL");
    DupArgs a = {};
    a.cfg = *cfg;
    if (a.cfg.early_filter_algo == 4) a.cfg.early_filter_algo = 3;
    a.ctx = *ctx;
    a.cursor = cursor;
    a.entries = entries;
    a.num = num;
    a.total_pairs = pair_capacity > 0 ? total_pairs : nullptr;
    a.pair_capacity = pair_capacity;
    if (a.cfg.early_filter_algo == 2)
        duplicate_keys_kernel<true, true><<<(unsigned)div_up64(total, 256), 256, 0, (cudaStream_t)stream>>>(a);
    else
        duplicate_keys_kernel<true, false><<<(unsigned)div_up64(total, 256), 256, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("duplicate_keys_kernel<bucket>");
    return D3GS_OK;
}
