// K8 preprocess backward: chain rule from the rasteriser's per-splat gradients (duv, dconic,
// dopacity, dcolor) back to the 59 parameter floats of every Gaussian.
//
// Reference semantics: d3sim/algos/d3gs/render.py:3176-3360 with
//   gaussian_2d_inverse_and_det_grad   d3sim/csrc/gs3d.py:559-588
//   project_gaussian_to_2d_grad        gs3d.py:472-532
//   scale_quat_to_cov3d_grad           gs3d.py:387-418
//   pos_cam_to_uv_no_distort_grad      d3sim/csrc/camera.py:335-371
//   sh_dir_to_rgb_grad                 gs3d.py:236-366
//   fused activation gradients         d3sim/algos/d3gs/origin/model.py:327-431
// One thread per Gaussian; the view batch is looped inside and summed (render.py:3182,
// origin/model.py:422-431).  Unlike the reference (zeros_like + skip, render.py:2918, 3218-3220) every
// output element is written here, zeros included, so the caller needs no memset of the
// 236-byte-per-Gaussian gradient.  The rasteriser's per-splat gradients arrive packed, 48 bytes per
// (view, Gaussian).
#include "common.cuh"
#include "exchange.cuh"

namespace d3gs {
namespace {

struct BwdArgs {
    D3gsOpConfig cfg;
    D3gsModel model;
    D3gsModelGrad grad;
    // Per view b, indexed by the Gaussian: what the backward reads of that view.  One process, B views: slices of
    // the [B*N, .] context arrays.  Data parallel (PEER): view b is rank b's, and the pointers are rank b's
    // buffers as mapped in this process -- the loads cross NVLink.
    const float* v_grads[D3GS_MAX_VIEWS];     // [N, 12]: dconic a b c, dopacity | dcolor r g b, dz | duv x y, - -
    const int32_t* v_radii[D3GS_MAX_VIEWS];   // [N]
    const float* v_cov2d[D3GS_MAX_VIEWS];     // [N, 3]
    const uint8_t* v_ne0[D3GS_MAX_VIEWS];     // [N]
    int64_t g_begin, g_count;                 // the Gaussians this launch covers (PEER: this rank's share)
    // PEER: where the updated parameters go -- every rank's flat parameter buffer, and the element offset of each
    // field inside it; the flags that order the ranks' launches
    D3gsPeerSet peers;
    int64_t field_off[6];
    uint32_t* status;                         // optional device word for D3GS_STATUS_COPY_TIMEOUT
    TestHooks hooks;
    // fused optimizer step (ADAM variant): per field xyz, quaternion, scale, opacity, sh_base, sh_rest
    SegConst sc[6];
    float* exp_avg[6];
    float* exp_avg_sq[6];
    int32_t has_stats;
    D3gsDensifyStats stats;
};

constexpr int kRow = 45;        // shared-memory row length in floats (odd: conflict-free per-thread rows)

__constant__ float kC2[5] = {1.0925484305920792f, -1.0925484305920792f, 0.31539156525252005f, -1.0925484305920792f,
                             0.5462742152960396f};
__constant__ float kC3[7] = {-0.5900435899266435f, 2.890611442640554f, -0.4570457994644658f, 0.3731763325901154f,
                             -0.4570457994644658f, 1.445305721320277f,  -0.5900435899266435f};

// One CTA handles 256 consecutive Gaussians.  The l>=1 SH coefficients (180 bytes per Gaussian) are
// brought into shared memory with coalesced loads, each thread works on its own row, writes the
// coefficient gradients back into the row, and the rows leave with coalesced stores: per-thread
// accesses with a 180-byte stride cost 20-30 sectors per request and throttled the load/store unit.
// MULTI (more than one view): gradients accumulate over views in a second shared-memory buffer.
// ADAM (single GPU, single view): the gradient is not written at all.  The thread applies Adam to the 14
// floats of its Gaussian's small fields straight from registers, and the CTA applies it to its 256 x 45
// higher-order SH coefficients with coalesced accesses, taking the gradient rows from shared memory.  Compared
// with a gradient buffer followed by the optimizer kernel this removes one write and one read of the whole
// 236-byte-per-Gaussian gradient.
//
// One tile of 256 Gaussians starting at Gaussian g0.  Returns false when the CTA must stop (a staging copy never
// arrived).  `phase`: parity of the staging barrier, toggled per staged tile.
// what one view contributes for one Gaussian: the rasteriser's packed gradient row and the context it left
struct ViewIn {
    float4 gA, gB, gC;
    float ca, cb, cc;
    uint32_t ne0;
};
__device__ __forceinline__ ViewIn load_view(const BwdArgs& a, int b, int64_t g) {
    ViewIn v;
    const float4* sg4 = reinterpret_cast<const float4*>(a.v_grads[b] + g * D3GS_SPLAT_GRAD_FLOATS);
    v.gA = sg4[0]; v.gB = sg4[1]; v.gC = sg4[2];
    const float* cv = a.v_cov2d[b] + g * 3;
    v.ca = cv[0]; v.cb = cv[1]; v.cc = cv[2];
    v.ne0 = a.v_ne0[b][g];
    return v;
}

template <int DEG, bool MULTI, bool ADAM, bool PEER, bool INST = false, int Q = 1>
__device__ __forceinline__ bool bwd_tile(const BwdArgs& a, float* smem, uint8_t* s_vis, uint64_t& s_bar, uint32_t& phase,
                                         const int64_t tile) {
    // PEER with Q = 2 or 4: Q lanes per Gaussian, lane vq taking the views b with b % Q == vq, so that the round
    // trips to the other GPUs for several of a Gaussian's views are in flight together (one lane per Gaussian walks
    // them one after the other, one view ahead); a tile is then 256 / Q Gaussians, every lane accumulates its views'
    // SH-gradient row in a plane of its own (summed when the optimizer sweep reads them) and the scalar sums are
    // reduced over the Q lanes.  Lanes without a view idle through the per-view arithmetic, so Q pays only when
    // there are several views per lane to wait for.
    static_assert(Q == 1 || (PEER && (Q == 2 || Q == 4)), "several lanes per Gaussian only in the peer launch");
    constexpr int kQuad = Q;
    constexpr int kTileG = 256 / kQuad;           // Gaussians per tile
    // floats between the lanes' planes of gradient rows: 32 / Q more than the rows take, so that the lanes of a
    // Gaussian (same row, same element) and the Gaussians of a warp fall into 32 different banks
    constexpr int kPlane = kTileG * kRow + (Q > 1 ? 32 / Q : 0);
    float* s_in = smem;
    float* s_out = MULTI ? smem + kTileG * kRow : smem;
    const int t = threadIdx.x;
    const int gi = t / Q;                          // this thread's Gaussian within the tile
    const int vq = t % Q;
    const unsigned qmask = Q > 1 ? (((1u << Q) - 1u) << (t & 31 & ~(Q - 1))) : 0xffffffffu;   // lanes sharing this Gaussian
    const D3gsOpConfig& cf = a.cfg;
    constexpr int NB = (DEG + 1) * (DEG + 1);
    constexpr int NR3 = (NB - 1) * 3;
    const int64_t range_end = a.g_begin + a.g_count;
    const int64_t g0 = a.g_begin + tile * kTileG;
    const int64_t g = g0 + gi;

    // Which views see this Gaussian, as a bit mask, and its largest radius.  All the views' radii are asked for
    // before any is used: with the views on other GPUs every load is a round trip over NVLink, and eight in a row
    // would cost eight of them.  (A/B on one 8-GPU box, two runs each: this and the one-view-ahead requests below
    // against the plain walk -- radius, test, loads, arithmetic per view -- 1.56 against 1.66 ms for the launch.)
    uint32_t vis = 0;
    int radmax = 0;
    if (g < range_end) {
        if constexpr (MULTI) {
            int rad[D3GS_MAX_VIEWS];
#pragma unroll
            for (int b = 0; b < D3GS_MAX_VIEWS; ++b)
                rad[b] = (b < cf.num_views && (b & (Q - 1)) == vq) ? a.v_radii[b][g] : 0;
#pragma unroll
            for (int b = 0; b < D3GS_MAX_VIEWS; ++b) {
                vis |= rad[b] != 0 ? 1u << b : 0u;
                radmax = max(radmax, rad[b]);
            }
        } else {
            radmax = a.v_radii[0][g];
            vis = radmax != 0 ? 1u : 0u;
        }
    }
    bool any_view = vis != 0;       // Q > 1: some lane of the Gaussian has a view that sees it
    if constexpr (Q > 1) {
        any_view = __ballot_sync(0xffffffffu, any_view) & qmask;
        if (vq == 0) s_vis[gi] = any_view ? 1 : 0;
    } else {
        s_vis[t] = any_view ? 1 : 0;
    }
    const int rows = (int)min((int64_t)kTileG, range_end - g0);
    // contiguous degree-3 layout: the CTA's rows are one 16-byte aligned span -> one bulk async copy
    const bool bulk_in = NR3 > 0 && a.model.sh_rest_stride == 45 && (rows & 3) == 0 &&
                         ((uintptr_t)(a.model.sh_rest + g0 * 45) & 15) == 0;
    if (bulk_in && t == 0) {
        mbar_arrive_expect_tx(&s_bar, (uint32_t)rows * 180u);
        if ((int)blockIdx.x != a.hooks.hold)      // test hook: this CTA's copy is never issued
            bulk_copy_g2s(s_in, a.model.sh_rest + g0 * 45, (uint32_t)rows * 180u, &s_bar);
    }
    if (ADAM && t >= 32 && t < 32 + 15) {
        // The optimizer sweep at the end of the kernel reads parameters and both moments of the five small fields
        // one field after the other, a dependent DRAM round trip each: ask for these 15 spans (1-4 KB each) now,
        // so that they sit in L2 when the sweep gets there.  (Prefetching the 45-coefficient spans as well made
        // the kernel slower: 444 resident CTAs x 138 KB no longer fit beside the streaming traffic.)
        const int j = t - 32, fld = j % 5, arr = j / 5;
        const int per = fld == 1 ? 4 : fld == 3 ? 1 : 3;
        const float* base = arr == 1 ? a.exp_avg[fld] : arr == 2 ? a.exp_avg_sq[fld]
                          : fld == 0 ? a.model.xyz : fld == 1 ? a.model.quaternion_xyzw : fld == 2 ? a.model.scale
                          : fld == 3 ? a.model.opacity : a.model.sh_base;
        const float* ptr = base + g0 * per;
        const uint32_t bytes = (uint32_t)(rows * per) * 4u;
        if ((bytes & 15u) == 0 && ((uintptr_t)ptr & 15) == 0)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"(bytes) : "memory");
    }
    __syncthreads();
    bool copy_ok = true;
    if constexpr (NR3 > 0) {
        if (bulk_in) {
            copy_ok = mbar_wait_bounded(&s_bar, phase, a.hooks.poll_limit);
            phase ^= 1u;
        } else {
            const float* src = a.model.sh_rest;
            const int64_t stride = a.model.sh_rest_stride;
            constexpr int kU = NR3 % 9 == 0 ? 9 : 3;
            for (int f0 = t; f0 < kTileG * NR3; f0 += 256 * kU) {
                float tmp[kU];
                int dst[kU];
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const int f = f0 + u * 256;
                    const int row = f / NR3, k = f - row * NR3;
                    const bool ok = f < kTileG * NR3 && s_vis[row];
                    dst[u] = ok ? row * kRow + k : -1;
                    tmp[u] = ok ? src[(g0 + row) * stride + k] : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < kU; ++u)
                    if (dst[u] >= 0) s_in[dst[u]] = tmp[u];
            }
            __syncthreads();
        }
    }
    if (__syncthreads_or(!copy_ok)) {
        // The coefficient rows never arrived: flag it, give the copy one more bounded wait (the shared memory must
        // not be released while it may still land), and change nothing for this CTA's Gaussians -- no gradient is
        // written and, in the fused variants, no optimizer step is taken.
        if (!copy_ok) mbar_wait_bounded(&s_bar, phase ^ 1u, a.hooks.poll_limit);
        if (t == 0 && a.status != nullptr) atomicOr(a.status, D3GS_STATUS_COPY_TIMEOUT);
        return false;
    }
    float* my_in = s_in + gi * kRow;
    float* my_out = s_out + vq * kPlane + gi * kRow;

    float axyz[3] = {0.f, 0.f, 0.f}, aq[4] = {0.f, 0.f, 0.f, 0.f}, as[3] = {0.f, 0.f, 0.f}, ao = 0.f;
    float abase[3] = {0.f, 0.f, 0.f};
    if (MULTI || !any_view) {
#pragma unroll
        for (int k = 0; k < NR3; ++k) my_out[k] = 0.f;
    }

    if (any_view) {
        // view-independent part: activations, rotation, M = R diag(s), Sigma
        const float px = a.model.xyz[g * 3], py = a.model.xyz[g * 3 + 1], pz = a.model.xyz[g * 3 + 2];
        const float4 qr = *reinterpret_cast<const float4*>(a.model.quaternion_xyzw + g * 4);
        const bool fused = cf.fused_activations != 0;
        const float qn = fused ? sqrtf(qr.x * qr.x + qr.y * qr.y + qr.z * qr.z + qr.w * qr.w) : 1.0f;
        const float qx = qr.x / qn, qy = qr.y / qn, qz = qr.z / qn, qw = qr.w / qn;
        const float r0 = a.model.scale[g * 3], r1 = a.model.scale[g * 3 + 1], r2 = a.model.scale[g * 3 + 2];
        const float s[3] = {fused ? act_exp(r0) : r0, fused ? act_exp(r1) : r1, fused ? act_exp(r2) : r2};
        const float oraw = a.model.opacity[g];
        const float opac = fused ? 1.0f / (1.0f + act_exp(-oraw)) : oraw;
        float R[3][3];
        {
            float xx = qx * qx, yy = qy * qy, zz = qz * qz, xy = qx * qy, xz = qx * qz, yz = qy * qz;
            float wx = qw * qx, wy = qw * qy, wz = qw * qz;
            R[0][0] = 1.0f - 2.0f * (yy + zz); R[0][1] = 2.0f * (xy - wz); R[0][2] = 2.0f * (xz + wy);
            R[1][0] = 2.0f * (xy + wz); R[1][1] = 1.0f - 2.0f * (xx + zz); R[1][2] = 2.0f * (yz - wx);
            R[2][0] = 2.0f * (xz - wy); R[2][1] = 2.0f * (yz + wx); R[2][2] = 1.0f - 2.0f * (xx + yy);
        }
        float M[3][3], Sg[3][3];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int c = 0; c < 3; ++c) M[r][c] = R[r][c] * s[c];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int c = r; c < 3; ++c) Sg[r][c] = Sg[c][r] = M[r][0] * M[c][0] + M[r][1] * M[c][1] + M[r][2] * M[c][2];
        float dSacc[3][3] = {{0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}};   // sum over views of dL/dSigma
        // PEER: the densification statistics of this Gaussian over ALL views (origin/strategy.py:93-122); the owner
        // of a Gaussian sees every view's duv and radius here, so the statistics come out already summed over ranks
        float st_len = 0.f, st_cnt = 0.f, st_rad = 0.f;

        // The views that see the Gaussian, one after the other; the next view's inputs (48 bytes of raster gradient,
        // the 2D covariance, the clamp bits) are requested before the current view's arithmetic starts.
        uint32_t rem = vis;
        int b = __ffs((int)rem) - 1;
        ViewIn cur = {};
        if (Q == 1 || vis != 0) cur = load_view(a, b, g);
        while (Q == 1 || vis != 0) {
            int b_next = -1;
            ViewIn nxt = cur;
            if constexpr (MULTI) {
                rem &= rem - 1;
                if (rem != 0) {
                    b_next = __ffs((int)rem) - 1;
                    nxt = load_view(a, b_next, g);
                }
            }
            const D3gsCamera& cam = cf.cameras[b];
            const float* Rt = cam.cam2world_T;
            float Ri[12];
            if constexpr (INST) {     // instance rendering: this Gaussian's camera in its object's frame
                if (instance_camera(cf, b, g, Ri)) Rt = Ri;
            }
            const float4 gA = cur.gA, gB = cur.gB, gC = cur.gC;
            const float d0 = px - Rt[9], d1 = py - Rt[10], d2 = pz - Rt[11];
            const float pc0 = Rt[0] * d0 + Rt[1] * d1 + Rt[2] * d2;
            const float pc1 = Rt[3] * d0 + Rt[4] * d1 + Rt[5] * d2;
            const float z = Rt[6] * d0 + Rt[7] * d1 + Rt[8] * d2;
            const float tanx = 0.5f * (float)cf.width / cam.fx, tany = 0.5f * (float)cf.height / cam.fy;
            const float limx = fabsf(tanx * cf.projected_clamp_factor * z), limy = fabsf(tany * cf.projected_clamp_factor * z);
            const float tx = fminf(limx, fmaxf(-limx, pc0)), ty = fminf(limy, fmaxf(-limy, pc1));
            const float xg = (pc0 < -limx || pc0 > limx) ? 0.0f : 1.0f;
            const float yg = (pc1 < -limy || pc1 > limy) ? 0.0f : 1.0f;
            const float zi = 1.0f / z, z2i = zi * zi;
            const float J00 = cam.fx * zi, J02 = -(tx * cam.fx) * z2i, J11 = cam.fy * zi, J12 = -(ty * cam.fy) * z2i;
            float T0[3], T1[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                T0[j] = J00 * Rt[j] + J02 * Rt[6 + j];
                T1[j] = J11 * Rt[3 + j] + J12 * Rt[6 + j];
            }
            // conic -> cov2d (gs3d.py:559-588)
            const float ca = cur.ca, cb = cur.cb, cc = cur.cc;
            const float g0c = gA.x, g1c = gA.y, g2c = gA.z;
            const float det = ca * cc - cb * cb;
            const float d2i = 1.0f / (det * det + 1e-8f);
            float da = d2i * (-cc * cc * g0c + cb * cc * g1c + (det - ca * cc) * g2c);
            float db = d2i * 2.0f * (cb * cc * g0c - (0.5f * det + cb * cb) * g1c + ca * cb * g2c);
            float dc = d2i * (-ca * ca * g2c + ca * cb * g1c + (det - ca * cc) * g0c);
            float gop = gA.w;   // d loss / d (opacity the rasteriser saw)
            if (cf.anti_aliasing) {
                // render.py:3295-3309, gs3d.py:621-683: the compensation sqrt(max(2.5e-5, det0 / det)) multiplied
                // the activated opacity; its gradient reaches the covariance and scales the opacity's own
                const float lf = cf.gaussian_lowpass_filter;
                const float det0 = (ca - lf) * (cc - lf) - cb * cb;
                const float comp = det0 / det;
                const float cs = sqrtf(fmaxf(0.000025f, comp));
                const float ddet = comp <= 0.000025f ? 0.0f : (gop * opac) * 0.5f / cs;
                const float gm = ddet * d2i;
                da += lf * (cc * cc + cb * cb - cc * lf) * gm;
                db += -2.0f * cb * lf * (ca + cc - lf) * gm;
                dc += lf * (ca * ca + cb * cb - ca * lf) * gm;
                gop = gop * cs;
            }
            // cov2d = T Sigma T^T (gs3d.py:472-532): dSigma = T^T G T, dT = 2 G T Sigma
            const float hb = 0.5f * db;
            float GT0[3], GT1[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                GT0[j] = da * T0[j] + hb * T1[j];
                GT1[j] = hb * T0[j] + dc * T1[j];
            }
#pragma unroll
            for (int k = 0; k < 3; ++k)
#pragma unroll
                for (int j = 0; j < 3; ++j) dSacc[k][j] += T0[k] * GT0[j] + T1[k] * GT1[j];
            float dT0[3], dT1[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                dT0[j] = 2.0f * (GT0[0] * Sg[0][j] + GT0[1] * Sg[1][j] + GT0[2] * Sg[2][j]);
                dT1[j] = 2.0f * (GT1[0] * Sg[0][j] + GT1[1] * Sg[1][j] + GT1[2] * Sg[2][j]);
            }
            // dJ = dT W^T; only the four non-zero entries of J matter
            const float dJ00 = dT0[0] * Rt[0] + dT0[1] * Rt[1] + dT0[2] * Rt[2];
            const float dJ02 = dT0[0] * Rt[6] + dT0[1] * Rt[7] + dT0[2] * Rt[8];
            const float dJ11 = dT1[0] * Rt[3] + dT1[1] * Rt[4] + dT1[2] * Rt[5];
            const float dJ12 = dT1[0] * Rt[6] + dT1[1] * Rt[7] + dT1[2] * Rt[8];
            const float txf = tx * cam.fx, tyf = ty * cam.fy;
            const float dm0 = xg * -dJ02 * cam.fx * z2i;
            const float dm1 = yg * -dJ12 * cam.fy * z2i;
            const float dm2 = -(cam.fx * dJ00 + cam.fy * dJ11) * z2i + 2.0f * (dJ02 * txf + dJ12 * tyf) * z2i * zi;
            if (PEER && a.has_stats) {
                const float lb = (float)(a.stats.loss_batch > 0 ? a.stats.loss_batch : cf.num_views);
                const float ax = gC.x * (0.5f * (float)a.stats.width * lb), ay = gC.y * (0.5f * (float)a.stats.height * lb);
                st_len += sqrtf(ax * ax + ay * ay);
                st_cnt += 1.0f;
                st_rad = (float)radmax / (float)max(a.stats.width, a.stats.height);
            }
            // pinhole (camera.py:335-371)
            const float du = gC.x * cam.fx, dv = gC.y * cam.fy;
            const float dp0 = du * zi + dm0, dp1 = dv * zi + dm1;
            // gB.w: gradient of this splat's depth value when a depth image was rendered (zero otherwise);
            // the depth value is z, or 1/z with render_inv_depth (render.py:3053-3057)
            const float dzv = cf.inv_depth ? -gB.w * z2i : gB.w;
            const float dp2 = -(du * pc0 + dv * pc1) * z2i + dm2 + dzv;
            float dxyz[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) dxyz[j] = Rt[j] * dp0 + Rt[3 + j] * dp1 + Rt[6 + j] * dp2;
            ao += gop;
            // colour (render.py:3341-3355)
            const float dn = sqrtf(d0 * d0 + d1 * d1 + d2 * d2);
            const float dni = 1.0f / dn;
            const float x = d0 * dni, y = d1 * dni, zz_ = d2 * dni;
            float cg[3] = {gB.x, gB.y, gB.z};
            const uint32_t m = cur.ne0;
            if (cf.clamp_mask_reference_order) {   // bit k gates channel k (render.py:3344-3350)
                if (m & 1) cg[0] = 0.f;
                if (m & 2) cg[1] = 0.f;
                if (m & 4) cg[2] = 0.f;
            } else {                               // pack order r<<2 | g<<1 | b (render.py:608)
                if (m & 4) cg[0] = 0.f;
                if (m & 2) cg[1] = 0.f;
                if (m & 1) cg[2] = 0.f;
            }
            const float C0 = 0.28209479177387814f, C1 = 0.4886025119029199f;
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) abase[ch] += C0 * cg[ch];
            float ddx = 0.f, ddy = 0.f, ddz = 0.f;
            if (DEG > 0) {
                float bs[16], gx[16], gy[16], gz[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) { bs[k] = gx[k] = gy[k] = gz[k] = 0.f; }
                bs[1] = -C1 * y; bs[2] = C1 * zz_; bs[3] = -C1 * x;
                gy[1] = -C1; gz[2] = C1; gx[3] = -C1;
                if (DEG > 1) {
                    const float xx = x * x, yy = y * y, zz = zz_ * zz_, xy = x * y, yz = y * zz_, xz = x * zz_;
                    bs[4] = kC2[0] * xy; bs[5] = kC2[1] * yz; bs[6] = kC2[2] * (2.0f * zz - xx - yy);
                    bs[7] = kC2[3] * xz; bs[8] = kC2[4] * (xx - yy);
                    gx[4] = kC2[0] * y; gy[4] = kC2[0] * x;
                    gy[5] = kC2[1] * zz_; gz[5] = kC2[1] * y;
                    gx[6] = kC2[2] * -2.0f * x; gy[6] = kC2[2] * -2.0f * y; gz[6] = kC2[2] * 4.0f * zz_;
                    gx[7] = kC2[3] * zz_; gz[7] = kC2[3] * x;
                    gx[8] = kC2[4] * 2.0f * x; gy[8] = kC2[4] * -2.0f * y;
                    if (DEG > 2) {
                        bs[9] = kC3[0] * y * (3.0f * xx - yy);
                        bs[10] = kC3[1] * xy * zz_;
                        bs[11] = kC3[2] * y * (4.0f * zz - xx - yy);
                        bs[12] = kC3[3] * zz_ * (2.0f * zz - 3.0f * xx - 3.0f * yy);
                        bs[13] = kC3[4] * x * (4.0f * zz - xx - yy);
                        bs[14] = kC3[5] * zz_ * (xx - yy);
                        bs[15] = kC3[6] * x * (xx - 3.0f * yy);
                        gx[9] = kC3[0] * 6.0f * xy; gy[9] = kC3[0] * 3.0f * (xx - yy);
                        gx[10] = kC3[1] * yz; gy[10] = kC3[1] * xz; gz[10] = kC3[1] * xy;
                        gx[11] = kC3[2] * -2.0f * xy; gy[11] = kC3[2] * (-3.0f * yy + 4.0f * zz - xx); gz[11] = kC3[2] * 8.0f * yz;
                        gx[12] = kC3[3] * -6.0f * xz; gy[12] = kC3[3] * -6.0f * yz; gz[12] = kC3[3] * 3.0f * (2.0f * zz - xx - yy);
                        gx[13] = kC3[4] * (-3.0f * xx + 4.0f * zz - yy); gy[13] = kC3[4] * -2.0f * xy; gz[13] = kC3[4] * 8.0f * xz;
                        gx[14] = kC3[5] * 2.0f * xz; gy[14] = kC3[5] * -2.0f * yz; gz[14] = kC3[5] * (xx - yy);
                        gx[15] = kC3[6] * 3.0f * (xx - yy); gy[15] = kC3[6] * -6.0f * xy;
                    }
                }
#pragma unroll
                for (int k = 1; k < NB; ++k) {
#pragma unroll
                    for (int ch = 0; ch < 3; ++ch) {
                        const int e = (k - 1) * 3 + ch;
                        const float coef = my_in[e] * cg[ch];
                        ddx += gx[k] * coef; ddy += gy[k] * coef; ddz += gz[k] * coef;
                        if (MULTI) my_out[e] += bs[k] * cg[ch];
                        else my_out[e] = bs[k] * cg[ch];   // in place: the coefficient was just consumed
                    }
                }
            }
            // normalize_grad (render.py:3354)
            const float dd = x * ddx + y * ddy + zz_ * ddz;
            axyz[0] += dxyz[0] + (ddx - x * dd) * dni;
            axyz[1] += dxyz[1] + (ddy - y * dd) * dni;
            axyz[2] += dxyz[2] + (ddz - zz_ * dd) * dni;
            if (b_next < 0) break;
            cur = nxt;
            b = b_next;
        }
        if constexpr (Q > 1) {     // the lanes' sums for this Gaussian
#pragma unroll
            for (int o = 1; o < Q; o <<= 1) {
#pragma unroll
                for (int r = 0; r < 3; ++r) {
#pragma unroll
                    for (int c = 0; c < 3; ++c) dSacc[r][c] += __shfl_xor_sync(qmask, dSacc[r][c], o);
                    axyz[r] += __shfl_xor_sync(qmask, axyz[r], o);
                    abase[r] += __shfl_xor_sync(qmask, abase[r], o);
                }
                ao += __shfl_xor_sync(qmask, ao, o);
                st_len += __shfl_xor_sync(qmask, st_len, o);
                st_cnt += __shfl_xor_sync(qmask, st_cnt, o);
                st_rad = fmaxf(st_rad, __shfl_xor_sync(qmask, st_rad, o));
            }
        }
        // Sigma = M M^T (gs3d.py:387-418): dM = 2 dSigma M (dSigma symmetric), ds_j = <dM[:,j], R[:,j]>
        float dM[3][3];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int c = 0; c < 3; ++c)
                dM[r][c] = 2.0f * (dSacc[r][0] * M[0][c] + dSacc[r][1] * M[1][c] + dSacc[r][2] * M[2][c]);
        float dR[3][3];
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            const float ds = dM[0][c] * R[0][c] + dM[1][c] * R[1][c] + dM[2][c] * R[2][c];
            as[c] = fused ? ds * s[c] : ds;          // exponential_grad_out: g * out
#pragma unroll
            for (int r = 0; r < 3; ++r) dR[r][c] = dM[r][c] * s[c];
        }
        float dq[4];
        dq[0] = 2.0f * (qy * (dR[0][1] + dR[1][0]) + qz * (dR[0][2] + dR[2][0]) + qw * (dR[2][1] - dR[1][2]) - 2.0f * qx * (dR[1][1] + dR[2][2]));
        dq[1] = 2.0f * (qx * (dR[0][1] + dR[1][0]) + qz * (dR[1][2] + dR[2][1]) + qw * (dR[0][2] - dR[2][0]) - 2.0f * qy * (dR[0][0] + dR[2][2]));
        dq[2] = 2.0f * (qx * (dR[0][2] + dR[2][0]) + qy * (dR[1][2] + dR[2][1]) + qw * (dR[1][0] - dR[0][1]) - 2.0f * qz * (dR[0][0] + dR[1][1]));
        dq[3] = 2.0f * (qx * (dR[2][1] - dR[1][2]) + qy * (dR[0][2] - dR[2][0]) + qz * (dR[1][0] - dR[0][1]));
        const float dot = fused ? qx * dq[0] + qy * dq[1] + qz * dq[2] + qw * dq[3] : 0.0f;
        const float qni = 1.0f / qn;                 // normalize_grad_out: (g - n <n,g>) / |raw|
        aq[0] = (dq[0] - qx * dot) * qni; aq[1] = (dq[1] - qy * dot) * qni;
        aq[2] = (dq[2] - qz * dot) * qni; aq[3] = (dq[3] - qw * dot) * qni;
        if (fused) ao = ao * opac * (1.0f - opac);   // sigmoid_grad_out: g * out * (1 - out)
        if (PEER && a.has_stats && vq == 0) {
            a.stats.duv_ndc_length[g] += st_len;
            a.stats.count[g] += st_cnt;
            if (a.stats.need_max_radii) a.stats.max_radii[g] = fmaxf(a.stats.max_radii[g], st_rad);
        }
    }
    if (ADAM) {
        // The 14 small-field gradients of every thread join the SH rows in shared memory, then the CTA walks
        // the six parameter spans of its 256 Gaussians with coalesced float4 accesses (several in flight per
        // thread), exactly like the stand-alone optimizer kernel but with the gradient coming from shared
        // memory.  The parameters are updated in place: a CTA reads and writes only its own Gaussians'.
        if (!PEER && a.has_stats && g < range_end) stats_update(a.stats, g);
        // per tile of T Gaussians: [xyz 3T | quaternion 4T | scale 3T | opacity T | sh_base 3T], behind the SH rows
        // (PEER: behind the coefficient rows and the four gradient planes)
        float* s_small = smem + kTileG * kRow + (MULTI ? kQuad * kPlane : 0);
        if (vq == 0) {
            s_small[gi * 3] = axyz[0]; s_small[gi * 3 + 1] = axyz[1]; s_small[gi * 3 + 2] = axyz[2];
            *reinterpret_cast<float4*>(s_small + 3 * kTileG + gi * 4) = make_float4(aq[0], aq[1], aq[2], aq[3]);
            s_small[7 * kTileG + gi * 3] = as[0]; s_small[7 * kTileG + gi * 3 + 1] = as[1]; s_small[7 * kTileG + gi * 3 + 2] = as[2];
            s_small[10 * kTileG + gi] = ao;
            s_small[11 * kTileG + gi * 3] = abase[0]; s_small[11 * kTileG + gi * 3 + 1] = abase[1];
            s_small[11 * kTileG + gi * 3 + 2] = abase[2];
        }
        __syncthreads();
        const float* params[6] = {a.model.xyz, a.model.quaternion_xyzw, a.model.scale, a.model.opacity,
                                  a.model.sh_base, a.model.sh_rest};
        const int per[6] = {3, 4, 3, 1, 3, 45};
        const int soff[6] = {0, 3 * kTileG, 7 * kTileG, 10 * kTileG, 11 * kTileG, -1};
#pragma unroll
        for (int fld = 0; fld < 6; ++fld) {
            const int count = rows * per[fld];
            float* pp = const_cast<float*>(params[fld]) + g0 * per[fld];
            float* pm = a.exp_avg[fld] + g0 * per[fld];
            float* pv = a.exp_avg_sq[fld] + g0 * per[fld];
            const float* gs = fld == 5 ? s_out : s_small + soff[fld];
            const SegConst c = a.sc[fld];
            const bool vec = (count & 3) == 0 && (((uintptr_t)pp | (uintptr_t)pm | (uintptr_t)pv) & 15) == 0;
            if (vec) {
                constexpr int kU = 4;
                for (int q0 = t; q0 < count / 4; q0 += 256 * kU) {
                    float4 p[kU], m[kU], v[kU];
#pragma unroll
                    for (int u = 0; u < kU; ++u) {
                        const int q = q0 + u * 256;
                        if (q < count / 4) {
                            p[u] = reinterpret_cast<const float4*>(pp)[q];
                            m[u] = reinterpret_cast<const float4*>(pm)[q];
                            v[u] = reinterpret_cast<const float4*>(pv)[q];
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kU; ++u) {
                        const int q = q0 + u * 256;
                        if (q < count / 4) {
                            float4 gr = reinterpret_cast<const float4*>(gs)[q];
                            if (Q > 1 && fld == 5) {     // the lanes' planes of SH-gradient rows
#pragma unroll
                                for (int pl = 1; pl < kQuad; ++pl) {
                                    const float4 o4 = reinterpret_cast<const float4*>(gs + pl * kPlane)[q];
                                    gr.x += o4.x; gr.y += o4.y; gr.z += o4.z; gr.w += o4.w;
                                }
                            }
                            if (fld == 5 && NR3 < 45) {   // coefficients above the active degree have no gradient
                                const int k0 = (q * 4) % 45;
                                if (k0 >= NR3) gr.x = 0.0f;
                                if ((k0 + 1) % 45 >= NR3) gr.y = 0.0f;
                                if ((k0 + 2) % 45 >= NR3) gr.z = 0.0f;
                                if ((k0 + 3) % 45 >= NR3) gr.w = 0.0f;
                            }
                            adam_update(gr.x, p[u].x, m[u].x, v[u].x, c);
                            adam_update(gr.y, p[u].y, m[u].y, v[u].y, c);
                            adam_update(gr.z, p[u].z, m[u].z, v[u].z, c);
                            adam_update(gr.w, p[u].w, m[u].w, v[u].w, c);
                            if (PEER) {   // every replica receives the new value (this rank's own through its own mapping)
                                const int64_t fo = a.field_off[fld] + g0 * per[fld];
                                for (int r = 0; r < a.peers.world; ++r)
                                    reinterpret_cast<float4*>(a.peers.param[r] + fo)[q] = p[u];
                            } else {
                                reinterpret_cast<float4*>(pp)[q] = p[u];
                            }
                            reinterpret_cast<float4*>(pm)[q] = m[u];
                            reinterpret_cast<float4*>(pv)[q] = v[u];
                        }
                    }
                }
            } else {
                for (int f = t; f < count; f += 256) {
                    float gr = gs[f];
                    if (Q > 1 && fld == 5) {
#pragma unroll
                        for (int pl = 1; pl < kQuad; ++pl) gr += gs[pl * kPlane + f];
                    }
                    if (fld == 5 && NR3 < 45 && f % 45 >= NR3) gr = 0.0f;
                    float p = pp[f], m = pm[f], v = pv[f];
                    adam_update(gr, p, m, v, c);
                    if (PEER) {
                        const int64_t fo = a.field_off[fld] + g0 * per[fld];
                        for (int r = 0; r < a.peers.world; ++r) a.peers.param[r][fo + f] = p;
                    } else {
                        pp[f] = p;
                    }
                    pm[f] = m; pv[f] = v;
                }
            }
        }
        return true;
    }
    if (g < range_end) {
        a.grad.xyz[g * 3] = axyz[0]; a.grad.xyz[g * 3 + 1] = axyz[1]; a.grad.xyz[g * 3 + 2] = axyz[2];
        *reinterpret_cast<float4*>(a.grad.quaternion_xyzw + g * 4) = make_float4(aq[0], aq[1], aq[2], aq[3]);
        a.grad.scale[g * 3] = as[0]; a.grad.scale[g * 3 + 1] = as[1]; a.grad.scale[g * 3 + 2] = as[2];
        a.grad.opacity[g] = ao;
        float* gb = a.grad.sh_base + g * a.grad.sh_base_stride;
        gb[0] = abase[0]; gb[1] = abase[1]; gb[2] = abase[2];
    }
    if (a.grad.sh_rest != nullptr) {
        // rows leave shared memory as one bulk async store when the destination span is contiguous and
        // aligned, else with coalesced per-element stores; coefficients above the active degree are zero
        const int rf = a.grad.sh_rest_floats;
        const int64_t stride = a.grad.sh_rest_stride;
        const bool bulk_out = rf == 45 && stride == 45 && (rows & 3) == 0 &&
                              ((uintptr_t)(a.grad.sh_rest + g0 * 45) & 15) == 0;
        if (bulk_out) {
#pragma unroll
            for (int k = NR3; k < 45; ++k) my_out[k] = 0.0f;
            fence_proxy_async_smem();   // generic-proxy writes to shared memory -> visible to the copy engine
            __syncthreads();
            if (t == 0) {
                bulk_copy_s2g(a.grad.sh_rest + g0 * 45, s_out, (uint32_t)rows * 180u);
                bulk_commit_group();
                bulk_wait_group_read0();
            }
        } else {
            __syncthreads();
            for (int f = t; f < rows * rf; f += 256) {
                const int row = f / rf, k = f - row * rf;
                a.grad.sh_rest[(g0 + row) * stride + k] = k < NR3 ? s_out[row * kRow + k] : 0.0f;
            }
        }
    }
    return true;
}

// PEER (data parallel, one view per rank; implies MULTI and ADAM): the launch covers this rank's share of the
// Gaussians.  For them it reads EVERY rank's per-splat raster gradients and context over NVLink, runs the
// backward through projection and SH for all views, sums in registers, applies Adam with this rank's moments and
// stores the new parameters into EVERY rank's parameter buffer.  The 236-byte-per-Gaussian parameter gradient
// never exists: what crosses the links is the rasteriser's 48 bytes per (view, Gaussian) plus 17 bytes of
// context inbound, and the parameters outbound.  The launches of the ranks are ordered by flags (exchange.cuh).
template <int DEG, bool MULTI, bool ADAM, bool PEER = false, bool INST = false, int Q = 1>
__global__ void __launch_bounds__(256, PEER ? 2 : 3) preprocess_bwd_kernel(const __grid_constant__ BwdArgs a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ uint8_t s_vis[256];
    __shared__ __align__(8) uint64_t s_bar;
    if (threadIdx.x == 0) {
        mbar_init(&s_bar, 1);
        fence_mbar_init();
    }
    uint32_t phase = 0;
    if constexpr (PEER) {
        // a resident grid that strides over the tiles: the flag exchange and the system-wide fence at the end are
        // paid once per CTA
        const bool ready = exchange_begin(a.peers);   // every rank's raster gradients are complete (contains a barrier)
        constexpr int kTileG = 256 / Q;
        const int64_t num_tiles = (a.g_count + kTileG - 1) / kTileG;
        if (ready) {      // else a rank never announced its gradients: change nothing
            for (int64_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
                if (!bwd_tile<DEG, MULTI, ADAM, PEER, INST, Q>(a, smem, s_vis, s_bar, phase, tile)) break;
                __syncthreads();      // the next tile reuses the shared memory
            }
        }
        exchange_end(a.peers);        // all parameters of every rank's share have arrived when the kernel ends
    } else {
        __syncthreads();
        bwd_tile<DEG, MULTI, ADAM, PEER, INST>(a, smem, s_vis, s_bar, phase, blockIdx.x);
    }
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

// one process, B views: view b's arrays are slices of the [B*N, .] context
static void fill_views(BwdArgs& a, const D3gsOpConfig* cfg, const D3gsModel* model, const D3gsSplatContext* ctx,
                       const float* splat_grads) {
    const int64_t N = model->num;
    for (int b = 0; b < cfg->num_views; ++b) {
        a.v_grads[b] = splat_grads + (int64_t)b * N * D3GS_SPLAT_GRAD_FLOATS;
        a.v_radii[b] = ctx->radii + (int64_t)b * N;
        a.v_cov2d[b] = ctx->cov2d_vecs + (int64_t)b * N * 3;
        a.v_ne0[b] = ctx->sh_to_rgb_ne_0 + (int64_t)b * N;
    }
    a.g_begin = 0;
    a.g_count = N;
}

static int32_t check_backward_inputs(const D3gsOpConfig* cfg, const D3gsModel* model, const D3gsSplatContext* ctx,
                                     const float* splat_grads) {
    D3GS_REQUIRE(cfg && model && ctx, "NULL argument");
    D3GS_REQUIRE(cfg->num_views >= 1 && cfg->num_views <= D3GS_MAX_VIEWS, "num_views %d outside [1,%d]", cfg->num_views,
                 D3GS_MAX_VIEWS);
    D3GS_REQUIRE(cfg->sh_degree >= 0 && cfg->sh_degree <= 3, "sh_degree %d outside [0,3]", cfg->sh_degree);
    D3GS_REQUIRE(splat_grads != nullptr && ((uintptr_t)splat_grads & 15) == 0, "splat_grads NULL or not 16-byte aligned");
    D3GS_REQUIRE(ctx->radii && ctx->cov2d_vecs && ctx->sh_to_rgb_ne_0, "context lacks radii/cov2d_vecs/sh_to_rgb_ne_0");
    D3GS_REQUIRE(((uintptr_t)model->quaternion_xyzw & 15) == 0, "quaternion tensors must be 16-byte aligned");
    return D3GS_OK;
}

extern "C" int32_t d3gs_preprocess_backward(const D3gsOpConfig* cfg, const D3gsModel* model,
                                            const D3gsSplatContext* ctx, const float* splat_grads,
                                            const D3gsModelGrad* grad, uint32_t* status, void* stream) {
    D3GS_REQUIRE(grad != nullptr, "NULL argument");
    int32_t rc = check_backward_inputs(cfg, model, ctx, splat_grads);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(grad->xyz && grad->quaternion_xyzw && grad->scale && grad->opacity && grad->sh_base,
                 "NULL gradient output");
    D3GS_REQUIRE(cfg->sh_degree == 0 || (grad->sh_rest && model->sh_rest), "sh_rest needed with sh_degree > 0");
    D3GS_REQUIRE(((uintptr_t)grad->quaternion_xyzw & 15) == 0, "quaternion tensors must be 16-byte aligned");
    D3GS_REQUIRE(grad->sh_rest == nullptr ||
                     (grad->sh_rest_floats >= ((cfg->sh_degree + 1) * (cfg->sh_degree + 1) - 1) * 3 &&
                      grad->sh_rest_floats <= grad->sh_rest_stride && grad->sh_rest_floats <= 45),
                 "sh_rest gradient: floats per Gaussian (%d) must cover the active degree and fit the stride (%d)",
                 grad->sh_rest_floats, grad->sh_rest_stride);
    if (model->num == 0) return D3GS_OK;
    BwdArgs a = {};
    a.cfg = *cfg;
    a.model = *model;
    a.grad = *grad;
    a.status = status;
    a.hooks = test_hooks();
    fill_views(a, cfg, model, ctx, splat_grads);
    dim3 grid((unsigned)div_up64(model->num, 256));
    cudaStream_t s = (cudaStream_t)stream;
    const bool multi = cfg->num_views > 1;
    const size_t smem = (size_t)256 * kRow * sizeof(float) * (multi ? 2 : 1);
#define D3GS_LAUNCH_BWD(DEG, MULTI)                                                                              \
    do {                                                                                                         \
        if (cfg->instance_id != nullptr) {                                                                       \
            D3GS_CUDA(cudaFuncSetAttribute(preprocess_bwd_kernel<DEG, MULTI, false, false, true>,                \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));             \
            preprocess_bwd_kernel<DEG, MULTI, false, false, true><<<grid, 256, smem, s>>>(a);                    \
        } else {                                                                                                 \
            D3GS_CUDA(cudaFuncSetAttribute(preprocess_bwd_kernel<DEG, MULTI, false>,                             \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));             \
            preprocess_bwd_kernel<DEG, MULTI, false><<<grid, 256, smem, s>>>(a);                                 \
        }                                                                                                        \
    } while (0)
    switch (cfg->sh_degree * 2 + (multi ? 1 : 0)) {
        case 0: D3GS_LAUNCH_BWD(0, false); break;
        case 1: D3GS_LAUNCH_BWD(0, true); break;
        case 2: D3GS_LAUNCH_BWD(1, false); break;
        case 3: D3GS_LAUNCH_BWD(1, true); break;
        case 4: D3GS_LAUNCH_BWD(2, false); break;
        case 5: D3GS_LAUNCH_BWD(2, true); break;
        case 6: D3GS_LAUNCH_BWD(3, false); break;
        default: D3GS_LAUNCH_BWD(3, true); break;
    }
#undef D3GS_LAUNCH_BWD
    D3GS_LAUNCH_CHECK("preprocess_bwd_kernel");
    return D3GS_OK;
}

// the six optimizer segments of a fused backward: xyz, quaternion, scale, opacity, sh_base, sh_rest over
// `count` Gaussians starting at Gaussian `begin` of the model
static int32_t fill_segments(BwdArgs& a, const D3gsModel* model, const D3gsAdamSegment* segments, int64_t begin,
                             int64_t count, bool params_are_slices) {
    const float* params[6] = {model->xyz, model->quaternion_xyzw, model->scale, model->opacity, model->sh_base,
                              model->sh_rest};
    const int64_t per[6] = {3, 4, 3, 1, 3, 45};
    for (int k = 0; k < 6; ++k) {
        const D3gsAdamSegment& sg = segments[k];
        D3GS_REQUIRE(sg.param == params[k] + (params_are_slices ? begin * per[k] : 0),
                     "segment %d does not point at the model's tensor", k);
        D3GS_REQUIRE(sg.count == per[k] * count, "segment %d: %lld elements, expected %lld", k, (long long)sg.count,
                     (long long)(per[k] * count));
        D3GS_REQUIRE(sg.exp_avg && sg.exp_avg_sq, "segment %d: NULL moment tensor", k);
        D3GS_REQUIRE(sg.grad_scale != 0.0f && sg.bias_correction1 != 0.0f && sg.bias_correction2_sqrt != 0.0f,
                     "segment %d: zero grad_scale / bias correction", k);
        a.sc[k] = make_seg_const(sg);
        // the kernel indexes the moments by the Gaussian's index in the whole model
        a.exp_avg[k] = sg.exp_avg - begin * per[k];
        a.exp_avg_sq[k] = sg.exp_avg_sq - begin * per[k];
    }
    return D3GS_OK;
}

extern "C" int32_t d3gs_preprocess_backward_adam(const D3gsOpConfig* cfg, const D3gsModel* model,
                                                 const D3gsSplatContext* ctx, const float* splat_grads,
                                                 const D3gsAdamSegment* segments, const D3gsDensifyStats* stats,
                                                 uint32_t* status, void* stream) {
    int32_t rc = check_backward_inputs(cfg, model, ctx, splat_grads);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(segments != nullptr, "segments is NULL");
    D3GS_REQUIRE(cfg->instance_id == nullptr, "instance rendering: use d3gs_preprocess_backward and d3gs_adam_step");
    D3GS_REQUIRE(cfg->num_views == 1, "the fused backward + Adam handles one view per launch (got %d)", cfg->num_views);
    D3GS_REQUIRE(model->sh_rest != nullptr && model->sh_rest_stride == 45 && model->sh_base_stride == 3,
                 "the fused backward + Adam needs the split degree-3 SH layout (strides 3 and 45)");
    BwdArgs a = {};
    rc = fill_segments(a, model, segments, 0, model->num, false);
    if (rc != D3GS_OK) return rc;
    if (stats != nullptr) {
        D3GS_REQUIRE(stats->num == model->num && stats->batch == 1, "statistics shape does not match the model / one view");
        D3GS_REQUIRE(stats->duv && stats->radii && stats->duv_ndc_length && stats->count, "NULL stats tensor");
        D3GS_REQUIRE(!stats->need_max_radii || stats->max_radii, "max_radii is NULL");
        D3GS_REQUIRE(((uintptr_t)stats->duv & 7) == 0 && (stats->duv_stride & 1) == 0,
                     "duv must be 8-byte aligned, stride even");
        a.has_stats = 1;
        a.stats = *stats;
    }
    if (model->num == 0) return D3GS_OK;
    a.cfg = *cfg;
    a.model = *model;
    a.status = status;
    a.hooks = test_hooks();
    fill_views(a, cfg, model, ctx, splat_grads);
    dim3 grid((unsigned)div_up64(model->num, 256));
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)256 * (kRow + 14) * sizeof(float);   // SH rows + the 14 small-field gradients
#define D3GS_LAUNCH_BWD_ADAM(DEG)                                                                               \
    do {                                                                                                        \
        D3GS_CUDA(cudaFuncSetAttribute(preprocess_bwd_kernel<DEG, false, true>,                                 \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                \
        preprocess_bwd_kernel<DEG, false, true><<<grid, 256, smem, s>>>(a);                                     \
    } while (0)
    switch (cfg->sh_degree) {
        case 0: D3GS_LAUNCH_BWD_ADAM(0); break;
        case 1: D3GS_LAUNCH_BWD_ADAM(1); break;
        case 2: D3GS_LAUNCH_BWD_ADAM(2); break;
        default: D3GS_LAUNCH_BWD_ADAM(3); break;
    }
#undef D3GS_LAUNCH_BWD_ADAM
    D3GS_LAUNCH_CHECK("preprocess_bwd_kernel<adam>");
    return D3GS_OK;
}

extern "C" int32_t d3gs_preprocess_backward_adam_peers(const D3gsOpConfig* cfg, const D3gsModel* model,
                                                       const D3gsPeerViews* views, int64_t g_begin, int64_t g_count,
                                                       const D3gsAdamSegment* segments, const D3gsDensifyStats* stats,
                                                       const D3gsPeerSet* peers, void* stream) {
    D3GS_REQUIRE(cfg && model && views && segments && peers, "NULL argument");
    D3GS_REQUIRE(peers->world >= 1 && peers->world <= D3GS_MAX_PEERS && peers->rank >= 0 && peers->rank < peers->world,
                 "bad world / rank");
    D3GS_REQUIRE(cfg->num_views == peers->world, "one view per rank: num_views %d, world %d", cfg->num_views, peers->world);
    D3GS_REQUIRE(cfg->instance_id == nullptr, "instance rendering: use d3gs_preprocess_backward and d3gs_adam_step");
    D3GS_REQUIRE(cfg->sh_degree >= 0 && cfg->sh_degree <= 3, "sh_degree %d outside [0,3]", cfg->sh_degree);
    D3GS_REQUIRE(model->sh_rest != nullptr && model->sh_rest_stride == 45 && model->sh_base_stride == 3,
                 "the fused backward + Adam needs the split degree-3 SH layout (strides 3 and 45)");
    D3GS_REQUIRE(g_begin >= 0 && g_count >= 0 && g_begin + g_count <= model->num, "Gaussian range [%lld, +%lld) outside the model",
                 (long long)g_begin, (long long)g_count);
    D3GS_REQUIRE((g_begin & 3) == 0, "the range must start at a multiple of four Gaussians (16-byte aligned spans)");
    D3GS_REQUIRE(((uintptr_t)model->quaternion_xyzw & 15) == 0, "quaternion tensors must be 16-byte aligned");
    const bool with_flags = peers->flags[0] != nullptr;
    D3GS_REQUIRE(!with_flags || peers->epoch != 0, "epoch must be positive when flag blocks are given");
    BwdArgs a = {};
    const float* params[6] = {model->xyz, model->quaternion_xyzw, model->scale, model->opacity, model->sh_base,
                              model->sh_rest};
    for (int b = 0; b < peers->world; ++b) {
        D3GS_REQUIRE(views->splat_grads[b] && views->radii[b] && views->cov2d_vecs[b] && views->sh_to_rgb_ne_0[b],
                     "view %d: NULL buffer", b);
        D3GS_REQUIRE(((uintptr_t)views->splat_grads[b] & 15) == 0, "view %d: splat_grads not 16-byte aligned", b);
        D3GS_REQUIRE(peers->param[b] != nullptr, "rank %d: NULL parameter buffer", b);
        D3GS_REQUIRE((peers->flags[b] != nullptr) == with_flags, "flag blocks must be given for all ranks or none");
        a.v_grads[b] = views->splat_grads[b];
        a.v_radii[b] = views->radii[b];
        a.v_cov2d[b] = views->cov2d_vecs[b];
        a.v_ne0[b] = views->sh_to_rgb_ne_0[b];
    }
    for (int k = 0; k < 6; ++k) {
        a.field_off[k] = params[k] - peers->param[peers->rank];
        D3GS_REQUIRE(a.field_off[k] >= 0 && (a.field_off[k] & 3) == 0,
                     "field %d does not lie 16-byte aligned inside this rank's flat parameter buffer", k);
    }
    int32_t rc = fill_segments(a, model, segments, g_begin, g_count, true);
    if (rc != D3GS_OK) return rc;
    if (stats != nullptr) {
        D3GS_REQUIRE(stats->num == model->num, "statistics shape does not match the model");
        D3GS_REQUIRE(stats->duv_ndc_length && stats->count && stats->width > 0 && stats->height > 0, "bad stats struct");
        D3GS_REQUIRE(!stats->need_max_radii || stats->max_radii, "max_radii is NULL");
        a.has_stats = 1;
        a.stats = *stats;
    }
    a.cfg = *cfg;
    a.model = *model;
    a.peers = *peers;
    for (int q = peers->world; q < D3GS_MAX_PEERS; ++q) a.peers.flags[q] = nullptr;
    a.status = peers->status;
    a.hooks = test_hooks();
    a.g_begin = g_begin;
    a.g_count = g_count;
    // lanes per Gaussian: 0 = chosen here from the number of views a lane would have to wait for
    int lanes = peers->lanes_per_gaussian;
    D3GS_REQUIRE(lanes == 0 || lanes == 1 || lanes == 2 || lanes == 4, "lanes_per_gaussian must be 0, 1, 2 or 4 (got %d)", lanes);
    // measured (cfg3, one box each): 8 ranks 3.61 / 3.47 / 3.45 ms per step with 1 / 2 / 4 lanes, 4 ranks 3.22 / 3.18 / 3.24,
    // 2 ranks 3.06 / - / 4.12
    if (lanes == 0) lanes = peers->world >= 8 ? 4 : (peers->world >= 4 ? 2 : 1);
    const int tile_g = 256 / lanes;
    const int64_t tiles = div_up64(g_count, tile_g);
    // every rank launches, even with an empty share: the flag exchange needs all ranks
    int dev = 0, sms = 0;
    D3GS_CUDA(cudaGetDevice(&dev));
    D3GS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int64_t grid = tiles < (int64_t)sms * 2 ? tiles : (int64_t)sms * 2;
    if (grid < 1) grid = 1;
    cudaStream_t s = (cudaStream_t)stream;
    // SH rows in, one (padded) plane of gradient rows per lane of a Gaussian, small fields
    const size_t smem = (size_t)(tile_g * kRow + lanes * (tile_g * kRow + (lanes > 1 ? 32 / lanes : 0)) + tile_g * 14) *
                        sizeof(float);
#define D3GS_LAUNCH_BWD_PEER_Q(DEG, QQ)                                                                         \
    do {                                                                                                        \
        D3GS_CUDA(cudaFuncSetAttribute(preprocess_bwd_kernel<DEG, true, true, true, false, QQ>,                 \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                \
        preprocess_bwd_kernel<DEG, true, true, true, false, QQ><<<(unsigned)grid, 256, smem, s>>>(a);           \
    } while (0)
#define D3GS_LAUNCH_BWD_PEER(DEG)                                                                               \
    do {                                                                                                        \
        if (lanes == 4) D3GS_LAUNCH_BWD_PEER_Q(DEG, 4);                                                         \
        else if (lanes == 2) D3GS_LAUNCH_BWD_PEER_Q(DEG, 2);                                                    \
        else D3GS_LAUNCH_BWD_PEER_Q(DEG, 1);                                                                    \
    } while (0)
    switch (cfg->sh_degree) {
        case 0: D3GS_LAUNCH_BWD_PEER(0); break;
        case 1: D3GS_LAUNCH_BWD_PEER(1); break;
        case 2: D3GS_LAUNCH_BWD_PEER(2); break;
        default: D3GS_LAUNCH_BWD_PEER(3); break;
    }
#undef D3GS_LAUNCH_BWD_PEER
#undef D3GS_LAUNCH_BWD_PEER_Q
    D3GS_LAUNCH_CHECK("preprocess_bwd_kernel<peers>");
    return D3GS_OK;
}
