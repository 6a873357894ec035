// K9/K10: SSIM map forward/backward and the fused L1 + D-SSIM loss gradient.
//
// Reference semantics: d3sim/ops/image/fused_ssim.py:93-377 (11x11 Gaussian window sigma 1.5 =
// outer product of the normalised 1-D window (32-40), zero padding (175-178), C1=1e-4, C2=9e-4,
// saved partials dmu1/dmu11/dmu12 (226-231), backward = three convolutions (341-361)), and
// d3sim/algos/d3gs/train.py:169-172 / losses.py:19-20 for the loss combination.
//
// The reference applies the window as 121 taps per output; here it is applied separably (11
// horizontal + 11 vertical taps) from shared memory, four outputs per thread along the filter direction.  In the fused entry point the rasteriser's
// NHWC colour is read directly and dL/dcolor is written NHWC, so the reference's
// permute(0,3,1,2).contiguous() round trip (train.py:169) and its autograd mirror disappear.
#include <cmath>

#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kWin = 11, kPad = 5;
constexpr int kTX = 32, kTY = 16;                       // output pixels per CTA
constexpr int kHX = kTX + 2 * kPad, kHY = kTY + 2 * kPad;   // 42 x 26 input halo
constexpr int kSX = 48;                                 // halo row stride: rows start on 16-byte boundaries
constexpr int kStrip = 4;                               // outputs per thread along the filter direction
constexpr int kTaps = kStrip + kWin - 1;                // 14 inputs feed 4 outputs
constexpr int kThreads = 128;                           // = columns x strips of the vertical pass: no idle warps there

struct Window {
    float g[kWin];
};

Window make_window() {
    // gaussian(11, 1.5) normalised, as float32 like torch.Tensor (fused_ssim.py:32-34)
    Window w;
    float tmp[kWin], s = 0.0f;
    for (int i = 0; i < kWin; ++i) {
        tmp[i] = (float)std::exp(-(double)((i - kPad) * (i - kPad)) / (2.0 * 1.5 * 1.5));
        s += tmp[i];
    }
    for (int i = 0; i < kWin; ++i) w.g[i] = tmp[i] / s;
    return w;
}

struct SsimArgs {
    const float* x;       // prediction, NHWC or NCHW
    const float* y;       // target, NCHW
    int batch, height, width;
    int x_is_nhwc;
    Window win;
    // forward outputs (NCHW, may be NULL)
    float* ssim_map;
    float* dmu1;
    float* dmu11;
    float* dmu12;
    double* sums;         // fused: [sum |x-y|, sum ssim]
    // backward
    const float* dssim;   // NCHW or NULL (fused: constant gs)
    float* dx;
    float gs, gl;         // fused: dloss/dssim per element, dloss/d|x-y| per element (both incl. grad_scale)
};

// Both kernels filter separably out of shared memory with register blocking: a thread produces kStrip
// consecutive outputs along the filter direction from kTaps inputs it loads once (as float4 in the
// horizontal pass), so a tap costs one FMA and 1/4 of a shared-memory load instead of one load per FMA.

// Starts the asynchronous load of the 42x26 halo of all three channels of an image into s[3][kHY][kSX]
// (zero outside the image, fused_ssim.py:175-178); the caller waits with cp_async_wait_all + __syncthreads.
// NHWC rows are read as runs of 126 consecutive floats.  cp.async keeps every element's load in flight at
// once; a register-staged loop had one load per thread in flight and was bound by DRAM latency.
__device__ __forceinline__ void load_halo(float (*s)[kHY][kSX], const float* img, bool nhwc, int b, int by, int bx,
                                          int height, int width, int t) {
    // Every thread keeps one fixed column (and channel / row-in-group) and walks down the rows, so that the
    // per-element work is an add and a compare instead of index divisions.
    static_assert(kThreads >= kHX * 3, "one thread per element of a 42-pixel, 3-channel row");
    if (nhwc) {
        if (t < kHX * 3) {   // thread = one float of the 126-float row
            const int lx = t / 3, c = t - lx * 3, gx = bx + lx - kPad;
            const bool col_ok = gx >= 0 && gx < width;
            const float* src = img + (((int64_t)b * height + (by - kPad)) * width + gx) * 3 + c;
            float* dst = &s[c][0][lx];
            for (int ly = 0; ly < kHY; ++ly) {
                const int gy = by + ly - kPad;
                const bool ok = col_ok && gy >= 0 && gy < height;
                cp_async4(dst, ok ? src : img, ok);
                src += (int64_t)width * 3;
                dst += kSX;
            }
        }
    } else {
        if (t < kHX * 3) {   // thread = one column of one of three consecutive rows
            const int r3 = t / kHX, lx = t - r3 * kHX, gx = bx + lx - kPad;
            const bool col_ok = gx >= 0 && gx < width;
            for (int c = 0; c < 3; ++c) {
                const float* plane0 = img + ((int64_t)b * 3 + c) * height * width;
                for (int ly = r3; ly < kHY; ly += 3) {
                    const int gy = by + ly - kPad;
                    const bool ok = col_ok && gy >= 0 && gy < height;
                    cp_async4(&s[c][ly][lx], ok ? plane0 + (int64_t)gy * width + gx : img, ok);
                }
            }
        }
    }
    for (int k = t; k < 3 * kHY * (kSX - kHX); k += kThreads) {   // the float4 loads touch the row padding
        const int c = k / (kHY * (kSX - kHX)), r = k - c * (kHY * (kSX - kHX)), ly = r / (kSX - kHX);
        s[c][ly][kHX + r - ly * (kSX - kHX)] = 0.0f;
    }
}

__device__ __forceinline__ void unpack16(const float* row, float (&v)[16]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float4 q = reinterpret_cast<const float4*>(row)[k];
        v[4 * k] = q.x; v[4 * k + 1] = q.y; v[4 * k + 2] = q.z; v[4 * k + 3] = q.w;
    }
}

template <bool FUSED>
__global__ void __launch_bounds__(kThreads) ssim_forward_kernel(const __grid_constant__ SsimArgs a) {
    __shared__ __align__(16) float s_x[3][kHY][kSX];
    __shared__ __align__(16) float s_y[3][kHY][kSX];
    __shared__ __align__(16) float s_h[5][kHY][kTX];
    __shared__ float s_red[2][kThreads / 32];
    const int t = threadIdx.x;
    const int bx = blockIdx.x * kTX, by = blockIdx.y * kTY, b = blockIdx.z;
    const int64_t plane = (int64_t)a.height * a.width;
    load_halo(s_x, a.x, a.x_is_nhwc != 0, b, by, bx, a.height, a.width, t);
    load_halo(s_y, a.y, false, b, by, bx, a.height, a.width, t);
    cp_async_wait_all();
    float acc_l1 = 0.0f, acc_ssim = 0.0f;
    for (int c = 0; c < 3; ++c) {
        __syncthreads();   // halo loaded (c == 0) / previous channel's vertical pass is done with s_h
        for (int item = t; item < kHY * (kTX / kStrip); item += kThreads) {   // horizontal: 26 rows x 8 strips of 4
            const int row = item >> 3, st = item & 7;
            float xv[16], yv[16];
            unpack16(&s_x[c][row][st * kStrip], xv);
            unpack16(&s_y[c][row][st * kStrip], yv);
            // the five maps as two packed pairs and a scalar: (x, y), (x^2, y^2), x y -- one issue slot per pair
            // (packed fp32 of sm_100, each half rounded like the scalar fma)
            float2 a01[kStrip], a23[kStrip];
            float a4[kStrip];
#pragma unroll
            for (int o = 0; o < kStrip; ++o) {
                a01[o] = make_float2(0.0f, 0.0f);
                a23[o] = make_float2(0.0f, 0.0f);
                a4[o] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < kTaps; ++i) {
                const float2 p = make_float2(xv[i], yv[i]);
                const float2 q = __fmul2_rn(p, p);
                const float xy = p.x * p.y;
#pragma unroll
                for (int o = 0; o < kStrip; ++o) {
                    const int j = i - o;
                    if (j >= 0 && j < kWin) {
                        const float w = a.win.g[j];
                        const float2 ww = make_float2(w, w);
                        a01[o] = __ffma2_rn(p, ww, a01[o]);
                        a23[o] = __ffma2_rn(q, ww, a23[o]);
                        a4[o] = fmaf(xy, w, a4[o]);
                    }
                }
            }
            *reinterpret_cast<float4*>(&s_h[0][row][st * kStrip]) = make_float4(a01[0].x, a01[1].x, a01[2].x, a01[3].x);
            *reinterpret_cast<float4*>(&s_h[1][row][st * kStrip]) = make_float4(a01[0].y, a01[1].y, a01[2].y, a01[3].y);
            *reinterpret_cast<float4*>(&s_h[2][row][st * kStrip]) = make_float4(a23[0].x, a23[1].x, a23[2].x, a23[3].x);
            *reinterpret_cast<float4*>(&s_h[3][row][st * kStrip]) = make_float4(a23[0].y, a23[1].y, a23[2].y, a23[3].y);
            *reinterpret_cast<float4*>(&s_h[4][row][st * kStrip]) = make_float4(a4[0], a4[1], a4[2], a4[3]);
        }
        __syncthreads();
        {   // vertical: 32 columns x 4 strips of 4 rows = one item per thread
            const int col = t & 31, st = t >> 5;
            float2 a01[kStrip], a23[kStrip];
            float a4[kStrip];
#pragma unroll
            for (int o = 0; o < kStrip; ++o) {
                a01[o] = make_float2(0.0f, 0.0f);
                a23[o] = make_float2(0.0f, 0.0f);
                a4[o] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < kTaps; ++i) {
                const float2 v01 = make_float2(s_h[0][st * kStrip + i][col], s_h[1][st * kStrip + i][col]);
                const float2 v23 = make_float2(s_h[2][st * kStrip + i][col], s_h[3][st * kStrip + i][col]);
                const float v4 = s_h[4][st * kStrip + i][col];
#pragma unroll
                for (int o = 0; o < kStrip; ++o) {
                    const int j = i - o;
                    if (j >= 0 && j < kWin) {
                        const float w = a.win.g[j];
                        const float2 ww = make_float2(w, w);
                        a01[o] = __ffma2_rn(v01, ww, a01[o]);
                        a23[o] = __ffma2_rn(v23, ww, a23[o]);
                        a4[o] = fmaf(v4, w, a4[o]);
                    }
                }
            }
            float acc[kStrip][5];
#pragma unroll
            for (int o = 0; o < kStrip; ++o) {
                acc[o][0] = a01[o].x; acc[o][1] = a01[o].y; acc[o][2] = a23[o].x; acc[o][3] = a23[o].y; acc[o][4] = a4[o];
            }
            const int px = bx + col;
#pragma unroll
            for (int o = 0; o < kStrip; ++o) {
                const int py = by + st * kStrip + o;
                if (px < a.width && py < a.height) {
                    const float m1 = acc[o][0], m2 = acc[o][1], m11 = acc[o][2], m22 = acc[o][3], m12 = acc[o][4];
                    const float C1 = 0.01f * 0.01f, C2 = 0.03f * 0.03f;
                    const float A1 = 2.0f * m1 * m2 + C1, A2 = 2.0f * (m12 - m1 * m2) + C2;
                    const float B1 = m1 * m1 + m2 * m2 + C1, B2 = (m11 - m1 * m1) + (m22 - m2 * m2) + C2;
                    const float inv = 1.0f / (B1 * B2);
                    const float ssim = A1 * A2 * inv;
                    const int64_t off = ((int64_t)b * 3 + c) * plane + (int64_t)py * a.width + px;
                    if (a.ssim_map) a.ssim_map[off] = ssim;
                    if (a.dmu1) {
                        // d ssim / d mu1, d E[x^2], d E[xy] with the other moments held fixed (fused_ssim.py:226-228)
                        a.dmu1[off] = 2.0f * m2 * (A2 - A1) * inv - 2.0f * m1 * ssim * (B2 - B1) * inv;
                        a.dmu11[off] = -ssim / B2;
                        a.dmu12[off] = 2.0f * A1 * inv;
                    }
                    if (FUSED) {
                        acc_ssim += ssim;
                        const int ly = st * kStrip + o + kPad, lx = col + kPad;
                        acc_l1 += fabsf(s_x[c][ly][lx] - s_y[c][ly][lx]);
                    }
                }
            }
        }
    }
    if (FUSED) {
        const int lane = t & 31, warp = t >> 5;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc_l1 += __shfl_xor_sync(0xffffffffu, acc_l1, o);
            acc_ssim += __shfl_xor_sync(0xffffffffu, acc_ssim, o);
        }
        if (lane == 0) { s_red[0][warp] = acc_l1; s_red[1][warp] = acc_ssim; }
        __syncthreads();
        if (t == 0) {
            double l1 = 0.0, ss = 0.0;
            for (int w = 0; w < kThreads / 32; ++w) { l1 += s_red[0][w]; ss += s_red[1][w]; }
            atomicAdd(&a.sums[0], l1);
            atomicAdd(&a.sums[1], ss);
        }
    }
}

template <bool FUSED>
__global__ void __launch_bounds__(kThreads) ssim_backward_kernel(const __grid_constant__ SsimArgs a) {
    __shared__ __align__(16) float s_m[3][kHY][kSX];   // ds*dmu1, ds*dmu11, ds*dmu12 of one channel
    __shared__ __align__(16) float s_h[3][kHY][kTX];
    const int t = threadIdx.x;
    const int bx = blockIdx.x * kTX, by = blockIdx.y * kTY, b = blockIdx.z;
    const int64_t plane = (int64_t)a.height * a.width;
    const int col = t & 31, vst = t >> 5;               // this thread's column / strip in the vertical pass
    const int px = bx + col;
    float d[kStrip][3];                                 // results of the vertical-pass threads, all channels
    // stage the three derivative maps of channel c (asynchronously in the fused variant)
    auto stage = [&](int c) {
        float(*dst)[kHY][kSX] = s_m;
        for (int k = t; k < kHY * kSX; k += kThreads) {
            const int ly = k / kSX, lx = k - ly * kSX;
            const int gy = by + ly - kPad, gx = bx + lx - kPad;
            const bool ok = lx < kHX && gy >= 0 && gy < a.height && gx >= 0 && gx < a.width;
            const int64_t o = ok ? ((int64_t)b * 3 + c) * plane + (int64_t)gy * a.width + gx : 0;
            if (FUSED) {   // the constant dloss/dssim is applied at the end: plain asynchronous copies
                cp_async4(&dst[0][ly][lx], a.dmu1 + o, ok);
                cp_async4(&dst[1][ly][lx], a.dmu11 + o, ok);
                cp_async4(&dst[2][ly][lx], a.dmu12 + o, ok);
            } else {
                const float ds = ok ? a.dssim[o] : 0.0f;
                dst[0][ly][lx] = ok ? ds * a.dmu1[o] : 0.0f;
                dst[1][ly][lx] = ok ? ds * a.dmu11[o] : 0.0f;
                dst[2][ly][lx] = ok ? ds * a.dmu12[o] : 0.0f;
            }
        }
    };
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        __syncthreads();   // everyone is done with the previous channel's s_m and s_h
        stage(c);
        if (FUSED) cp_async_wait_all();
        __syncthreads();
        float(*s_cur)[kHY][kSX] = s_m;
        for (int item = t; item < kHY * (kTX / kStrip); item += kThreads) {
            const int row = item >> 3, st = item & 7;
            {   // maps 0 and 1 as one packed pair, map 2 alone
                float v0[16], v1[16], v2[16];
                unpack16(&s_cur[0][row][st * kStrip], v0);
                unpack16(&s_cur[1][row][st * kStrip], v1);
                unpack16(&s_cur[2][row][st * kStrip], v2);
                float2 a01[kStrip];
                float a2[kStrip];
#pragma unroll
                for (int o = 0; o < kStrip; ++o) {
                    a01[o] = make_float2(0.0f, 0.0f);
                    a2[o] = 0.0f;
                }
#pragma unroll
                for (int i = 0; i < kTaps; ++i) {
                    const float2 p = make_float2(v0[i], v1[i]);
#pragma unroll
                    for (int o = 0; o < kStrip; ++o) {
                        const int j = i - o;
                        if (j >= 0 && j < kWin) {
                            const float w = a.win.g[j];
                            a01[o] = __ffma2_rn(p, make_float2(w, w), a01[o]);
                            a2[o] = fmaf(v2[i], w, a2[o]);
                        }
                    }
                }
                *reinterpret_cast<float4*>(&s_h[0][row][st * kStrip]) = make_float4(a01[0].x, a01[1].x, a01[2].x, a01[3].x);
                *reinterpret_cast<float4*>(&s_h[1][row][st * kStrip]) = make_float4(a01[0].y, a01[1].y, a01[2].y, a01[3].y);
                *reinterpret_cast<float4*>(&s_h[2][row][st * kStrip]) = make_float4(a2[0], a2[1], a2[2], a2[3]);
            }
        }
        __syncthreads();
        {
            float acc[kStrip][3];
#pragma unroll
            for (int o = 0; o < kStrip; ++o) acc[o][0] = acc[o][1] = acc[o][2] = 0.0f;
#pragma unroll
            for (int i = 0; i < kTaps; ++i) {
                const float v0 = s_h[0][vst * kStrip + i][col], v1 = s_h[1][vst * kStrip + i][col],
                            v2 = s_h[2][vst * kStrip + i][col];
#pragma unroll
                for (int o = 0; o < kStrip; ++o) {
                    const int j = i - o;
                    if (j >= 0 && j < kWin) {
                        const float w = a.win.g[j];
                        const float2 r = __ffma2_rn(make_float2(v0, v1), make_float2(w, w), make_float2(acc[o][0], acc[o][1]));
                        acc[o][0] = r.x; acc[o][1] = r.y;
                        acc[o][2] = fmaf(v2, w, acc[o][2]);
                    }
                }
            }
#pragma unroll
            for (int o = 0; o < kStrip; ++o) {
                const int py = by + vst * kStrip + o;
                d[o][c] = 0.0f;
                if (px < a.width && py < a.height) {
                    const float xv = a.x_is_nhwc ? a.x[(((int64_t)b * a.height + py) * a.width + px) * 3 + c]
                                                 : a.x[((int64_t)b * 3 + c) * plane + (int64_t)py * a.width + px];
                    const float yv = a.y[((int64_t)b * 3 + c) * plane + (int64_t)py * a.width + px];
                    float g = acc[o][0] + 2.0f * xv * acc[o][1] + acc[o][2] * yv;                 // fused_ssim.py:361
                    if (FUSED) {
                        const float df = xv - yv;
                        const float sg = df > 0.0f ? 1.0f : (df < 0.0f ? -1.0f : 0.0f);
                        g = a.gs * g + a.gl * sg;
                    }
                    d[o][c] = g;
                }
            }
        }
    }
    {
#pragma unroll
        for (int o = 0; o < kStrip; ++o) {
            const int py = by + vst * kStrip + o;
            if (px < a.width && py < a.height) {
                if (a.x_is_nhwc) {
                    float* dst = a.dx + (((int64_t)b * a.height + py) * a.width + px) * 3;
                    dst[0] = d[o][0]; dst[1] = d[o][1]; dst[2] = d[o][2];
                } else {
#pragma unroll
                    for (int c = 0; c < 3; ++c) a.dx[((int64_t)b * 3 + c) * plane + (int64_t)py * a.width + px] = d[o][c];
                }
            }
        }
    }
}

int32_t check_shape(int32_t batch, int32_t height, int32_t width) {
    D3GS_REQUIRE(batch >= 1 && batch <= 65535, "batch %d outside [1,65535]", batch);
    D3GS_REQUIRE(height >= 1 && width >= 1, "bad image size %dx%d", width, height);
    D3GS_REQUIRE((height + kTY - 1) / kTY <= 65535, "image too tall");
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" int32_t d3gs_ssim_forward(const float* x, const float* y, int32_t batch, int32_t height, int32_t width,
                                     int32_t x_is_nhwc, float* ssim_map, float* dmu1, float* dmu11, float* dmu12,
                                     void* stream) {
    int32_t rc = check_shape(batch, height, width);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(x && y, "NULL image");
    D3GS_REQUIRE((dmu1 == nullptr) == (dmu11 == nullptr) && (dmu1 == nullptr) == (dmu12 == nullptr),
                 "dmu1/dmu11/dmu12 must be given together");
    SsimArgs a = {};
    a.x = x; a.y = y; a.batch = batch; a.height = height; a.width = width; a.x_is_nhwc = x_is_nhwc;
    a.win = make_window();
    a.ssim_map = ssim_map; a.dmu1 = dmu1; a.dmu11 = dmu11; a.dmu12 = dmu12;
    dim3 grid((width + kTX - 1) / kTX, (height + kTY - 1) / kTY, batch), block(kThreads);
    ssim_forward_kernel<false><<<grid, block, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("ssim_forward_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_ssim_backward(const float* dssim_map, const float* dmu1, const float* dmu11,
                                      const float* dmu12, const float* x, const float* y, int32_t batch,
                                      int32_t height, int32_t width, int32_t x_is_nhwc, float* dx, void* stream) {
    int32_t rc = check_shape(batch, height, width);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(dssim_map && dmu1 && dmu11 && dmu12 && x && y && dx, "NULL argument");
    SsimArgs a = {};
    a.x = x; a.y = y; a.batch = batch; a.height = height; a.width = width; a.x_is_nhwc = x_is_nhwc;
    a.win = make_window();
    a.dmu1 = const_cast<float*>(dmu1); a.dmu11 = const_cast<float*>(dmu11); a.dmu12 = const_cast<float*>(dmu12);
    a.dssim = dssim_map; a.dx = dx;
    dim3 grid((width + kTX - 1) / kTX, (height + kTY - 1) / kTY, batch), block(kThreads);
    ssim_backward_kernel<false><<<grid, block, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("ssim_backward_kernel");
    return D3GS_OK;
}

extern "C" size_t d3gs_l1_dssim_scratch_bytes(int32_t batch, int32_t height, int32_t width) {
    if (batch < 0 || height < 0 || width < 0) return 0;
    return (size_t)3 * batch * 3 * height * width * sizeof(float);
}

extern "C" int32_t d3gs_l1_dssim_forward_backward(const float* x, const float* y, int32_t batch, int32_t height,
                                                  int32_t width, float lambda_dssim, float grad_scale, double* sums,
                                                  float* dx, void* scratch, size_t scratch_bytes, void* stream) {
    int32_t rc = check_shape(batch, height, width);
    if (rc != D3GS_OK) return rc;
    D3GS_REQUIRE(x && y && sums, "NULL argument");
    D3GS_REQUIRE(dx == nullptr || scratch != nullptr, "scratch is NULL");
    D3GS_REQUIRE(dx == nullptr || scratch_bytes >= d3gs_l1_dssim_scratch_bytes(batch, height, width),
                 "loss scratch too small");
    cudaStream_t s = (cudaStream_t)stream;
    D3GS_CUDA(cudaMemsetAsync(sums, 0, 2 * sizeof(double), s));
    const size_t plane3 = (size_t)batch * 3 * height * width;
    SsimArgs a = {};
    a.x = x; a.y = y; a.batch = batch; a.height = height; a.width = width; a.x_is_nhwc = 1;
    a.win = make_window();
    a.sums = sums;
    if (dx != nullptr) {
        a.dmu1 = reinterpret_cast<float*>(scratch);
        a.dmu11 = a.dmu1 + plane3;
        a.dmu12 = a.dmu11 + plane3;
    }
    dim3 grid((width + kTX - 1) / kTX, (height + kTY - 1) / kTY, batch), block(kThreads);
    ssim_forward_kernel<true><<<grid, block, 0, s>>>(a);
    D3GS_LAUNCH_CHECK("ssim_forward_kernel<fused>");
    if (dx == nullptr) return D3GS_OK;
    const double n = (double)plane3;
    a.gs = (float)(-(double)lambda_dssim * (double)grad_scale / n);   // d/dssim of lambda*(1-mean ssim)
    a.gl = (float)((1.0 - (double)lambda_dssim) * (double)grad_scale / n);
    a.dx = dx;
    ssim_backward_kernel<true><<<grid, block, 0, s>>>(a);
    D3GS_LAUNCH_CHECK("ssim_backward_kernel<fused>");
    return D3GS_OK;
}
