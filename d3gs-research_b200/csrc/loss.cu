// K9/K10: SSIM map forward/backward and the fused L1 + D-SSIM loss gradient.
//
// Reference semantics: d3sim/ops/image/fused_ssim.py:93-377 (11x11 Gaussian window sigma 1.5 =
// outer product of the normalised 1-D window (32-40), zero padding (175-178), C1=1e-4, C2=9e-4,
// saved partials dmu1/dmu11/dmu12 (226-231), backward = three convolutions (341-361)), and
// d3sim/algos/d3gs/train.py:169-172 / losses.py:19-20 for the loss combination.
//
// The reference applies the window as 121 taps per output; here it is applied separably (11
// horizontal + 11 vertical taps) from shared memory.  In the fused entry point the rasteriser's
// NHWC colour is read directly and dL/dcolor is written NHWC, so the reference's
// permute(0,3,1,2).contiguous() round trip (train.py:169) and its autograd mirror disappear.
#include <cmath>

#include "common.cuh"

namespace d3gs {
namespace {

constexpr int kWin = 11, kPad = 5, kTile = 16, kHalo = kTile + 2 * kPad;   // 26

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

__device__ __forceinline__ float load_x(const SsimArgs& a, int b, int c, int yy, int xx) {
    if (a.x_is_nhwc) return a.x[(((int64_t)b * a.height + yy) * a.width + xx) * 3 + c];
    return a.x[(((int64_t)b * 3 + c) * a.height + yy) * a.width + xx];
}

template <bool FUSED>
__global__ void __launch_bounds__(256) ssim_forward_kernel(const __grid_constant__ SsimArgs a) {
    __shared__ float s_x[kHalo][kHalo + 1];
    __shared__ float s_y[kHalo][kHalo + 1];
    __shared__ float s_h[5][kHalo][kTile];
    __shared__ float s_red[2][8];
    const int tx = threadIdx.x, ty = threadIdx.y, t = ty * kTile + tx;
    const int bx = blockIdx.x * kTile, by = blockIdx.y * kTile, b = blockIdx.z;
    const int px = bx + tx, py = by + ty;
    const bool inside = px < a.width && py < a.height;
    const int64_t plane = (int64_t)a.height * a.width;
    float acc_l1 = 0.0f, acc_ssim = 0.0f;
    for (int c = 0; c < 3; ++c) {
        __syncthreads();
        for (int k = t; k < kHalo * kHalo; k += 256) {
            const int ly = k / kHalo, lx = k - ly * kHalo;
            const int gy = by + ly - kPad, gx = bx + lx - kPad;
            const bool ok = gy >= 0 && gy < a.height && gx >= 0 && gx < a.width;
            s_x[ly][lx] = ok ? load_x(a, b, c, gy, gx) : 0.0f;
            s_y[ly][lx] = ok ? a.y[((int64_t)b * 3 + c) * plane + (int64_t)gy * a.width + gx] : 0.0f;
        }
        __syncthreads();
        for (int k = t; k < kHalo * kTile; k += 256) {
            const int ly = k / kTile, lx = k - ly * kTile;
            float hx = 0.f, hy = 0.f, hxx = 0.f, hyy = 0.f, hxy = 0.f;
#pragma unroll
            for (int j = 0; j < kWin; ++j) {
                const float xv = s_x[ly][lx + j], yv = s_y[ly][lx + j], w = a.win.g[j];
                hx += xv * w; hy += yv * w; hxx += xv * xv * w; hyy += yv * yv * w; hxy += xv * yv * w;
            }
            s_h[0][ly][lx] = hx; s_h[1][ly][lx] = hy; s_h[2][ly][lx] = hxx; s_h[3][ly][lx] = hyy; s_h[4][ly][lx] = hxy;
        }
        __syncthreads();
        float m1 = 0.f, m2 = 0.f, m11 = 0.f, m22 = 0.f, m12 = 0.f;
#pragma unroll
        for (int i = 0; i < kWin; ++i) {
            const float w = a.win.g[i];
            m1 += s_h[0][ty + i][tx] * w; m2 += s_h[1][ty + i][tx] * w; m11 += s_h[2][ty + i][tx] * w;
            m22 += s_h[3][ty + i][tx] * w; m12 += s_h[4][ty + i][tx] * w;
        }
        if (inside) {
            const float C1 = 0.01f * 0.01f, C2 = 0.03f * 0.03f;
            const float A1 = 2.0f * m1 * m2 + C1, A2 = 2.0f * (m12 - m1 * m2) + C2;
            const float B1 = m1 * m1 + m2 * m2 + C1, B2 = (m11 - m1 * m1) + (m22 - m2 * m2) + C2;
            const float inv = 1.0f / (B1 * B2);
            const float ssim = A1 * A2 * inv;
            const int64_t o = ((int64_t)b * 3 + c) * plane + (int64_t)py * a.width + px;
            if (a.ssim_map) a.ssim_map[o] = ssim;
            if (a.dmu1) {
                // d ssim / d mu1, d E[x^2], d E[xy] with the other moments held fixed (fused_ssim.py:226-228)
                a.dmu1[o] = 2.0f * m2 * (A2 - A1) * inv - 2.0f * m1 * ssim * (B2 - B1) * inv;
                a.dmu11[o] = -ssim / B2;
                a.dmu12[o] = 2.0f * A1 * inv;
            }
            if (FUSED) {
                acc_ssim += ssim;
                acc_l1 += fabsf(s_x[ty + kPad][tx + kPad] - s_y[ty + kPad][tx + kPad]);
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
            for (int w = 0; w < 8; ++w) { l1 += s_red[0][w]; ss += s_red[1][w]; }
            atomicAdd(&a.sums[0], l1);
            atomicAdd(&a.sums[1], ss);
        }
    }
}

template <bool FUSED>
__global__ void __launch_bounds__(256) ssim_backward_kernel(const __grid_constant__ SsimArgs a) {
    __shared__ float s_a[kHalo][kHalo + 1];
    __shared__ float s_b[kHalo][kHalo + 1];
    __shared__ float s_c[kHalo][kHalo + 1];
    __shared__ float s_h[3][kHalo][kTile];
    const int tx = threadIdx.x, ty = threadIdx.y, t = ty * kTile + tx;
    const int bx = blockIdx.x * kTile, by = blockIdx.y * kTile, b = blockIdx.z;
    const int px = bx + tx, py = by + ty;
    const bool inside = px < a.width && py < a.height;
    const int64_t plane = (int64_t)a.height * a.width;
    for (int c = 0; c < 3; ++c) {
        __syncthreads();
        for (int k = t; k < kHalo * kHalo; k += 256) {
            const int ly = k / kHalo, lx = k - ly * kHalo;
            const int gy = by + ly - kPad, gx = bx + lx - kPad;
            const bool ok = gy >= 0 && gy < a.height && gx >= 0 && gx < a.width;
            float va = 0.f, vb = 0.f, vc = 0.f;
            if (ok) {
                const int64_t o = ((int64_t)b * 3 + c) * plane + (int64_t)gy * a.width + gx;
                const float ds = FUSED ? 1.0f : a.dssim[o];   // fused: the constant factor is applied at the end
                va = ds * a.dmu1[o]; vb = ds * a.dmu11[o]; vc = ds * a.dmu12[o];
            }
            s_a[ly][lx] = va; s_b[ly][lx] = vb; s_c[ly][lx] = vc;
        }
        __syncthreads();
        for (int k = t; k < kHalo * kTile; k += 256) {
            const int ly = k / kTile, lx = k - ly * kTile;
            float ha = 0.f, hb = 0.f, hc = 0.f;
#pragma unroll
            for (int j = 0; j < kWin; ++j) {
                const float w = a.win.g[j];
                ha += s_a[ly][lx + j] * w; hb += s_b[ly][lx + j] * w; hc += s_c[ly][lx + j] * w;
            }
            s_h[0][ly][lx] = ha; s_h[1][ly][lx] = hb; s_h[2][ly][lx] = hc;
        }
        __syncthreads();
        float c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
        for (int i = 0; i < kWin; ++i) {
            const float w = a.win.g[i];
            c1 += s_h[0][ty + i][tx] * w; c2 += s_h[1][ty + i][tx] * w; c3 += s_h[2][ty + i][tx] * w;
        }
        if (inside) {
            const float xv = load_x(a, b, c, py, px);
            const float yv = a.y[((int64_t)b * 3 + c) * plane + (int64_t)py * a.width + px];
            float d = c1 + 2.0f * xv * c2 + c3 * yv;                 // fused_ssim.py:361
            if (FUSED) {
                const float df = xv - yv;
                const float sg = df > 0.0f ? 1.0f : (df < 0.0f ? -1.0f : 0.0f);
                d = a.gs * d + a.gl * sg;
            }
            if (a.x_is_nhwc) a.dx[(((int64_t)b * a.height + py) * a.width + px) * 3 + c] = d;
            else a.dx[((int64_t)b * 3 + c) * plane + (int64_t)py * a.width + px] = d;
        }
    }
}

int32_t check_shape(int32_t batch, int32_t height, int32_t width) {
    D3GS_REQUIRE(batch >= 1 && batch <= 65535, "batch %d outside [1,65535]", batch);
    D3GS_REQUIRE(height >= 1 && width >= 1, "bad image size %dx%d", width, height);
    D3GS_REQUIRE((height + kTile - 1) / kTile <= 65535, "image too tall");
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
    dim3 grid((width + kTile - 1) / kTile, (height + kTile - 1) / kTile, batch), block(kTile, kTile);
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
    dim3 grid((width + kTile - 1) / kTile, (height + kTile - 1) / kTile, batch), block(kTile, kTile);
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
    dim3 grid((width + kTile - 1) / kTile, (height + kTile - 1) / kTile, batch), block(kTile, kTile);
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
