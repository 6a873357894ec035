// Shared device/host helpers for the d3gs_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "d3gs_b200.h"

namespace d3gs {

// ---- host-side error plumbing ------------------------------------------------------------
void set_error(const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what);
void count_launch();

// Test hooks (d3gs_test_hooks): a poll limit for every bounded wait of the kernels launched afterwards (0 = the
// built-in limits) and the index of one CTA / tile that withholds what others wait for -- its look-back flag, or
// the bulk copy its own mbarrier expects (-1 = nobody).  With them a test makes a bounded wait run out without
// touching memory it should not: the waiting code gives up, sets its status bit and returns.
struct TestHooks {
    uint32_t poll_limit;
    int32_t hold;
};
TestHooks test_hooks();

#define D3GS_REQUIRE(cond, ...)                 \
    do {                                        \
        if (!(cond)) {                          \
            ::d3gs::set_error(__VA_ARGS__);     \
            return D3GS_ERR_INVALID_ARGUMENT;   \
        }                                       \
    } while (0)

#define D3GS_CUDA(expr)                                          \
    do {                                                         \
        cudaError_t e__ = (expr);                                \
        if (e__ != cudaSuccess) return ::d3gs::cuda_fail(e__, #expr); \
    } while (0)

// every kernel launch of the library passes here once: the launch is counted (d3gs_kernel_launch_count)
#define D3GS_LAUNCH_CHECK(name)                                  \
    do {                                                         \
        ::d3gs::count_launch();                                  \
        cudaError_t e__ = cudaGetLastError();                    \
        if (e__ != cudaSuccess) return ::d3gs::cuda_fail(e__, name); \
    } while (0)

inline int64_t div_up64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device math with a defined bit pattern -----------------------------------------------
// The integer results of the binning stages (radius, tile rect, culling compares, sort keys)
// and n_contrib depend on a handful of float expressions.  Those expressions are written with
// explicit round-to-nearest intrinsics / fmaf so that the compiler can neither contract nor
// reorder them; a host program using IEEE float arithmetic and fmaf reproduces every bit.

__device__ __forceinline__ float f_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float f_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float f_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float f_fma(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ float f_div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float f_sqrt(float a) { return __fsqrt_rn(a); }

// Instance rendering (render.py:346-354): the camera of view b in the frame of Gaussian g's object instance,
// out[k*3 + j] = k-th column of the camera-to-instance rotation, out[9..11] = the camera centre in that frame.
// cam2instance = inverse(instance2world) @ cam2world with the rigid inverse: R = Ri^T Rc, c = Ri^T (cc - ti); a
// [4,3] transform T holds Ri^T in rows 0-2 (T[j*3 + m] = Ri[m][j]) and ti in row 3.  Returns false (out untouched)
// for a Gaussian that belongs to no instance.
__device__ __forceinline__ bool instance_camera(const D3gsOpConfig& cf, int b, int64_t g, float* out) {
    const int inst = cf.instance_id[g];
    if (inst < 0) return false;
    const float* T = cf.instance2world_T + ((int64_t)cf.frame_ids[b] * cf.num_instance + inst) * 12;
    const float* Rc = cf.cameras[b].cam2world_T;
    float t[12];
#pragma unroll
    for (int k = 0; k < 12; ++k) t[k] = T[k];
    const float dc0 = f_sub(Rc[9], t[9]), dc1 = f_sub(Rc[10], t[10]), dc2 = f_sub(Rc[11], t[11]);
#pragma unroll
    for (int j = 0; j < 3; ++j) {
#pragma unroll
        for (int k = 0; k < 3; ++k)
            out[k * 3 + j] = f_add(f_add(f_mul(t[j * 3], Rc[k * 3]), f_mul(t[j * 3 + 1], Rc[k * 3 + 1])),
                                   f_mul(t[j * 3 + 2], Rc[k * 3 + 2]));
        out[9 + j] = f_add(f_add(f_mul(t[j * 3], dc0), f_mul(t[j * 3 + 1], dc1)), f_mul(t[j * 3 + 2], dc2));
    }
    return true;
}

// exp(x) of the fused "exponential"/"sigmoid" activations (origin/model.py:453-462): Cephes-style
// reduction, degree-5 polynomial.
__device__ __forceinline__ float act_exp(float x) {
    x = fminf(fmaxf(x, -87.0f), 88.0f);
    float n = rintf(f_mul(x, 1.44269504088896341f));
    float r = f_fma(n, -0.693359375f, x);
    r = f_fma(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = f_fma(p, r, 1.3981999507e-3f);
    p = f_fma(p, r, 8.3334519073e-3f);
    p = f_fma(p, r, 4.1665795894e-2f);
    p = f_fma(p, r, 1.6666665459e-1f);
    p = f_fma(p, r, 5.0000001201e-1f);
    float y = f_add(f_fma(p, f_mul(r, r), r), 1.0f);
    int ni = (int)n;
    return f_mul(y, __uint_as_float((uint32_t)(ni + 127) << 23));
}

// log(x), x > 0 finite (early-filter bound, render.py:1020): Cephes logf.
__device__ __forceinline__ float act_log(float x) {
    uint32_t u = __float_as_uint(x);
    int e = (int)((u >> 23) & 0xff) - 126;
    float m = __uint_as_float((u & 0x007fffffu) | 0x3f000000u);
    if (m < 0.707106781186547524f) { e -= 1; m = f_sub(f_add(m, m), 1.0f); } else { m = f_sub(m, 1.0f); }
    float z = f_mul(m, m);
    float p = 7.0376836292e-2f;
    p = f_fma(p, m, -1.1514610310e-1f);
    p = f_fma(p, m, 1.1676998740e-1f);
    p = f_fma(p, m, -1.2420140846e-1f);
    p = f_fma(p, m, 1.4249322787e-1f);
    p = f_fma(p, m, -1.6668057665e-1f);
    p = f_fma(p, m, 2.0000714765e-1f);
    p = f_fma(p, m, -2.4999993993e-1f);
    p = f_fma(p, m, 3.3333331174e-1f);
    float y = f_mul(f_mul(m, z), p);
    float fe = (float)e;
    y = f_fma(fe, -2.12194440e-4f, y);
    y = f_fma(-0.5f, z, y);
    float r = f_add(m, y);
    return f_fma(fe, 0.693359375f, r);
}

// exp(power) of the blend loop (`fast_exp`, render.py:1768): 2^t by magic-number rounding and a
// degree-5 minimax polynomial (max rel. error 2.2e-7), ten FP32-pipe operations, no SFU.
__device__ __forceinline__ float blend_exp(float power) {
    float t = fmaxf(f_mul(power, 1.44269504088896341f), -125.0f);
    t = fminf(t, 125.0f);
    float m = f_add(t, 12582912.0f);
    float n = f_sub(m, 12582912.0f);
    float f = f_sub(t, n);
    float p = 0.001327647129073739f;
    p = f_fma(p, f, 0.009675540961325169f);
    p = f_fma(p, f, 0.05550713092088699f);
    p = f_fma(p, f, 0.24022120237350464f);
    p = f_fma(p, f, 0.6931469440460205f);
    p = f_fma(p, f, 1.0f);
    return __uint_as_float(__float_as_uint(p) + (__float_as_uint(m) << 23));
}

// power = -0.5(a dx^2 + c dy^2) - b dx dy evaluated as dx*(ha*dx + nb*dy) + (hc*dy)*dy with
// ha=-0.5a, nb=-b, hc=-0.5c (render.py:1765-1767).
__device__ __forceinline__ float blend_power(float ha, float nb, float hc, float dx, float dy) {
    float t = f_fma(nb, dy, f_mul(ha, dx));
    float u = f_mul(hc, dy);
    return f_fma(t, dx, f_mul(u, dy));
}

// The 48-byte record the raster kernels read for a splat: [u v hx hy][ha nb hc o][r g b thr], where
// (ha, nb, hc) = (-0.5 a, -b, -0.5 c) of the conic.  thr is a lower bound of the `power` at which the splat
// still reaches alpha_eps: power < thr  =>  opacity*exp(power) < 0.99*alpha_eps, so the blend loop may skip
// such a pixel without changing any result.  (hx, hy) are the half extents of the axis-aligned box around
// {power >= thr}, slightly inflated and widened by the half size of an 8x4 pixel block (3.5, 1.5): a block
// whose centre is further than (hx, hy) from (u, v) contains no pixel that the splat can touch.
__device__ __forceinline__ void make_splat_record(float2 uv, float4 co, float r, float g, float b, float alpha_eps,
                                                  float4& rec0, float4& rec1, float4& rec2) {
    float thr = -1.0e30f, hx = 1.0e30f, hy = 1.0e30f;
    if (co.w > alpha_eps && co.w < 1.0e30f) {
        thr = act_log(alpha_eps / co.w) - 0.01f;
        // {a dx^2 + 2 b dx dy + c dy^2 <= R}, R = -2 thr: |dx| <= sqrt(R c / det), |dy| <= sqrt(R a / det)
        const float det = co.x * co.z - co.y * co.y;
        // Very elongated splats (a*c >> det) are left unculled: there the float evaluation of `power`
        // cancels heavily and can exceed thr slightly outside the exact box.  Up to a*c/det = 1e3 the
        // rounding error of power stays below 1e-3, a tenth of the 0.01 margin built into thr.
        if (det > 0.0f && co.x * co.z < 1.0e3f * det) {
            const float R = -2.0f * thr;
            hx = sqrtf(R * co.z / det) * 1.0005f + 0.02f + 3.5f;
            hy = sqrtf(R * co.x / det) * 1.0005f + 0.02f + 1.5f;
        }
    }
    rec0 = make_float4(uv.x, uv.y, hx, hy);
    rec1 = make_float4(-0.5f * co.x, -co.y, -0.5f * co.z, co.w);
    rec2 = make_float4(r, g, b, thr);
}

// ---- Adam (d3sim/csrc/optim.py:22-49), shared by the optimizer kernels and the fused backward -------------
// per-tensor scalars with the uniform divisions hoisted out of the element loop
struct SegConst {
    float inv_grad_scale, weight_decay, beta1, omb1, beta2, omb2, step_size, inv_bc2_sqrt, eps;
};

inline SegConst make_seg_const(const D3gsAdamSegment& s) {
    SegConst c;
    c.inv_grad_scale = (float)(1.0 / (double)s.grad_scale);
    c.weight_decay = s.weight_decay;
    c.beta1 = s.beta1;
    c.omb1 = 1.0f - s.beta1;
    c.beta2 = s.beta2;
    c.omb2 = 1.0f - s.beta2;
    c.step_size = s.lr / s.bias_correction1;
    c.inv_bc2_sqrt = (float)(1.0 / (double)s.bias_correction2_sqrt);
    c.eps = s.eps;
    return c;
}

// g /= grad_scale; m = mix(g, m, b1); v = mix(g*g, v, b2); p -= (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps).
// The three divisions by per-tensor constants are multiplications by reciprocals computed once on the host in
// double; the one per-element division is a single correctly rounded reciprocal.  Every operation is an
// explicit round-to-nearest intrinsic, so every kernel that applies Adam produces the same bits for the same
// inputs whatever the compiler would have contracted.
__device__ __forceinline__ void adam_update(float g, float& p, float& m, float& v, const SegConst& c) {
    g = __fmul_rn(g, c.inv_grad_scale);
    if (c.weight_decay != 0.0f) g = __fmaf_rn(p, c.weight_decay, g);
    m = __fmaf_rn(g, c.omb1, __fmul_rn(m, c.beta1));
    v = __fmaf_rn(__fmul_rn(g, g), c.omb2, __fmul_rn(v, c.beta2));
    const float denom = __fmaf_rn(__fsqrt_rn(v), c.inv_bc2_sqrt, c.eps);
    p = __fmaf_rn(-__fmul_rn(c.step_size, m), __frcp_rn(denom), p);
}

// densification statistics of one Gaussian (d3sim/algos/d3gs/origin/strategy.py:93-122)
__device__ __forceinline__ void stats_update(const D3gsDensifyStats& st, int64_t i) {
    float la = 0.0f, ca = 0.0f, mr = st.need_max_radii ? st.max_radii[i] : 0.0f;
    const float lb = (float)(st.loss_batch > 0 ? st.loss_batch : st.batch);
    const float sx = 0.5f * (float)st.width * lb, sy = 0.5f * (float)st.height * lb;
    const float mwh = (float)max(st.width, st.height);
    const int64_t stride = st.duv_stride > 0 ? st.duv_stride : 2;
    for (int j = 0; j < st.batch; ++j) {
        const int64_t k = (int64_t)j * st.num + i;
        const float2 d = *reinterpret_cast<const float2*>(st.duv + k * stride);
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

__device__ __forceinline__ int f2i_sat(float v) {
    v = fminf(fmaxf(v, -2.0e9f), 2.0e9f);
    return (int)v;
}
__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// ---- mbarrier + bulk async copy (TMA engine, non-tensor form), own memory only ---------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// global -> shared bulk copy; dst/src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// shared -> global bulk copy (bulk-group completion); same alignment rules
__device__ __forceinline__ void bulk_copy_s2g(void* dst_gmem, const void* src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until the committed bulk stores have finished READING shared memory (it may then be reused/freed)
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// 4-byte asynchronous global -> shared copy (no register staging, any number in flight per thread);
// valid == false writes zero and reads nothing.
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src_gmem, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem),
                 "r"(valid ? 4 : 0)
                 : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// 16-byte asynchronous global -> shared copy through L2 (both addresses 16-byte aligned)
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (seconds), returns false so the caller can flag
// D3GS_STATUS_COPY_TIMEOUT and leave instead of hanging the device.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = 0) {
    const uint32_t polls = limit != 0 ? limit : (1u << 22);
    for (uint32_t it = 0; it < polls; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(64);
    }
    return false;
}

}  // namespace d3gs
