// Densification, pruning and opacity reset: the step on the far side of the training iteration.
//
// Reference semantics: GaussianStrategyOrigin.refine_gs (d3sim/algos/d3gs/origin/strategy.py:159-363),
// the optimizer-state surgery it triggers (select_gs_optimizer_by_mask / zero_optimizer_by_range,
// d3sim/algos/d3gs/strategy.py:131-178) and the opacity reset of the trainer
// (d3sim/algos/d3gs/origin/trainer.py:388-417, reset_param_in_optim strategy.py:181-202).
//
// The reference builds the new model with a chain of boolean-mask indexing, concatenations and per-tensor
// optimizer-state gathers in torch.  Here the whole refinement is three launches around one host read:
//   1. classify: one thread per Gaussian decides duplicate / split / prune with the reference's tests and
//      writes four 0/1 columns (keep, kept duplicate, kept split pair, split) for the scans;
//   2. (the caller scans the columns with d3gs_scan_tiles and reads the four totals: the new count)
//   3. apply: one thread per source Gaussian writes its up to four output rows -- parameters, Adam moments
//      (gathered for survivors, zero for new Gaussians) -- at the positions the scans give, in the reference's
//      output order [survivors | duplicates | first split copies | second split copies].
#include "common.cuh"

namespace d3gs {
namespace {

struct ClassifyArgs {
    D3gsModel model;
    D3gsRefineConfig rc;
    const float* duv_ndc_length;
    const float* count;
    const float* max_radii;
    int32_t* cols;   // [4][N]: keep, dup_kept, split_kept, split
    uint8_t* flags;  // [N]: bit0 duplicate, bit1 split, bit2 prune (origin), bit3 split children pruned
};

__device__ __forceinline__ void load_scale_opacity(const D3gsModel& m, const D3gsRefineConfig& rc, int64_t i, float* s,
                                                   float* opac) {
    const float r0 = m.scale[i * 3], r1 = m.scale[i * 3 + 1], r2 = m.scale[i * 3 + 2];
    s[0] = rc.fused_activations ? act_exp(r0) : r0;
    s[1] = rc.fused_activations ? act_exp(r1) : r1;
    s[2] = rc.fused_activations ? act_exp(r2) : r2;
    const float o = m.opacity[i];
    *opac = rc.fused_activations ? 1.0f / (1.0f + act_exp(-o)) : o;
}

// origin/strategy.py:195-241 (masks) and 318-331 (prune test of the split children, which depends only on the
// parent: new_scaling = scale / 1.6, same opacity and max_radii for both copies)
__global__ void __launch_bounds__(256) refine_classify_kernel(const __grid_constant__ ClassifyArgs a) {
    const int64_t n = a.model.num;
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const D3gsRefineConfig& rc = a.rc;
    float s[3], opac;
    load_scale_opacity(a.model, rc, i, s, &opac);
    const float cnt = a.count[i];
    const bool grad_high = (a.duv_ndc_length[i] / fmaxf(cnt, 1.0f)) >= rc.grow_grad2d;
    const float smax = fmaxf(fmaxf(s[0], s[1]), s[2]);
    const bool small = smax <= rc.grow_scale3d * rc.scene_scale;
    const bool dup = grad_high && small;
    bool large = !small;
    const float mr = a.max_radii[i];
    bool prune = opac < rc.prune_opacity_thresh;
    if (rc.prune_too_big) prune = prune || smax > rc.prune_scale3d * rc.scene_scale;
    if (rc.refine_by_radii) {
        large = large || mr > rc.grow_scale2d;
        prune = prune || mr > rc.prune_scale2d;
    }
    const bool split = grad_high && large;
    const bool origin_prune = prune || split;
    bool child_prune = opac < rc.prune_opacity_thresh;
    if (rc.prune_too_big) child_prune = child_prune || (smax / 1.6f) > rc.prune_scale3d * rc.scene_scale;
    if (rc.refine_by_radii) child_prune = child_prune || mr > rc.prune_scale2d;
    a.cols[i] = origin_prune ? 0 : 1;
    a.cols[n + i] = (dup && !origin_prune) ? 1 : 0;
    a.cols[2 * n + i] = (split && !child_prune) ? 1 : 0;
    a.cols[3 * n + i] = split ? 1 : 0;
    a.flags[i] = (uint8_t)((dup ? 1 : 0) | (split ? 2 : 0) | (origin_prune ? 4 : 0) | (child_prune ? 8 : 0));
}

struct ApplyArgs {
    D3gsModel src, dst;                 // dst.num = new count
    D3gsRefineConfig rc;
    const float* m_src[6];              // Adam moments per field (xyz, quaternion, scale, opacity, sh_base, sh_rest); may be NULL
    const float* v_src[6];
    float* m_dst[6];
    float* v_dst[6];
    const int32_t* scans;               // [4][N] inclusive scans of the classify columns
    const uint8_t* flags;
    const float* normals;               // [2 * n_split, 3]
    int32_t* src_index;                 // [new count]: source Gaussian of every output row (may be NULL)
    int64_t t_keep, t_dup, t_split_kept, n_split;
};

// D3gsModel describes read-only inputs elsewhere; the destination model of a refinement is written through it
__device__ __forceinline__ float* w(const float* p) { return const_cast<float*>(p); }

__device__ __forceinline__ void copy_row(const D3gsModel& src, const D3gsModel& dst, int64_t i, int64_t o) {
#pragma unroll
    for (int k = 0; k < 3; ++k) w(dst.xyz)[o * 3 + k] = src.xyz[i * 3 + k];
#pragma unroll
    for (int k = 0; k < 4; ++k) w(dst.quaternion_xyzw)[o * 4 + k] = src.quaternion_xyzw[i * 4 + k];
#pragma unroll
    for (int k = 0; k < 3; ++k) w(dst.scale)[o * 3 + k] = src.scale[i * 3 + k];
    w(dst.opacity)[o] = src.opacity[i];
    for (int k = 0; k < src.sh_base_stride; ++k)
        w(dst.sh_base)[o * dst.sh_base_stride + k] = src.sh_base[i * src.sh_base_stride + k];
    if (src.sh_rest != nullptr)
        for (int k = 0; k < src.sh_rest_stride; ++k)
            w(dst.sh_rest)[o * dst.sh_rest_stride + k] = src.sh_rest[i * src.sh_rest_stride + k];
}

// Adam moments of an output row: gathered from the source for a survivor, zero for a new Gaussian
// (strategy.py:131-178: state[inds] followed by zeroing the new range).
__device__ __forceinline__ void moments_row(const ApplyArgs& a, int64_t i, int64_t o, bool survivor) {
    const int per[6] = {3, 4, 3, 1, a.src.sh_base_stride, a.src.sh_rest != nullptr ? a.src.sh_rest_stride : 0};
#pragma unroll
    for (int f = 0; f < 6; ++f) {
        if (a.m_dst[f] == nullptr) continue;
        for (int k = 0; k < per[f]; ++k) {
            a.m_dst[f][o * per[f] + k] = survivor ? a.m_src[f][i * per[f] + k] : 0.0f;
            a.v_dst[f][o * per[f] + k] = survivor ? a.v_src[f][i * per[f] + k] : 0.0f;
        }
    }
}

// origin/strategy.py:303-317: new_xyz = R(q) (normal * scale) + xyz, new raw scale = log(scale / 1.6)
__device__ __forceinline__ void split_child(const ApplyArgs& a, int64_t i, int64_t o, const float* nrm) {
    const D3gsRefineConfig& rc = a.rc;
    float s[3], opac;
    load_scale_opacity(a.src, rc, i, s, &opac);
    const float4 qr = *reinterpret_cast<const float4*>(a.src.quaternion_xyzw + i * 4);
    const float qn = rc.fused_activations ? sqrtf(((qr.x * qr.x + qr.y * qr.y) + qr.z * qr.z) + qr.w * qr.w) : 1.0f;
    const float qx = qr.x / qn, qy = qr.y / qn, qz = qr.z / qn, qw = qr.w / qn;
    const float xx = qx * qx, yy = qy * qy, zz = qz * qz, xy = qx * qy, xz = qx * qz, yz = qy * qz;
    const float wx = qw * qx, wy = qw * qy, wz = qw * qz;
    const float R[3][3] = {{1.0f - 2.0f * (yy + zz), 2.0f * (xy - wz), 2.0f * (xz + wy)},
                           {2.0f * (xy + wz), 1.0f - 2.0f * (xx + zz), 2.0f * (yz - wx)},
                           {2.0f * (xz - wy), 2.0f * (yz + wx), 1.0f - 2.0f * (xx + yy)}};
    const float v0 = nrm[0] * s[0], v1 = nrm[1] * s[1], v2 = nrm[2] * s[2];
#pragma unroll
    for (int r = 0; r < 3; ++r)
        w(a.dst.xyz)[o * 3 + r] = ((R[r][0] * v0 + R[r][1] * v1) + R[r][2] * v2) + a.src.xyz[i * 3 + r];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const float ns = s[k] / 1.6f;
        w(a.dst.scale)[o * 3 + k] = rc.fused_activations ? act_log(ns) : ns;
    }
}

__global__ void __launch_bounds__(256) refine_apply_kernel(const __grid_constant__ ApplyArgs a) {
    const int64_t n = a.src.num;
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const uint8_t f = a.flags[i];
    const bool dup = f & 1, split = f & 2, origin_prune = f & 4, child_prune = f & 8;
    if (!origin_prune) {
        const int64_t o = a.scans[i] - 1;
        copy_row(a.src, a.dst, i, o);
        moments_row(a, i, o, true);
        if (a.src_index) a.src_index[o] = (int32_t)i;
    }
    if (dup && !origin_prune) {
        const int64_t o = a.t_keep + a.scans[n + i] - 1;
        copy_row(a.src, a.dst, i, o);
        moments_row(a, i, o, false);
        if (a.src_index) a.src_index[o] = (int32_t)i;
    }
    if (split && !child_prune) {
        const int64_t rank = a.scans[3 * n + i] - 1;          // position among all split Gaussians: selects the normals
        const int64_t k = a.scans[2 * n + i] - 1;
        const int64_t oa = a.t_keep + a.t_dup + k, ob = oa + a.t_split_kept;
        copy_row(a.src, a.dst, i, oa);
        copy_row(a.src, a.dst, i, ob);
        split_child(a, i, oa, a.normals + rank * 3);
        split_child(a, i, ob, a.normals + (a.n_split + rank) * 3);
        moments_row(a, i, oa, false);
        moments_row(a, i, ob, false);
        if (a.src_index) {
            a.src_index[oa] = (int32_t)i;
            a.src_index[ob] = (int32_t)i;
        }
    }
}

// trainer.py:388-417: opacity = logit(min(opacity_act, thresh)); the opacity moments are zeroed
__global__ void __launch_bounds__(256)
reset_opacity_kernel(float* opacity, int64_t n, float thresh, int fused, float* exp_avg, float* exp_avg_sq) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float o = opacity[i];
    if (fused) o = 1.0f / (1.0f + act_exp(-o));
    o = fminf(o, thresh);
    opacity[i] = act_log(o / (1.0f - o));
    if (exp_avg) exp_avg[i] = 0.0f;
    if (exp_avg_sq) exp_avg_sq[i] = 0.0f;
}

int32_t check_model(const D3gsModel* m, const char* what) {
    D3GS_REQUIRE(m != nullptr, "%s is NULL", what);
    D3GS_REQUIRE(m->num >= 0 && m->num < ((int64_t)1 << 31), "%s: Gaussian count out of range", what);
    D3GS_REQUIRE(m->num == 0 || (m->xyz && m->quaternion_xyzw && m->scale && m->opacity && m->sh_base),
                 "%s: tensor pointer is NULL", what);
    D3GS_REQUIRE(((uintptr_t)m->quaternion_xyzw & 15) == 0, "%s: quaternion_xyzw must be 16-byte aligned", what);
    return D3GS_OK;
}

}  // namespace
}  // namespace d3gs

using namespace d3gs;

extern "C" int32_t d3gs_refine_classify(const D3gsModel* model, const D3gsRefineConfig* rc, const float* duv_ndc_length,
                                        const float* count, const float* max_radii, int32_t* columns, uint8_t* flags,
                                        void* stream) {
    int32_t r = check_model(model, "model");
    if (r != D3GS_OK) return r;
    D3GS_REQUIRE(rc && duv_ndc_length && count && max_radii && columns && flags, "NULL argument");
    if (model->num == 0) return D3GS_OK;
    ClassifyArgs a;
    a.model = *model;
    a.rc = *rc;
    a.duv_ndc_length = duv_ndc_length;
    a.count = count;
    a.max_radii = max_radii;
    a.cols = columns;
    a.flags = flags;
    refine_classify_kernel<<<(unsigned)div_up64(model->num, 256), 256, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("refine_classify_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_refine_apply(const D3gsModel* src, const D3gsModel* dst, const D3gsRefineConfig* rc,
                                     const D3gsRefineMoments* moments, const int32_t* scans, const uint8_t* flags,
                                     const float* normals, const int64_t* totals, int32_t* src_index, void* stream) {
    int32_t r = check_model(src, "src");
    if (r != D3GS_OK) return r;
    r = check_model(dst, "dst");
    if (r != D3GS_OK) return r;
    D3GS_REQUIRE(rc && scans && flags && totals, "NULL argument");
    D3GS_REQUIRE(totals[0] >= 0 && totals[1] >= 0 && totals[2] >= 0 && totals[3] >= 0, "negative total");
    D3GS_REQUIRE(dst->num == totals[0] + totals[1] + 2 * totals[2], "dst.num %lld != keep + dup + 2 split_kept = %lld",
                 (long long)dst->num, (long long)(totals[0] + totals[1] + 2 * totals[2]));
    D3GS_REQUIRE(totals[3] == 0 || normals != nullptr, "normals is NULL");
    D3GS_REQUIRE(src->sh_base_stride == dst->sh_base_stride && src->sh_rest_stride == dst->sh_rest_stride &&
                     (src->sh_rest == nullptr) == (dst->sh_rest == nullptr || dst->num == 0),
                 "source and destination SH layouts differ");
    if (src->num == 0) return D3GS_OK;
    ApplyArgs a = {};
    a.src = *src;
    a.dst = *dst;
    a.rc = *rc;
    if (moments != nullptr) {
        for (int f = 0; f < 6; ++f) {
            D3GS_REQUIRE((moments->exp_avg_src[f] == nullptr) == (moments->exp_avg_dst[f] == nullptr) &&
                             (moments->exp_avg_src[f] == nullptr) == (moments->exp_avg_sq_src[f] == nullptr) &&
                             (moments->exp_avg_src[f] == nullptr) == (moments->exp_avg_sq_dst[f] == nullptr),
                         "moment pointers of field %d must be given together", f);
            a.m_src[f] = moments->exp_avg_src[f];
            a.v_src[f] = moments->exp_avg_sq_src[f];
            a.m_dst[f] = moments->exp_avg_dst[f];
            a.v_dst[f] = moments->exp_avg_sq_dst[f];
        }
    }
    a.scans = scans;
    a.flags = flags;
    a.normals = normals;
    a.src_index = src_index;
    a.t_keep = totals[0];
    a.t_dup = totals[1];
    a.t_split_kept = totals[2];
    a.n_split = totals[3];
    refine_apply_kernel<<<(unsigned)div_up64(src->num, 256), 256, 0, (cudaStream_t)stream>>>(a);
    D3GS_LAUNCH_CHECK("refine_apply_kernel");
    return D3GS_OK;
}

extern "C" int32_t d3gs_reset_opacity(float* opacity, int64_t num, float thresh, int32_t fused_activations,
                                      float* exp_avg, float* exp_avg_sq, void* stream) {
    D3GS_REQUIRE(num >= 0, "negative count");
    if (num == 0) return D3GS_OK;
    D3GS_REQUIRE(opacity != nullptr, "opacity is NULL");
    D3GS_REQUIRE(thresh > 0.0f && thresh < 1.0f, "threshold %g outside (0,1)", (double)thresh);
    reset_opacity_kernel<<<(unsigned)div_up64(num, 256), 256, 0, (cudaStream_t)stream>>>(opacity, num, thresh,
                                                                                       fused_activations, exp_avg,
                                                                                       exp_avg_sq);
    D3GS_LAUNCH_CHECK("reset_opacity_kernel");
    return D3GS_OK;
}
