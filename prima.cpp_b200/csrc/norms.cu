// prima.cpp_b200/csrc/norms.cu — the frame of a pre-norm layer with token shift and depth average, and the gated steps around its
// mixers and feed-forward (declarations and semantics: layers.h): RMS norm in groups, the blend of a token's normed input with the
// previous token's (state per sequence slot), the weighted sum over the results of all layers so far, RMS norm + gate of a linear
// attention's output, the clamped gated unit.  Everything is fp32; only a value written for a dense product takes its operand type.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include <algorithm>

#include "layers.h"
#include "mixers.cuh"

namespace pb {
namespace {

constexpr int MAX_NORM_GROUPS = 64;

// 1 / sqrt(mean(part^2) + eps) of every group of a row -> inv[0..groups) in shared memory; all threads of the CTA take part.
// Several groups: a warp sums a whole group (no CTA-wide reduction, one barrier); one group: the CTA sums it together.
__device__ __forceinline__ void group_inv_rms(const float * __restrict__ row, int width, int groups, float eps, float * inv, float * red) {
    const int part = width / groups;
    if (groups == 1) {
        float q = 0.f;
        for (int i = threadIdx.x; i < part; i += blockDim.x) { const float v = row[i]; q = fmaf(v, v, q); }
        const float s = block_sum(q, red);
        if (threadIdx.x == 0) inv[0] = 1.f / sqrtf(s / (float) part + eps);
    } else {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
        for (int g = warp; g < groups; g += nw) {
            float q0 = 0.f, q1 = 0.f;
            int i = lane;
            for (; i + 32 < part; i += 64) { const float a = row[g * part + i], b = row[g * part + i + 32]; q0 = fmaf(a, a, q0); q1 = fmaf(b, b, q1); }
            if (i < part) { const float a = row[g * part + i]; q0 = fmaf(a, a, q0); }
            const float s = wsum(q0 + q1);
            if (lane == 0) inv[g] = 1.f / sqrtf(s / (float) part + eps);
        }
    }
    __syncthreads();
}

template <typename OT>
__global__ void __launch_bounds__(256) k_group_rmsnorm(const float * __restrict__ x, const int32_t * __restrict__ rows, const float * __restrict__ w, int groups,
                                                       float eps, OT * __restrict__ y, int width) {
    __shared__ float red[33];
    __shared__ float inv[MAX_NORM_GROUPS];
    const int r = blockIdx.x;
    const float * in = x + (int64_t) (rows ? rows[r] : r) * width;
    group_inv_rms(in, width, groups, eps, inv, red);
    const int part = width / groups;
    for (int i = threadIdx.x; i < width; i += blockDim.x) put(y, (int64_t) r * width + i, in[i] * inv[i / part] * w[i]);
}

// one CTA per token: the norm of the token and of the one before it (recomputed: a second read of a row that is in L2), then the blend
template <typename OT>
__global__ void __launch_bounds__(256) k_group_rmsnorm_shift(const float * __restrict__ x, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                                             const int32_t * __restrict__ entry_of, const float * __restrict__ w, int groups, float eps,
                                                             const float * __restrict__ mu, float * __restrict__ shift_state, int64_t slot_stride,
                                                             OT * __restrict__ y, int width) {
    __shared__ float red[33];
    __shared__ float inv[MAX_NORM_GROUPS], invp[MAX_NORM_GROUPS];
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const bool first = t == off[e], only = first && off[e + 1] == t + 1;
    const float * in = x + (int64_t) t * width;
    group_inv_rms(in, width, groups, eps, inv, red);
    if (!first) group_inv_rms(in - width, width, groups, eps, invp, red);
    float * st = shift_state + (int64_t) slot[e] * slot_stride;
    const int part = width / groups;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float h = in[i] * inv[i / part] * w[i];
        const float hp = first ? st[i] : in[i - width] * invp[i / part] * w[i];
        put(y, (int64_t) t * width + i, h + (hp - h) * mu[i]);
        if (only) st[i] = h;   // an entry of one token: this CTA is the state's only reader and writer (k_shift_state serves longer entries)
    }
}
// one CTA per entry: the normed input of its last token becomes the slot's shift state
__global__ void __launch_bounds__(256) k_shift_state(const float * __restrict__ x, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                                     const float * __restrict__ w, int groups, float eps, float * __restrict__ shift_state, int64_t slot_stride,
                                                     int width) {
    __shared__ float red[33];
    __shared__ float inv[MAX_NORM_GROUPS];
    const int e = blockIdx.x;
    if (off[e + 1] - off[e] <= 1) return;   // written by k_group_rmsnorm_shift
    const float * in = x + (int64_t) (off[e + 1] - 1) * width;
    group_inv_rms(in, width, groups, eps, inv, red);
    float * st = shift_state + (int64_t) slot[e] * slot_stride;
    const int part = width / groups;
    for (int i = threadIdx.x; i < width; i += blockDim.x) st[i] = in[i] * inv[i / part] * w[i];
}

// sum_j coef[j] * planes[j * plane_stride + i], eight planes' loads in flight
__device__ __forceinline__ float depth_sum(const float * __restrict__ planes, int64_t plane_stride, const float * __restrict__ coef, int n, int64_t i) {
    float acc = 0.f;
    int j = 0;
    for (; j + 7 < n; j += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = planes[(int64_t) (j + u) * plane_stride + i];
#pragma unroll
        for (int u = 0; u < 8; u++) acc = fmaf(coef[j + u], v[u], acc);
    }
    for (; j < n; j++) acc = fmaf(coef[j], planes[(int64_t) j * plane_stride + i], acc);
    return acc;
}
__global__ void k_depth_average(const float * __restrict__ planes, int64_t plane_stride, const float * __restrict__ coef, int n, float * __restrict__ out,
                                int64_t count) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    out[i] = depth_sum(planes, plane_stride, coef, n, i);
}
// batches of one-token entries: the depth average that closes a layer, and the next layer's norm and token shift with its state update, on
// one row held in shared memory
template <typename OT>
__global__ void __launch_bounds__(256) k_depth_average_norm_shift(const float * __restrict__ planes, int64_t plane_stride, const float * __restrict__ coef, int n,
                                                                  float * __restrict__ x, const int32_t * __restrict__ slot, const float * __restrict__ w,
                                                                  int groups, float eps, const float * __restrict__ mu, float * __restrict__ shift_state,
                                                                  int64_t slot_stride, OT * __restrict__ y, int width) {
    extern __shared__ __align__(16) float row[];   // [width]
    __shared__ float red[33];
    __shared__ float inv[MAX_NORM_GROUPS];
    const int t = blockIdx.x;        // entry t brings token t
    if ((width & 3) == 0 && (plane_stride & 3) == 0) {   // four elements per load, eight planes in flight: one CTA has to cover the row's latency alone
        const float4 * p4 = reinterpret_cast<const float4 *>(planes + (int64_t) t * width);
        const int64_t ps4 = plane_stride / 4;
        for (int i = threadIdx.x; i < width / 4; i += blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            int j = 0;
            for (; j + 7 < n; j += 8) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) v[u] = p4[(int64_t) (j + u) * ps4 + i];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const float c = coef[j + u];
                    acc.x = fmaf(c, v[u].x, acc.x); acc.y = fmaf(c, v[u].y, acc.y); acc.z = fmaf(c, v[u].z, acc.z); acc.w = fmaf(c, v[u].w, acc.w);
                }
            }
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (j + u < n) v[u] = p4[(int64_t) (j + u) * ps4 + i];
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (j + u < n) {
                    const float c = coef[j + u];
                    acc.x = fmaf(c, v[u].x, acc.x); acc.y = fmaf(c, v[u].y, acc.y); acc.z = fmaf(c, v[u].z, acc.z); acc.w = fmaf(c, v[u].w, acc.w);
                }
            reinterpret_cast<float4 *>(row)[i] = acc;
            reinterpret_cast<float4 *>(x + (int64_t) t * width)[i] = acc;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = depth_sum(planes, plane_stride, coef, n, (int64_t) t * width + i);
            row[i] = v;
            x[(int64_t) t * width + i] = v;
        }
    }
    __syncthreads();
    group_inv_rms(row, width, groups, eps, inv, red);
    float * st = shift_state + (int64_t) slot[t] * slot_stride;
    const int part = width / groups;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float h = row[i] * inv[i / part] * w[i];
        put(y, (int64_t) t * width + i, h + (st[i] - h) * mu[i]);
        st[i] = h;
    }
}

template <typename OT>
__global__ void __launch_bounds__(256) k_norm_gate(const float * __restrict__ y, const float * __restrict__ gate, int64_t ldg, int part,
                                                   const float * __restrict__ w, int gate_act, float eps, OT * __restrict__ out, int inner, int64_t ldo,
                                                   float out_scale) {
    __shared__ float red[33];
    const int t = blockIdx.x, grp = blockIdx.y;
    const float * yr = y + (int64_t) t * inner + grp * part;
    const float * gr = gate_act >= 0 ? gate + (int64_t) t * ldg + grp * part : nullptr;
    float q = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) q = fmaf(yr[i], yr[i], q);
    const float inv = 1.f / sqrtf(block_sum(q, red) / (float) part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        float v = yr[i] * inv;
        if (w) v *= w[grp * part + i];
        if (gr) v *= gate_act == 0 ? sigmoid_f(gr[i]) : silu_f(gr[i]);
        put(out, (int64_t) t * ldo + grp * part + i, v * out_scale);
    }
}

template <typename OT>
__global__ void k_clamped_glu(const float * __restrict__ gu, OT * __restrict__ y, int n_tokens, int ff, float limit) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t) n_tokens * ff) return;
    const int64_t t = i / ff, j = i - t * ff;
    const float g = fminf(gu[t * 2 * ff + j], limit);
    const float u = fminf(fmaxf(gu[t * 2 * ff + ff + j], -limit), limit);
    put(y, i, g * sigmoid_f(1.702f * g) * (u + 1.f));
}

}  // namespace

int launch_group_rmsnorm(const float * x, const int32_t * rows, const float * w, int groups, float eps, void * y, int otype, int n_rows, int width,
                         cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (groups <= 0 || groups > MAX_NORM_GROUPS || width % groups != 0) return (int) cudaErrorInvalidValue;
    return ck_launch([&] {
        if (otype == T_BF16) k_group_rmsnorm<__nv_bfloat16><<<n_rows, 256, 0, st>>>(x, rows, w, groups, eps, (__nv_bfloat16 *) y, width);
        else k_group_rmsnorm<float><<<n_rows, 256, 0, st>>>(x, rows, w, groups, eps, (float *) y, width);
    });
}
int launch_group_rmsnorm_shift(const float * x, const BatchView & b, const float * w, int groups, float eps, const float * mu, float * shift_state,
                               int64_t slot_stride, void * y, int otype, int width, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (!mu) return launch_group_rmsnorm(x, nullptr, w, groups, eps, y, otype, b.n_tokens, width, st);
    if (groups <= 0 || groups > MAX_NORM_GROUPS || width % groups != 0 || !shift_state) return (int) cudaErrorInvalidValue;
    int rc = ck_launch([&] {
        if (otype == T_BF16)
            k_group_rmsnorm_shift<__nv_bfloat16><<<b.n_tokens, 256, 0, st>>>(x, b.slot, b.off, b.entry_of, w, groups, eps, mu, shift_state, slot_stride,
                                                                             (__nv_bfloat16 *) y, width);
        else k_group_rmsnorm_shift<float><<<b.n_tokens, 256, 0, st>>>(x, b.slot, b.off, b.entry_of, w, groups, eps, mu, shift_state, slot_stride, (float *) y, width);
    });
    if (rc || b.max_n <= 1) return rc;   // one-token entries have written their state themselves
    return ck_launch([&] { k_shift_state<<<b.n_entries, 256, 0, st>>>(x, b.slot, b.off, w, groups, eps, shift_state, slot_stride, width); });
}
int launch_depth_average(const float * planes, int64_t plane_stride, const float * coef, int n, float * out, int64_t count, cudaStream_t st) {
    if (count <= 0 || n <= 0) return 0;
    return ck_launch([&] { k_depth_average<<<(unsigned) ((count + 255) / 256), 256, 0, st>>>(planes, plane_stride, coef, n, out, count); });
}
int launch_depth_average_norm_shift(const float * planes, int64_t plane_stride, const float * coef, int n, float * x, const BatchView & b, const float * w,
                                    int groups, float eps, const float * mu, float * shift_state, int64_t slot_stride, void * y, int otype, int width,
                                    cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (b.max_n != 1 || b.n_tokens != b.n_entries || groups <= 0 || groups > MAX_NORM_GROUPS || width % groups != 0 || !mu || !shift_state || n <= 0)
        return (int) cudaErrorInvalidValue;
    const size_t smem = (size_t) width * sizeof(float);
    if (otype == T_BF16) {
        int rc = raise_smem(k_depth_average_norm_shift<__nv_bfloat16>, smem);
        if (rc) return rc;
        return ck_launch([&] {
            k_depth_average_norm_shift<__nv_bfloat16><<<b.n_tokens, 256, smem, st>>>(planes, plane_stride, coef, n, x, b.slot, w, groups, eps, mu, shift_state,
                                                                                     slot_stride, (__nv_bfloat16 *) y, width);
        });
    }
    int rc = raise_smem(k_depth_average_norm_shift<float>, smem);
    if (rc) return rc;
    return ck_launch([&] {
        k_depth_average_norm_shift<float><<<b.n_tokens, 256, smem, st>>>(planes, plane_stride, coef, n, x, b.slot, w, groups, eps, mu, shift_state, slot_stride,
                                                                         (float *) y, width);
    });
}
int launch_norm_gate(const float * y, const float * gate, int64_t ldg, int groups, const float * w, int gate_act, float eps, void * out, int otype,
                     int n_tokens, int inner, cudaStream_t st, int64_t ldo, float out_scale) {
    if (n_tokens <= 0) return 0;
    if (groups <= 0 || inner % groups != 0) return (int) cudaErrorInvalidValue;
    if (!gate) gate_act = -1;
    if (ldo <= 0) ldo = inner;
    const dim3 grid((unsigned) n_tokens, (unsigned) groups);
    return ck_launch([&] {
        if (otype == T_BF16) k_norm_gate<__nv_bfloat16><<<grid, 256, 0, st>>>(y, gate, ldg, inner / groups, w, gate_act, eps, (__nv_bfloat16 *) out, inner, ldo, out_scale);
        else k_norm_gate<float><<<grid, 256, 0, st>>>(y, gate, ldg, inner / groups, w, gate_act, eps, (float *) out, inner, ldo, out_scale);
    });
}
int launch_clamped_glu(const float * gu, void * y, int otype, int n_tokens, int ff, float limit, cudaStream_t st) {
    const int64_t n = (int64_t) n_tokens * ff;
    if (n <= 0) return 0;
    const unsigned grid = (unsigned) ((n + 255) / 256);
    return ck_launch([&] {
        if (otype == T_BF16) k_clamped_glu<__nv_bfloat16><<<grid, 256, 0, st>>>(gu, (__nv_bfloat16 *) y, n_tokens, ff, limit);
        else k_clamped_glu<float><<<grid, 256, 0, st>>>(gu, (float *) y, n_tokens, ff, limit);
    });
}

}  // namespace pb
