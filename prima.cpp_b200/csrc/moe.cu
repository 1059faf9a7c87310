// prima.cpp_b200/csrc/moe.cu — routed mixture of experts (declarations and semantics: layers.h).  An expert is a clamped gated unit, a
// squared-ReLU unit or a SiLU gated unit (MoeParams::act); its routing weight multiplies its result or its input (weight_on_input).  The router runs in fp32, in one of two forms: logits + bias, the `top` largest (ties: the lower
// index), softmax over the chosen logits (k_moe_route); or sigmoid scores, a per-expert correction added for the choice only, the choice
// limited to the best groups of neighbouring experts, weights = the uncorrected scores of the chosen divided by their sum, times a factor
// (k_moe_route_sigmoid, which also yields the sigmoid gate of a shared expert).  Two ways through the experts:
//   few tokens   every (token, chosen expert) pair streams the rows of its expert (weights are read once per pair, mostly from L2 when
//                tokens share experts); no host round trip, so a decode step stays one replayable graph
//   many tokens  pairs are sorted by expert (stable counting sort on the device), activations gathered into expert-contiguous rows, the
//                engine's dense product runs over every expert's rows (one grouped tensor-core launch each way whose row counts stay on
//                the device; expert by expert where that kernel does not apply), and the results are summed per token in the order of the choice
// Either way the sum over a token's experts runs in the order of the choice, so a token's result does not depend on the batch around it.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "layers.h"
#include "mixers.cuh"

namespace pb {
namespace {

template <typename WT> struct Pack;
template <> struct Pack<float> { static constexpr int n = 4; };
template <> struct Pack<__nv_bfloat16> { static constexpr int n = 8; };
__device__ __forceinline__ void unpack16(const uint4 & r, float (&f)[4], float) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
}
__device__ __forceinline__ void unpack16(const uint4 & r, float (&f)[8], __nv_bfloat16) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
// lane's share of sum_k w[k] a[k]; VEC: 16-byte loads (K a multiple of the pack, both rows 16-byte aligned)
template <typename WT, bool VEC>
__device__ __forceinline__ float dot_part(const WT * __restrict__ w, const WT * __restrict__ a, int K, int lane) {
    float acc = 0.f;
    if constexpr (VEC) {
        constexpr int V = Pack<WT>::n;
        for (int k = lane * V; k < K; k += 32 * V) {
            float wf[V], af[V];
            unpack16(__ldg(reinterpret_cast<const uint4 *>(w + k)), wf, WT());
            unpack16(*reinterpret_cast<const uint4 *>(a + k), af, WT());
#pragma unroll
            for (int i = 0; i < V; i++) acc = fmaf(wf[i], af[i], acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(ld_f(w, k), ld_f(a, k), acc);
    }
    return acc;
}

// one CTA per token: the activations in shared memory as fp32, warps split the experts, warp 0 picks
template <typename HT>
__global__ void __launch_bounds__(256) k_moe_route(const HT * __restrict__ h, const float * __restrict__ wr, const float * __restrict__ bias, MoeParams p,
                                                   int width, int32_t * __restrict__ idx, float * __restrict__ wt) {
    extern __shared__ float sm[];
    float * hs = sm;            // [width]
    float * z = hs + width;     // [experts]
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += blockDim.x) hs[i] = ld_f(h, (int64_t) t * width + i);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = warp; e < p.experts; e += (int) (blockDim.x >> 5)) {
        const float acc = wsum(dot_lane8(wr + (int64_t) e * width, hs, width, lane));
        if (lane == 0) z[e] = acc + bias[e];
    }
    __syncthreads();
    if (warp != 0) return;
    float zmax = 0.f, sum = 0.f, mine = 0.f;   // lane k keeps the k-th chosen logit (top <= 32)
    for (int k = 0; k < p.top; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < p.experts; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; bi = e; }   // ascending e: the lower index wins a tie inside a lane
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;             // only with non-finite logits
        if (k == 0) zmax = best;
        if (lane == k) mine = best;
        if (lane == 0) { idx[(int64_t) t * p.top + k] = bi; z[bi] = -INFINITY; }
        __syncwarp();
    }
    const float pe = lane < p.top ? expf(mine - zmax) : 0.f;
    sum = wsum(pe);
    if (lane < p.top) wt[(int64_t) t * p.top + lane] = pe / sum;
}

// warp arg-max over v[0..n) in shared memory (ties: the lower index); every lane gets (value, index); index 0x7fffffff if nothing is finite
__device__ __forceinline__ void warp_argmax(const float * v, int n, int lane, float & best, int & bi) {
    best = -INFINITY;
    bi = 0x7fffffff;
    for (int e = lane; e < n; e += 32) {
        const float c = v[e];
        if (c > best) { best = c; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
}

// one CTA per token: sigmoid scores, choice with the correction among the experts of the best groups, weights from the plain scores
template <typename HT>
__global__ void __launch_bounds__(1024) k_moe_route_sigmoid(const HT * __restrict__ h, const float * __restrict__ wr, const float * __restrict__ corr, MoeParams p,
                                                           int width, const float * __restrict__ sgw, int32_t * __restrict__ idx, float * __restrict__ wt,
                                                           float * __restrict__ sg_out) {
    extern __shared__ float sm[];
    float * hs = sm;                 // [width]
    float * sc = hs + width;         // [experts] sigmoid scores
    float * ch = sc + p.experts;     // [experts] choice scores, -inf once taken or not eligible
    float * gs = ch + p.experts;     // [groups] group scores
    float * kp = gs + p.groups;      // [groups] 1: the group stays eligible
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += blockDim.x) hs[i] = ld_f(h, (int64_t) t * width + i);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int e = warp; e < p.experts + (sgw ? 1 : 0); e += nw) {
        if (e == p.experts) {        // the shared expert's gate rides along as one more row
            const float acc = wsum(dot_lane8(sgw, hs, width, lane));
            if (lane == 0) sg_out[t] = sigmoid_f(acc);
        } else {
            const float acc = wsum(dot_lane8(wr + (int64_t) e * width, hs, width, lane));
            if (lane == 0) { const float s = sigmoid_f(acc); sc[e] = s; ch[e] = corr ? s + corr[e] : s; }
        }
    }
    __syncthreads();
    if (warp != 0) return;
    const int per = p.experts / p.groups;
    if (p.groups > 1 && p.keep_groups < p.groups) {
        for (int g = lane; g < p.groups; g += 32) {   // the two largest choice scores of the group, summed
            float a = -INFINITY, b = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; e++) {
                const float c = ch[e];
                if (c > a) { b = a; a = c; } else if (c > b) b = c;
            }
            gs[g] = per > 1 ? a + b : a;
            kp[g] = 0.f;
        }
        __syncwarp();
        // the keep_groups best groups stay (ties: the lower index); the others lose their experts
        for (int k = 0; k < p.keep_groups; k++) {
            float best; int bi;
            warp_argmax(gs, p.groups, lane, best, bi);
            if (bi == 0x7fffffff) break;
            if (lane == 0) { gs[bi] = -INFINITY; kp[bi] = 1.f; }
            __syncwarp();
        }
        for (int g = 0; g < p.groups; g++)
            if (kp[g] == 0.f)
                for (int e = g * per + lane; e < (g + 1) * per; e += 32) ch[e] = -INFINITY;
        __syncwarp();
    }
    float mine = 0.f;   // lane k keeps the score of the k-th chosen expert (top <= 32)
    for (int k = 0; k < p.top; k++) {
        float best; int bi;
        warp_argmax(ch, p.experts, lane, best, bi);
        if (bi == 0x7fffffff) bi = 0;             // only with non-finite scores
        if (lane == k) mine = sc[bi];
        if (lane == 0) { idx[(int64_t) t * p.top + k] = bi; ch[bi] = -INFINITY; }
        __syncwarp();
    }
    const float sum = wsum(lane < p.top ? mine : 0.f);
    if (lane < p.top) wt[(int64_t) t * p.top + lane] = (p.norm_weights ? mine / (sum + 1e-20f) : mine) * p.route_scale;
}

// grid (ceil(ff / 8), pairs): warp -> row j of gate and of up of the pair's expert
template <typename WT, bool VEC>
__global__ void __launch_bounds__(256) k_moe_gateup_rows(const WT * __restrict__ h, const WT * __restrict__ gateup, const int32_t * __restrict__ idx, MoeParams p,
                                                         int width, WT * __restrict__ y, const float * __restrict__ in_wt) {
    const int pair = blockIdx.y, t = pair / p.top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * 8 + warp;
    if (j >= p.ff) return;
    const WT * we = gateup + (int64_t) idx[pair] * moe_up_rows(p) * width;
    const WT * a = h + (int64_t) t * width;
    float g = dot_part<WT, VEC>(we + (int64_t) j * width, a, width, lane);
    if (p.act == 1) {   // squared ReLU of the only row
        g = fmaxf(wsum(g), 0.f);
        if (lane == 0) put(y, (int64_t) pair * p.ff + j, g * g);
        return;
    }
    float u = dot_part<WT, VEC>(we + (int64_t) (p.ff + j) * width, a, width, lane);
    g = wsum(g);
    u = wsum(u);
    if (lane == 0) {
        if (in_wt) { g *= in_wt[pair]; u *= in_wt[pair]; }   // the weight on the expert's input, applied to the products that are linear in it
        if (p.act == 2) {
            put(y, (int64_t) pair * p.ff + j, silu_f(g) * u);
        } else {
            g = fminf(g, p.limit);
            u = fminf(fmaxf(u, -p.limit), p.limit);
            put(y, (int64_t) pair * p.ff + j, g * sigmoid_f(1.702f * g) * (u + 1.f));
        }
    }
}
// grid (ceil(width / 8), tokens): warp -> output n of the token, summed over its experts in the order of the choice
template <typename WT, bool VEC>
__global__ void __launch_bounds__(256) k_moe_down_rows(const WT * __restrict__ y, const WT * __restrict__ down, const int32_t * __restrict__ idx,
                                                       const float * __restrict__ wt, MoeParams p, int width, float * __restrict__ x, int base,
                                                       const float * __restrict__ xscale, float out_scale) {
    const int t = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= width) return;
    float acc = 0.f;
    for (int k = 0; k < p.top; k++) {
        const int pair = t * p.top + k;
        const WT * w = down + ((int64_t) idx[pair] * width + n) * p.ff;
        const float d = wsum(dot_part<WT, VEC>(w, y + (int64_t) pair * p.ff, p.ff, lane));
        acc = wt ? fmaf(wt[pair], d, acc) : acc + d;
    }
    if (lane == 0) {
        float * xo = x + (int64_t) t * width + n;
        *xo = (base == MOE_SET ? 0.f : base == MOE_SCALE ? *xo * xscale[t] : *xo) + acc * out_scale;
    }
}

// ---- sort by expert ----
__global__ void __launch_bounds__(256) k_moe_count(const int32_t * __restrict__ idx, int n_pairs, int32_t * __restrict__ count) {
    __shared__ float red[33];
    const int e = blockIdx.x;
    int c = 0;
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) c += idx[i] == e;
    const float s = block_sum((float) c, red);   // exact below 2^24 pairs
    if (threadIdx.x == 0) count[e] = (int32_t) s;
}
// one CTA per expert: walks the pairs in order, 256 at a time, and places its own at start[e] + rank (stable)
__global__ void __launch_bounds__(256) k_moe_place(const int32_t * __restrict__ idx, int n_pairs, const int32_t * __restrict__ count, int32_t * __restrict__ start,
                                                   int32_t * __restrict__ perm) {
    __shared__ int wbase[9];
    const int e = blockIdx.x;
    int s0 = 0;
    for (int k = 0; k < e; k++) s0 += count[k];
    if (threadIdx.x == 0) start[e] = s0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int placed = 0;
    for (int i0 = 0; i0 < n_pairs; i0 += 256) {
        const int i = i0 + threadIdx.x;
        const bool hit = i < n_pairs && idx[i] == e;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        __syncthreads();
        if (lane == 0) wbase[warp] = __popc(m);
        __syncthreads();
        if (threadIdx.x == 0) {
            int a = 0;
            for (int w = 0; w < 8; w++) { const int c = wbase[w]; wbase[w] = a; a += c; }
            wbase[8] = a;
        }
        __syncthreads();
        if (hit) perm[s0 + placed + wbase[warp] + __popc(m & ((1u << lane) - 1u))] = i;
        placed += wbase[8];
    }
}
template <typename WT>
__global__ void k_moe_gather(const WT * __restrict__ h, const int32_t * __restrict__ perm, int top, int width, WT * __restrict__ hs) {
    const int r = blockIdx.x;
    const WT * src = h + (int64_t) (perm[r] / top) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) hs[(int64_t) r * width + i] = src[i];
}
__global__ void k_moe_invert(const int32_t * __restrict__ perm, int32_t * __restrict__ row_of, int n_pairs) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n_pairs) row_of[perm[r]] = r;
}
__global__ void k_moe_combine(const float * __restrict__ ds, const int32_t * __restrict__ row_of, const float * __restrict__ wt, int top, int width,
                              float * __restrict__ x, int base, const float * __restrict__ xscale, float out_scale) {
    const int t = blockIdx.x;
    for (int n = threadIdx.x; n < width; n += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; k++) {
            const float d = ds[(int64_t) row_of[(int64_t) t * top + k] * width + n];
            acc = wt ? fmaf(wt[(int64_t) t * top + k], d, acc) : acc + d;
        }
        float * xo = x + (int64_t) t * width + n;
        *xo = (base == MOE_SET ? 0.f : base == MOE_SCALE ? *xo * xscale[t] : *xo) + acc * out_scale;
    }
}

template <typename OT>
__global__ void k_silu_mul(const float * __restrict__ gu, OT * __restrict__ y, int n_rows, int ff, const float * __restrict__ in_wt, const int32_t * __restrict__ perm) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t) n_rows * ff) return;
    const int64_t r = i / ff, j = i - r * ff;
    const float s = in_wt ? in_wt[perm ? perm[r] : r] : 1.f;
    put(y, i, silu_f(s * gu[r * 2 * ff + j]) * (s * gu[r * 2 * ff + ff + j]));
}

template <typename WT> bool vec_ok(const void * a, const void * b, int K) {
    return K % Pack<WT>::n == 0 && ((uintptr_t) a & 15) == 0 && ((uintptr_t) b & 15) == 0;
}

}  // namespace

static bool moe_ok(const MoeParams & p) { return p.experts > 0 && p.top > 0 && p.top <= p.experts && p.top <= 32 && p.ff > 0; }

int launch_moe_route(const void * h, int htype, const float * wr, const float * bias, const MoeParams & p, int width, int32_t * idx, float * wt, int n_tokens,
                     cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (!moe_ok(p)) return (int) cudaErrorInvalidValue;
    const size_t smem = ((size_t) width + p.experts) * sizeof(float);
    if (htype == T_BF16) {
        int rc = raise_smem(k_moe_route<__nv_bfloat16>, smem);
        if (rc) return rc;
        return ck_launch([&] { k_moe_route<__nv_bfloat16><<<n_tokens, 256, smem, st>>>((const __nv_bfloat16 *) h, wr, bias, p, width, idx, wt); });
    }
    int rc = raise_smem(k_moe_route<float>, smem);
    if (rc) return rc;
    return ck_launch([&] { k_moe_route<float><<<n_tokens, 256, smem, st>>>((const float *) h, wr, bias, p, width, idx, wt); });
}
int launch_moe_route_sigmoid(const void * h, int htype, const float * wr, const float * correction, const MoeParams & p, int width, const float * shared_gate,
                             int32_t * idx, float * wt, float * sg_out, int n_tokens, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (!moe_ok(p) || p.groups <= 0 || p.experts % p.groups || p.keep_groups <= 0 || p.keep_groups > p.groups || (shared_gate && !sg_out) ||
        (int64_t) p.keep_groups * (p.experts / p.groups) < p.top)
        return (int) cudaErrorInvalidValue;
    const size_t smem = ((size_t) width + 2 * (size_t) p.experts + 2 * (size_t) p.groups) * sizeof(float);
    // one warp per router row (the shared gate included) up to 32 warps, so that all rows stream at once
    const int rows = p.experts + (shared_gate ? 1 : 0);
    const int threads = rows <= 8 ? 256 : rows >= 32 ? 1024 : 32 * rows;
    if (htype == T_BF16) {
        int rc = raise_smem(k_moe_route_sigmoid<__nv_bfloat16>, smem);
        if (rc) return rc;
        return ck_launch([&] {
            k_moe_route_sigmoid<__nv_bfloat16><<<n_tokens, threads, smem, st>>>((const __nv_bfloat16 *) h, wr, correction, p, width, shared_gate, idx, wt, sg_out);
        });
    }
    int rc = raise_smem(k_moe_route_sigmoid<float>, smem);
    if (rc) return rc;
    return ck_launch([&] { k_moe_route_sigmoid<float><<<n_tokens, threads, smem, st>>>((const float *) h, wr, correction, p, width, shared_gate, idx, wt, sg_out); });
}
int launch_silu_mul(const float * gu, void * y, int otype, int n_rows, int ff, const float * in_wt, const int32_t * perm, cudaStream_t st) {
    const int64_t n = (int64_t) n_rows * ff;
    if (n <= 0) return 0;
    const unsigned grid = (unsigned) ((n + 255) / 256);
    return ck_launch([&] {
        if (otype == T_BF16) k_silu_mul<__nv_bfloat16><<<grid, 256, 0, st>>>(gu, (__nv_bfloat16 *) y, n_rows, ff, in_wt, perm);
        else k_silu_mul<float><<<grid, 256, 0, st>>>(gu, (float *) y, n_rows, ff, in_wt, perm);
    });
}
int launch_moe_gateup_rows(const void * h, int type, const void * gateup, const int32_t * idx, const MoeParams & p, int width, void * y, int n_tokens,
                           cudaStream_t st, const float * in_wt) {
    if (n_tokens <= 0) return 0;
    if (!moe_ok(p)) return (int) cudaErrorInvalidValue;
    const dim3 grid((unsigned) ((p.ff + 7) / 8), (unsigned) (n_tokens * p.top));
    return ck_launch([&] {
        if (type == T_BF16) {
            using B = __nv_bfloat16;
            if (vec_ok<B>(h, gateup, width)) k_moe_gateup_rows<B, true><<<grid, 256, 0, st>>>((const B *) h, (const B *) gateup, idx, p, width, (B *) y, in_wt);
            else k_moe_gateup_rows<B, false><<<grid, 256, 0, st>>>((const B *) h, (const B *) gateup, idx, p, width, (B *) y, in_wt);
        } else {
            if (vec_ok<float>(h, gateup, width)) k_moe_gateup_rows<float, true><<<grid, 256, 0, st>>>((const float *) h, (const float *) gateup, idx, p, width, (float *) y, in_wt);
            else k_moe_gateup_rows<float, false><<<grid, 256, 0, st>>>((const float *) h, (const float *) gateup, idx, p, width, (float *) y, in_wt);
        }
    });
}
int launch_moe_down_rows(const void * y, int type, const void * down, const int32_t * idx, const float * wt, const MoeParams & p, int width, float * x,
                         int n_tokens, cudaStream_t st, int base, const float * xscale, float out_scale) {
    if (n_tokens <= 0) return 0;
    if (!moe_ok(p) || (base == MOE_SCALE && !xscale)) return (int) cudaErrorInvalidValue;
    const dim3 grid((unsigned) ((width + 7) / 8), (unsigned) n_tokens);
    return ck_launch([&] {
        if (type == T_BF16) {
            using B = __nv_bfloat16;
            if (vec_ok<B>(y, down, p.ff)) k_moe_down_rows<B, true><<<grid, 256, 0, st>>>((const B *) y, (const B *) down, idx, wt, p, width, x, base, xscale, out_scale);
            else k_moe_down_rows<B, false><<<grid, 256, 0, st>>>((const B *) y, (const B *) down, idx, wt, p, width, x, base, xscale, out_scale);
        } else {
            if (vec_ok<float>(y, down, p.ff)) k_moe_down_rows<float, true><<<grid, 256, 0, st>>>((const float *) y, (const float *) down, idx, wt, p, width, x, base, xscale, out_scale);
            else k_moe_down_rows<float, false><<<grid, 256, 0, st>>>((const float *) y, (const float *) down, idx, wt, p, width, x, base, xscale, out_scale);
        }
    });
}
int launch_moe_sort(const int32_t * idx, const MoeParams & p, int n_tokens, int32_t * count, int32_t * start, int32_t * perm, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (!moe_ok(p) || (int64_t) n_tokens * p.top >= (1 << 24)) return (int) cudaErrorInvalidValue;
    const int n_pairs = n_tokens * p.top;
    int rc = ck_launch([&] { k_moe_count<<<p.experts, 256, 0, st>>>(idx, n_pairs, count); });
    if (rc) return rc;
    return ck_launch([&] { k_moe_place<<<p.experts, 256, 0, st>>>(idx, n_pairs, count, start, perm); });
}
int launch_moe_gather(const void * h, int type, const int32_t * perm, int top, int width, void * hs, int n_rows, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    return ck_launch([&] {
        if (type == T_BF16) k_moe_gather<__nv_bfloat16><<<n_rows, 128, 0, st>>>((const __nv_bfloat16 *) h, perm, top, width, (__nv_bfloat16 *) hs);
        else k_moe_gather<float><<<n_rows, 128, 0, st>>>((const float *) h, perm, top, width, (float *) hs);
    });
}
int launch_moe_combine(const float * ds, const int32_t * perm, int32_t * row_of, const float * wt, int top, int width, float * x, int n_tokens,
                       cudaStream_t st, int base, const float * xscale, float out_scale) {
    if (n_tokens <= 0) return 0;
    if (base == MOE_SCALE && !xscale) return (int) cudaErrorInvalidValue;
    const int n_pairs = n_tokens * top;
    int rc = ck_launch([&] { k_moe_invert<<<(unsigned) ((n_pairs + 255) / 256), 256, 0, st>>>(perm, row_of, n_pairs); });
    if (rc) return rc;
    return ck_launch([&] { k_moe_combine<<<n_tokens, 256, 0, st>>>(ds, row_of, wt, top, width, x, base, xscale, out_scale); });
}

}  // namespace pb
