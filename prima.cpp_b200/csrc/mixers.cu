// prima.cpp_b200/csrc/mixers.cu — sequence mixers, norms and element-wise steps of the layer-list engine (declarations and the
// semantics of every launcher: layers.h).  Everything here runs in fp32: scores, soft-cap, softmax weights, norms, the recurrent
// state, decays and step sizes; only the value written for a following dense product is rounded to that product's operand type.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdlib.h>

#include <algorithm>
#include <atomic>

#include "layers.h"
#include "mixers.cuh"

namespace pb {
namespace {

// ---------------------------------------------------------------------------------------------------------------
template <typename WT>
__global__ void k_embed(const WT * __restrict__ table, int width, const int32_t * __restrict__ tokens, float * __restrict__ x, float * __restrict__ x2) {
    const int t = blockIdx.x;
    const WT * row = table + (int64_t) tokens[t] * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v;
        if constexpr (sizeof(WT) == 2) v = __bfloat162float(row[i]); else v = row[i];
        x[(int64_t) t * width + i] = v;
        if (x2) x2[(int64_t) t * width + i] = v;
    }
}

template <typename OT>
__global__ void k_cast(const float * __restrict__ x, OT * __restrict__ y, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) put(y, i, x[i]);
}

// layer norm with a weight and an optional bias; two passes over the row (mean, then the mean of squared deviations)
template <typename OT, bool RESID>
__global__ void __launch_bounds__(256) k_layernorm(const float * __restrict__ x, const int32_t * __restrict__ rows, const float * __restrict__ w,
                                                   const float * __restrict__ bias, float eps, OT * __restrict__ y, float * __restrict__ xres, int width) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const float * in = x + (int64_t) (rows ? rows[r] : r) * width;
    float s = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) s += in[i];
    const float mean = block_sum(s, red) / (float) width;
    float q = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = in[i] - mean; q = fmaf(d, d, q); }
    const float var = block_sum(q, red) / (float) width;
    const float inv = 1.f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = (in[i] - mean) * inv * w[i] + (bias ? bias[i] : 0.f);
        if constexpr (RESID) xres[(int64_t) r * width + i] += v;
        else put(y, (int64_t) r * width + i, v);
    }
}

// x[t] += layernorm(m[t]) * wa, then y[t] = layernorm(x[t]) * wb: the post-norm + residual of one sublayer and the pre-norm of the next in
// one pass over the token (every thread re-reads only the elements of x it has written itself)
template <typename OT>
__global__ void __launch_bounds__(256) k_layernorm_residual_next(const float * __restrict__ m, const float * __restrict__ wa, const float * __restrict__ wb,
                                                                 float eps, float * __restrict__ x, OT * __restrict__ y, int width) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const float * in = m + (int64_t) r * width;
    float * xr = x + (int64_t) r * width;
    float s = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) s += in[i];
    const float mean = block_sum(s, red) / (float) width;
    float q = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = in[i] - mean; q = fmaf(d, d, q); }
    const float inv = 1.f / sqrtf(block_sum(q, red) / (float) width + eps);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i] + (in[i] - mean) * inv * wa[i];
        xr[i] = v;
        s2 += v;
    }
    const float mean2 = block_sum(s2, red) / (float) width;
    float q2 = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = xr[i] - mean2; q2 = fmaf(d, d, q2); }
    const float inv2 = 1.f / sqrtf(block_sum(q2, red) / (float) width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) put(y, (int64_t) r * width + i, (xr[i] - mean2) * inv2 * wb[i]);
}

// x[t] += mult * (layernorm(m[t]) * w + bias); xa[t] = x[t] in the operand type.  The row of m is kept in registers (width <= 256 * LNR)
// or re-read; x is read and written once.
template <typename OT>
__global__ void __launch_bounds__(256) k_layernorm_affine_residual(const float * __restrict__ m, const float * __restrict__ w, const float * __restrict__ bias,
                                                                   float mult, float eps, float * __restrict__ x, OT * __restrict__ xa, int width) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const float * in = m + (int64_t) r * width;
    float * xr = x + (int64_t) r * width;
    float s = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) s += in[i];
    const float mean = block_sum(s, red) / (float) width;
    float q = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = in[i] - mean; q = fmaf(d, d, q); }
    const float inv = 1.f / sqrtf(block_sum(q, red) / (float) width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i] + mult * ((in[i] - mean) * inv * w[i] + (bias ? bias[i] : 0.f));
        xr[i] = v;
        if (xa) put(xa, (int64_t) r * width + i, v);
    }
}

template <typename OT>
__global__ void k_relu2(const float * __restrict__ u, OT * __restrict__ y, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = fmaxf(u[i], 0.f);
    put(y, i, v * v);
}
__global__ void k_softcap(float * __restrict__ x, int64_t n, float cap) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// x[t] = table[token] + pos_table[position]; positions count from the entry's pos0
template <typename WT, typename OT>
__global__ void k_embed_pos(const WT * __restrict__ table, const WT * __restrict__ ptab, int width, const int32_t * __restrict__ tokens,
                            const int32_t * __restrict__ off, const int32_t * __restrict__ pos0, const int32_t * __restrict__ entry_of, float * __restrict__ x,
                            OT * __restrict__ xa) {
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int64_t p = pos0[e] + (t - off[e]);
    const WT * row = table + (int64_t) tokens[t] * width;
    const WT * prow = ptab + p * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = ld_f(row, i) + ld_f(prow, i);
        x[(int64_t) t * width + i] = v;
        if (xa) put(xa, (int64_t) t * width + i, v);
    }
}

template <typename OT>
__global__ void k_gelu_mul(const float * __restrict__ gu, OT * __restrict__ y, int n_tokens, int ff) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t) n_tokens * ff) return;
    const int64_t t = i / ff, j = i - t * ff;
    const float g = gu[t * 2 * ff + j], u = gu[t * 2 * ff + ff + j];
    const float act = 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    put(y, i, act * u);
}

// first index of the row's maximum: one CTA per row, every thread walks its elements in ascending order (16-byte loads when the row allows)
__global__ void __launch_bounds__(1024) k_argmax_rows(const float * __restrict__ x, int n, int32_t * __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float * row = x + (int64_t) blockIdx.x * n;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    if ((n & 3) == 0 && ((uintptr_t) row & 15) == 0) {
        const float4 * r4 = reinterpret_cast<const float4 *>(row);
        for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
            const float4 v = r4[i];
            if (v.x > best) { best = v.x; bi = 4 * i; }
            if (v.y > best) { best = v.y; bi = 4 * i + 1; }
            if (v.z > best) { best = v.z; bi = 4 * i + 2; }
            if (v.w > best) { best = v.w; bi = 4 * i + 3; }
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = row[i];
            if (v > best) { best = v; bi = i; }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < (int) (blockDim.x >> 5); k++)
            if (sv[k] > best || (sv[k] == best && si[k] < bi)) { best = sv[k]; bi = si[k]; }
        out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// attention.  Cache row of position p: p itself below keep_first, else keep_first + (p - keep_first) mod ring.
__device__ __forceinline__ int cache_row(int p, int keep_first, int ring) { return p < keep_first ? p : keep_first + (p - keep_first) % ring; }

// key element d of (token row, kv head): the head's own part, then the part all heads share
__device__ __forceinline__ float attn_key(const AttnIO & io, int64_t row, int kvh, int d, int DN) {
    return d < DN ? io.k[row * io.ldk + (int64_t) kvh * DN + d] : io.ks[row * io.ldks + (d - DN)];
}
// factor on output element d of head h: sigmoid of a gate logit per head, per element, or none
__device__ __forceinline__ float attn_gate(const AttnIO & io, int64_t row, int h, int d, int DV) {
    if (io.gate_mode == 1) return sigmoid_f(io.gate[row * io.ldg + h]);
    if (io.gate_mode == 2) return sigmoid_f(io.gate[row * io.ldg + (int64_t) h * DV + d]);
    return 1.f;
}

__global__ void k_attn_kv_store(const float * __restrict__ qkvg, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                const int32_t * __restrict__ pos0, const int32_t * __restrict__ entry_of, AttnParams a, float * __restrict__ kcache,
                                float * __restrict__ vcache, int64_t slot_stride) {
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int n = off[e + 1] - off[e];
    const int p = pos0[e] + (t - off[e]), pend = pos0[e] + n;
    const int keep = min(a.keep_first, a.cache_rows), ring = a.cache_rows - keep;
    // of the positions that share a ring row only the last one of this entry is stored
    if (p >= keep && (ring <= 0 || p < pend - ring)) return;
    const int row = cache_row(p, keep, max(ring, 1));
    const int KD = a.kv_heads * a.dim, VD = a.kv_heads * a.vdim, C = attn_qkvg_cols(a);
    const float * src = qkvg + (int64_t) t * C + a.heads * a.dim;
    float * kd = kcache + (int64_t) slot[e] * slot_stride + (int64_t) row * KD;
    float * vd = vcache + (int64_t) slot[e] * slot_stride + (int64_t) row * VD;
    for (int i = threadIdx.x; i < KD; i += blockDim.x) kd[i] = src[i];
    for (int i = threadIdx.x; i < VD; i += blockDim.x) vd[i] = src[KD + i];
}

// One CTA per token.  First every query head and key head of the token's fused projection is divided by its root mean square and
// multiplied by the weight all heads share (one warp per head, in place); then the rows later tokens can still see go to the cache.
__global__ void __launch_bounds__(256) k_attn_qknorm_kv_store(float * __restrict__ qkvg, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                                              const int32_t * __restrict__ pos0, const int32_t * __restrict__ entry_of, AttnParams a,
                                                              const float * __restrict__ wq, const float * __restrict__ wk, float eps,
                                                              float * __restrict__ kcache, float * __restrict__ vcache, int64_t slot_stride) {
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int KD = a.kv_heads * a.dim, VD = a.kv_heads * a.vdim, C = attn_qkvg_cols(a);
    float * row = qkvg + (int64_t) t * C;
    for (int hh = warp; hh < a.heads + a.kv_heads; hh += nw) {
        float * v = row + (int64_t) hh * a.dim;                   // q heads, then k heads, back to back
        const float * w = hh < a.heads ? wq : wk;
        float ss = 0.f;
        for (int i = lane; i < a.dim; i += 32) ss = fmaf(v[i], v[i], ss);
        const float inv = 1.f / sqrtf(wsum(ss) / (float) a.dim + eps);
        for (int i = lane; i < a.dim; i += 32) v[i] = v[i] * inv * w[i];
    }
    __syncthreads();
    const int e = entry_of[t];
    const int n = off[e + 1] - off[e];
    const int p = pos0[e] + (t - off[e]), pend = pos0[e] + n;
    const int keep = min(a.keep_first, a.cache_rows), ring = a.cache_rows - keep;
    if (p >= keep && (ring <= 0 || p < pend - ring)) return;
    const int crow = cache_row(p, keep, max(ring, 1));
    const float * src = row + a.heads * a.dim;
    float * kd = kcache + (int64_t) slot[e] * slot_stride + (int64_t) crow * KD;
    float * vd = vcache + (int64_t) slot[e] * slot_stride + (int64_t) crow * VD;
    for (int i = threadIdx.x; i < KD; i += blockDim.x) kd[i] = src[i];
    for (int i = threadIdx.x; i < VD; i += blockDim.x) vd[i] = src[KD + i];
}

// One warp owns one query row; a CTA of 4 warps shares key / value tiles of 32 positions in shared memory.
// Lane j scores key j of the tile (fp32 dot over dim), the warp keeps a running max / sum (online softmax), then every lane
// accumulates its share of the value dimensions.  NV = ceil(vdim / 32) accumulators per lane.
constexpr int AQ = 4;      // queries per CTA (one per warp)
constexpr int AKT = 32;    // keys per tile

template <int NV>
__device__ __forceinline__ void attn_tile_update(float score, bool valid, const float * __restrict__ vt, int vdim, int lane, float & m, float & l,
                                                 float (&acc)[NV]) {
    const float s = valid ? score : -INFINITY;
    const float tmax = wmax(s);
    if (tmax == -INFINITY) return;   // no visible key in this tile (uniform over the warp)
    const float mn = fmaxf(m, tmax);
    const float corr = m == -INFINITY ? 0.f : expf(m - mn);
    const float p = valid ? expf(s - mn) : 0.f;
    l = l * corr + wsum(p);
#pragma unroll
    for (int c = 0; c < NV; c++) acc[c] *= corr;
    for (int j = 0; j < AKT; j++) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        if (pj != 0.f) {
#pragma unroll
            for (int c = 0; c < NV; c++) {
                const int d = lane + 32 * c;
                if (d < vdim) acc[c] = fmaf(pj, vt[j * vdim + d], acc[c]);
            }
        }
    }
    m = mn;
}

template <typename OT, int NV>
__global__ void __launch_bounds__(AQ * 32) k_attn_window_prefill(const AttnIO io, const int32_t * __restrict__ off, AttnParams a,
                                                                  OT * __restrict__ out) {
    extern __shared__ float sm[];
    const int e = blockIdx.z, h = blockIdx.y;
    const int t_begin = off[e], n = off[e + 1] - t_begin;
    const int q0 = blockIdx.x * AQ;
    if (q0 >= n) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = a.dim, DV = a.vdim, DN = a.dim - a.shared_dim;
    const int kvh = h / (a.heads / a.kv_heads);
    float * qs = sm;                       // [AQ][D]
    float * kt = qs + AQ * D;              // [AKT][D + 1]
    float * vt = kt + AKT * (D + 1);       // [AKT][DV]
    const int qi = q0 + warp;              // this warp's query position (entries handled here start at position 0)
    const bool qok = qi < n;
    for (int d = lane; d < D; d += 32) qs[warp * D + d] = qok ? io.q[(int64_t) (t_begin + qi) * io.ldq + h * D + d] : 0.f;
    const int q_last = min(q0 + AQ, n) - 1;
    const bool windowed = a.window > 0;
    const int w_lo = windowed ? max(0, q0 - a.window + 1) : 0;          // first key any query of the CTA sees through its window
    const int s_hi = windowed ? min(a.keep_first, w_lo) : 0;            // kept first tokens below the window: [0, s_hi)
    float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
    for (int c = 0; c < NV; c++) acc[c] = 0.f;
    // key ranges: the kept first tokens not covered by the window range, then the window range up to the last query
    for (int range = 0; range < 2; range++) {
        const int lo = range == 0 ? 0 : w_lo, hi = range == 0 ? s_hi : q_last + 1;
        for (int k0 = lo; k0 < hi; k0 += AKT) {
            __syncthreads();
            const int nk = min(AKT, hi - k0);
            for (int i = threadIdx.x; i < AKT * D; i += blockDim.x) {
                const int j = i / D, d = i - j * D;
                kt[j * (D + 1) + d] = j < nk ? attn_key(io, t_begin + k0 + j, kvh, d, DN) : 0.f;
            }
            for (int i = threadIdx.x; i < AKT * DV; i += blockDim.x) {
                const int j = i / DV, d = i - j * DV;
                vt[i] = j < nk ? io.v[(int64_t) (t_begin + k0 + j) * io.ldv + kvh * DV + d] : 0.f;
            }
            __syncthreads();
            if (!qok) continue;
            const int kj = k0 + lane;
            bool valid = lane < nk && kj <= qi && (!windowed || qi - kj < a.window || kj < a.keep_first);
            float s = 0.f;
            const float * qr = qs + warp * D, * kr = kt + lane * (D + 1);
            for (int d = 0; d < D; d++) s = fmaf(qr[d], kr[d], s);
            s *= a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            attn_tile_update<NV>(s, valid, vt, DV, lane, m, l, acc);
        }
    }
    if (!qok) return;
    if (a.sink && m != -INFINITY) l += expf(-m);   // the sink: a key of score 0 in the denominator only
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int c = 0; c < NV; c++) {
        const int d = lane + 32 * c;
        if (d < DV) put(out, (int64_t) (t_begin + qi) * (a.heads * DV) + h * DV + d, acc[c] * inv * attn_gate(io, t_begin + qi, h, d, DV));
    }
}

// Prompt attention, register-tiled: a CTA of 256 threads owns 64 queries of one (entry, head) and walks key tiles of 64 positions
// (only tiles some query of the CTA can see: the kept first tokens below the window, then the window up to the diagonal).
// Thread (ty, tx) = (tid / 16, tid % 16) computes the 4 x 4 block of scores of queries 4 ty .. +3 and keys tx, tx + 16, .. (fp32 FMA over
// dim from transposed shared-memory tiles), the 16 threads of a query row agree on the running max / sum by shuffles, the weights go to
// shared memory and every thread accumulates queries 4 ty .. +3 x value columns tx + 16 c.  Everything is fp32.
constexpr int PQ = 64, PK = 64;
__host__ __device__ inline bool attn_tiled_ps_aliased(int dim) { return dim * (PK + 1) >= PQ * (PK + 1); }
inline size_t attn_tiled_smem(int dim, int vdim) {
    return ((size_t) dim * (PQ + 4) + (size_t) dim * (PK + 1) + (size_t) PK * vdim + (attn_tiled_ps_aliased(dim) ? 0 : (size_t) PQ * (PK + 1))) * sizeof(float);
}
template <typename OT, int NVC>
__global__ void __launch_bounds__(256) k_attn_window_prefill_tiled(const AttnIO io, const int32_t * __restrict__ off, AttnParams a,
                                                                   OT * __restrict__ out) {
    extern __shared__ float sm[];
    const int e = blockIdx.z, h = blockIdx.y;
    const int t_begin = off[e], n = off[e + 1] - t_begin;
    const int q0 = blockIdx.x * PQ;
    if (q0 >= n) return;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int D = a.dim, DV = a.vdim, DN = a.dim - a.shared_dim;
    const int kvh = h / (a.heads / a.kv_heads);
    constexpr int PQS = PQ + 4, PKS = PK + 1;   // padded strides: the transposing stores of a tile load spread over the banks
    float * Qt = sm;                    // [D][PQS]  transposed: Qt[d][q]
    float * Kt = Qt + D * PQS;          // [D][PKS]  transposed: Kt[d][k]
    float * Vs = Kt + D * PKS;          // [PK][DV]
    float * Ps = attn_tiled_ps_aliased(D) ? Kt : Vs + PK * DV;   // [PQ][PK + 1]; shares the key tile's memory when that is large enough (two CTAs per SM fit then)
    for (int i = tid; i < PQ * D; i += 256) {
        const int q = i / D, d = i - q * D;
        Qt[d * PQS + q] = q0 + q < n ? io.q[(int64_t) (t_begin + q0 + q) * io.ldq + h * D + d] * a.scale : 0.f;
    }
    const int q_last = min(q0 + PQ, n) - 1;
    const bool windowed = a.window > 0;
    const int w_lo = windowed ? max(0, q0 - a.window + 1) : 0;
    const int s_hi = windowed ? min(a.keep_first, w_lo) : 0;
    float m[4], l[4], acc[4][NVC];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < NVC; c++) acc[i][c] = 0.f;
    }
    for (int range = 0; range < 2; range++) {
        const int lo = range == 0 ? 0 : w_lo, hi = range == 0 ? s_hi : q_last + 1;
        for (int k0 = lo; k0 < hi; k0 += PK) {
            const int nk = min(PK, hi - k0);
            __syncthreads();
            // eight loads per thread in flight before the first store: with one CTA per SM nothing else hides a load's latency
            for (int i0 = tid; i0 < PK * D; i0 += 256 * 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int i = i0 + 256 * u, k = i / D, d = i - k * D;
                    v[u] = (i < PK * D && k < nk) ? attn_key(io, t_begin + k0 + k, kvh, d, DN) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int i = i0 + 256 * u, k = i / D, d = i - k * D;
                    if (i < PK * D) Kt[d * PKS + k] = v[u];
                }
            }
            for (int i0 = tid; i0 < PK * DV; i0 += 256 * 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int i = i0 + 256 * u, k = i / DV, d = i - k * DV;
                    v[u] = (i < PK * DV && k < nk) ? io.v[(int64_t) (t_begin + k0 + k) * io.ldv + kvh * DV + d] : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int i = i0 + 256 * u;
                    if (i < PK * DV) Vs[i] = v[u];
                }
            }
            __syncthreads();
            float s[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) s[i][j] = 0.f;
            for (int d = 0; d < D; d++) {
                const float4 qv = *reinterpret_cast<const float4 *>(Qt + d * PQS + ty * 4);
                float kv[4];
#pragma unroll
                for (int j = 0; j < 4; j++) kv[j] = Kt[d * PKS + tx + 16 * j];
                const float qq[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) s[i][j] = fmaf(qq[i], kv[j], s[i][j]);
            }
            __syncthreads();   // every warp is done with the key tile before the weights overwrite it
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int qi = q0 + ty * 4 + i;
                float tmax = -INFINITY;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int kj = k0 + tx + 16 * j;
                    const bool valid = tx + 16 * j < nk && kj <= qi && (!windowed || qi - kj < a.window || kj < a.keep_first);
                    float v = s[i][j];
                    if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
                    s[i][j] = valid ? v : -INFINITY;
                    tmax = fmaxf(tmax, s[i][j]);
                }
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
                const float mn = fmaxf(m[i], tmax);
                const float corr = (m[i] == -INFINITY || mn == -INFINITY) ? (mn == -INFINITY ? 1.f : 0.f) : expf(m[i] - mn);
                float psum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float pv = s[i][j] == -INFINITY ? 0.f : expf(s[i][j] - mn);
                    Ps[(ty * 4 + i) * (PK + 1) + tx + 16 * j] = pv;
                    psum += pv;
                }
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
                l[i] = l[i] * corr + psum;
#pragma unroll
                for (int c = 0; c < NVC; c++) acc[i][c] *= corr;
                m[i] = mn;
            }
            __syncwarp();   // a query row's weights are written and read by the 16 threads of one half-warp
            for (int k = 0; k < nk; k++) {
                float pv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) pv[i] = Ps[(ty * 4 + i) * (PK + 1) + k];
#pragma unroll
                for (int c = 0; c < NVC; c++) {
                    const int dv = tx + 16 * c;
                    const float vv = dv < DV ? Vs[k * DV + dv] : 0.f;
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[i][c] = fmaf(pv[i], vv, acc[i][c]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int qi = q0 + ty * 4 + i;
        if (qi >= n) continue;
        if (a.sink && m[i] != -INFINITY) l[i] += expf(-m[i]);
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
        for (int c = 0; c < NVC; c++) {
            const int dv = tx + 16 * c;
            if (dv < DV) put(out, (int64_t) (t_begin + qi) * (a.heads * DV) + h * DV + dv, acc[i][c] * inv * attn_gate(io, t_begin + qi, h, dv, DV));
        }
    }
}

// decode: CTA (head, entry, split).  Warp w takes cache rows 4 w .. 4 w + 3 of the split's chunk, then 4 * warps further on, ...: the lanes
// split the key's dimensions (coalesced row reads, four rows in flight), the score is a warp sum, the running max / sum are uniform over the
// warp, and every lane accumulates its share of the value dimensions.  The warps' partial softmax states are merged in shared memory.  With
// one split (32 warps over all rows) the CTA writes the output; with several (8 warps over `chunk` rows each) it writes its partial state
// [max, sum, weighted values] and k_attn_decode_merge finishes.  The number of splits comes from the cache's row count alone (the layer's
// window and the context size), so a sequence's result does not depend on the batch around it.
constexpr int DEC_WARPS = 32, DEC_ROWS = 4, DEC_SPLIT_WARPS = 8;
template <typename OT, int NV>
__global__ void __launch_bounds__(DEC_WARPS * 32) k_attn_window_decode(const AttnIO io, const int32_t * __restrict__ slot,
                                                                       const int32_t * __restrict__ off, const int32_t * __restrict__ pos0, AttnParams a,
                                                                       const float * __restrict__ kcache, const float * __restrict__ vcache,
                                                                       int64_t slot_stride, OT * __restrict__ out, float * __restrict__ part, int chunk) {
    extern __shared__ float sm[];
    const int e = blockIdx.y, h = blockIdx.x;
    const int t = off[e];
    const int pi = pos0[e];               // position of the query (its own K / V row is in the cache already)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = a.dim, DV = a.vdim;
    const int kvh = h / (a.heads / a.kv_heads);
    const int64_t KD = io.k_row, VD = io.v_row;
    const int keep = min(a.keep_first, a.cache_rows), ring = a.cache_rows - keep;
    const int nw = blockDim.x >> 5;
    float * qs = sm;                       // [D], scaled
    float * mm = qs + ((D + 3) & ~3);      // [nw] max, [nw] sum
    float * accs = mm + 2 * nw;            // [nw][NV*32]
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = io.q[(int64_t) t * io.ldq + h * D + d] * a.scale;
    __syncthreads();
    const float * kc = kcache + (int64_t) slot[e] * slot_stride, * vc = vcache + (int64_t) slot[e] * slot_stride;
    float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
    for (int c = 0; c < NV; c++) acc[c] = 0.f;
    const int rows_used = min(a.cache_rows, pi + 1);
    const int r_begin = gridDim.z > 1 ? blockIdx.z * chunk : 0, r_end = gridDim.z > 1 ? min(rows_used, r_begin + chunk) : rows_used;
    const bool vec4 = (D & 3) == 0 && (KD & 3) == 0;
    for (int r0 = r_begin + warp * DEC_ROWS; r0 < r_end; r0 += nw * DEC_ROWS) {
        // DEC_ROWS rows per step so that their loads are in flight together; which position does row r hold right now?
        float sc[DEC_ROWS];
#pragma unroll
        for (int j = 0; j < DEC_ROWS; j++) {
            const int r = r0 + j;
            int p = -1;
            if (r < r_end) {
                if (r < keep) p = r;
                else {
                    const int rr = r - keep, ip = pi - keep;       // ip >= 0 here because r < r_end <= rows_used <= pi + 1
                    p = keep + ip - ((ip - rr) % ring + ring) % ring;
                    if (p < keep) p = -1;
                }
            }
            const bool valid = p >= 0 && p <= pi && (a.window <= 0 || pi - p < a.window || p < a.keep_first);   // uniform over the warp
            float s = 0.f;
            if (valid) {
                const float * kr = kc + (int64_t) r * KD + kvh * D;
                if (vec4) {
                    for (int d = lane * 4; d < D; d += 128) {
                        const float4 kv = *reinterpret_cast<const float4 *>(kr + d);
                        const float4 qv = *reinterpret_cast<const float4 *>(qs + d);
                        s = fmaf(qv.x, kv.x, s); s = fmaf(qv.y, kv.y, s); s = fmaf(qv.z, kv.z, s); s = fmaf(qv.w, kv.w, s);
                    }
                } else {
                    for (int d = lane; d < D; d += 32) s = fmaf(qs[d], kr[d], s);
                }
            }
            sc[j] = valid ? s : -INFINITY;
        }
        float tmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < DEC_ROWS; j++) {
            if (sc[j] != -INFINITY) {                               // uniform: validity does not depend on the lane
                float s = wsum(sc[j]);
                if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
                sc[j] = s;
                tmax = fmaxf(tmax, s);
            }
        }
        if (tmax == -INFINITY) continue;
        const float mn = fmaxf(m, tmax);
        const float corr = m == -INFINITY ? 0.f : expf(m - mn);
        float pj[DEC_ROWS], psum = 0.f;
#pragma unroll
        for (int j = 0; j < DEC_ROWS; j++) { pj[j] = sc[j] == -INFINITY ? 0.f : expf(sc[j] - mn); psum += pj[j]; }
        l = l * corr + psum;
#pragma unroll
        for (int c = 0; c < NV; c++) {
            const int d = lane + 32 * c;
            float v = acc[c] * corr;
#pragma unroll
            for (int j = 0; j < DEC_ROWS; j++)
                if (pj[j] != 0.f && d < DV) v = fmaf(pj[j], vc[(int64_t) (r0 + j) * VD + kvh * DV + d], v);
            acc[c] = v;
        }
        m = mn;
    }
    if (lane == 0) { mm[warp] = m; mm[nw + warp] = l; }
#pragma unroll
    for (int c = 0; c < NV; c++) accs[warp * NV * 32 + c * 32 + lane] = acc[c];
    __syncthreads();
    if (warp == 0) {
        float M = -INFINITY;
        for (int w = 0; w < nw; w++) M = fmaxf(M, mm[w]);
        float L = 0.f, o[NV];
#pragma unroll
        for (int c = 0; c < NV; c++) o[c] = 0.f;
        for (int w = 0; w < nw; w++) {
            if (mm[w] == -INFINITY) continue;
            const float f = expf(mm[w] - M);
            L += mm[nw + w] * f;
#pragma unroll
            for (int c = 0; c < NV; c++) o[c] = fmaf(accs[w * NV * 32 + c * 32 + lane], f, o[c]);
        }
        if (gridDim.z > 1) {   // partial state of this split
            float * pp = part + (((int64_t) e * a.heads + h) * gridDim.z + blockIdx.z) * (DV + 2);
            if (lane == 0) { pp[0] = M; pp[1] = L; }
#pragma unroll
            for (int c = 0; c < NV; c++) {
                const int d = lane + 32 * c;
                if (d < DV) pp[2 + d] = o[c];
            }
            return;
        }
        if (a.sink && M != -INFINITY) L += expf(-M);
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
        for (int c = 0; c < NV; c++) {
            const int d = lane + 32 * c;
            if (d < DV) put(out, (int64_t) t * (a.heads * DV) + h * DV + d, o[c] * inv * attn_gate(io, t, h, d, DV));
        }
    }
}

// merges the partial softmax states of a (head, entry): grid (heads, entries), one thread per value dimension
template <typename OT>
__global__ void __launch_bounds__(128) k_attn_decode_merge(const AttnIO io, const int32_t * __restrict__ off, AttnParams a, const float * __restrict__ part,
                                                           int splits, OT * __restrict__ out) {
    const int e = blockIdx.y, h = blockIdx.x, DV = a.vdim;
    const int t = off[e];
    const float * pp = part + ((int64_t) e * a.heads + h) * splits * (DV + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; s++) M = fmaxf(M, pp[(int64_t) s * (DV + 2)]);
    float L = 0.f;
    for (int s = 0; s < splits; s++) {
        const float ms = pp[(int64_t) s * (DV + 2)];
        if (ms != -INFINITY) L += pp[(int64_t) s * (DV + 2) + 1] * expf(ms - M);
    }
    if (a.sink && M != -INFINITY) L += expf(-M);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = threadIdx.x; d < DV; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; s++) {
            const float ms = pp[(int64_t) s * (DV + 2)];
            if (ms != -INFINITY) o = fmaf(pp[(int64_t) s * (DV + 2) + 2 + d], expf(ms - M), o);
        }
        put(out, (int64_t) t * (a.heads * DV) + h * DV + d, o * inv * attn_gate(io, t, h, d, DV));
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Mamba-2
__global__ void k_mamba2_conv(const float * __restrict__ u, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                              const int32_t * __restrict__ entry_of, Mamba2Params p, const float * __restrict__ w, const float * __restrict__ bias,
                              const float * __restrict__ conv_state, int64_t slot_stride, float * __restrict__ xbc) {
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int lt = t - off[e];
    const int CH = mamba2_conv_channels(p), U = mamba2_in_cols(p), inner = mamba2_inner(p), taps = p.conv;
    const float * st = conv_state + (int64_t) slot[e] * slot_stride;   // [taps-1][CH], row taps-2 = the input just before this entry
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < CH; c += gridDim.y * blockDim.x) {
        float acc = bias[c];
        for (int d = 0; d < taps; d++) {
            const int l2 = lt - d;
            const float in = l2 >= 0 ? u[(int64_t) (t - d) * U + inner + c] : st[(int64_t) (taps - 1 + l2) * CH + c];
            acc = fmaf(w[(int64_t) c * taps + (taps - 1 - d)], in, acc);
        }
        xbc[(int64_t) t * CH + c] = silu_f(acc);
    }
}
__global__ void k_mamba2_conv_state(const float * __restrict__ u, const int32_t * __restrict__ slot, const int32_t * __restrict__ off, Mamba2Params p,
                                    float * __restrict__ conv_state, int64_t slot_stride) {
    const int e = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int CH = mamba2_conv_channels(p), U = mamba2_in_cols(p), inner = mamba2_inner(p), taps = p.conv;
    if (c >= CH) return;
    const int n = off[e + 1] - off[e];
    float * st = conv_state + (int64_t) slot[e] * slot_stride;
    for (int k = 0; k < taps - 1; k++) {     // ascending: row k + n is read before a later iteration overwrites it
        const int l2 = n - (taps - 1) + k;   // index within the entry of the input that becomes state row k
        st[(int64_t) k * CH + c] = l2 >= 0 ? u[(int64_t) (off[e] + l2) * U + inner + c] : st[(int64_t) (k + n) * CH + c];
    }
}

// one CTA per (head, entry); the state S [N][P] lives in shared memory for the whole entry, tokens are walked in order
__global__ void __launch_bounds__(256) k_mamba2_scan(const float * __restrict__ u, const float * __restrict__ xbc, const int32_t * __restrict__ slot,
                                                     const int32_t * __restrict__ off, Mamba2Params p, const float * __restrict__ dt_bias,
                                                     const float * __restrict__ A_log, const float * __restrict__ Dp, float * __restrict__ ssm_state,
                                                     int64_t slot_stride, float * __restrict__ y) {
    extern __shared__ float sm[];
    const int h = blockIdx.x, e = blockIdx.y;
    const int N = p.state, P = p.vdim, inner = mamba2_inner(p), CH = mamba2_conv_channels(p), U = mamba2_in_cols(p);
    const int g = h / (p.heads / p.groups);
    float * S = sm;               // [N][P]
    float * Bs = S + N * P;       // [N]
    float * Cs = Bs + N;          // [N]
    float * xs = Cs + N;          // [P]
    float * gst = ssm_state + (int64_t) slot[e] * slot_stride + (int64_t) h * N * P;
    for (int i = threadIdx.x; i < N * P; i += blockDim.x) S[i] = gst[i];
    const float A = -expf(A_log[h]), dtb = dt_bias[h], Dh = Dp[h];
    const int t0 = off[e], n = off[e + 1] - t0;
    for (int lt = 0; lt < n; lt++) {
        const int t = t0 + lt;
        __syncthreads();
        for (int i = threadIdx.x; i < N; i += blockDim.x) {
            Bs[i] = xbc[(int64_t) t * CH + inner + g * N + i];
            Cs[i] = xbc[(int64_t) t * CH + inner + p.groups * N + g * N + i];
        }
        for (int i = threadIdx.x; i < P; i += blockDim.x) xs[i] = xbc[(int64_t) t * CH + h * P + i];
        const float raw = u[(int64_t) t * U + 2 * inner + 2 * p.groups * N + h] + dtb;
        const float dt = raw > 20.f ? raw : log1pf(expf(raw));
        const float decay = expf(A * dt);
        __syncthreads();
        for (int i = threadIdx.x; i < N * P; i += blockDim.x) {
            const int nn = i / P, pp = i - nn * P;
            S[i] = fmaf(decay, S[i], dt * Bs[nn] * xs[pp]);
        }
        __syncthreads();
        for (int pp = threadIdx.x; pp < P; pp += blockDim.x) {
            float acc = 0.f;
            for (int nn = 0; nn < N; nn++) acc = fmaf(S[nn * P + pp], Cs[nn], acc);
            y[(int64_t) t * inner + h * P + pp] = acc + Dh * xs[pp];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < N * P; i += blockDim.x) gst[i] = S[i];
}

// The same recurrence with the state in registers: a CTA of 128 threads owns one head and 32 value columns; thread (pl = tid / 8,
// part ng = tid % 8) keeps S[n][column] for columns pl and pl + 16 and n = ng, ng + 8, ...  (2 x NREG values; a B / C value read from
// shared memory serves both columns).  Tokens are walked in chunks of 16 whose B, C, x rows and
// step sizes / decays are staged in shared memory by the whole CTA (two CTA barriers per chunk, none per token); y needs one 8-lane
// shuffle reduction per token.  Used for state sizes up to 128; larger states take k_mamba2_scan.
constexpr int SCAN_CHUNK = 16, SCAN_COLS = 32;
template <int NREG>
__global__ void __launch_bounds__(128) k_mamba2_scan_reg(const float * __restrict__ u, const float * __restrict__ xbc, const int32_t * __restrict__ slot,
                                                         const int32_t * __restrict__ off, Mamba2Params p, const float * __restrict__ dt_bias,
                                                         const float * __restrict__ A_log, const float * __restrict__ Dp, float * __restrict__ ssm_state,
                                                         int64_t slot_stride, float * __restrict__ y) {
    extern __shared__ float sm[];
    const int N = p.state, P = p.vdim, inner = mamba2_inner(p), CH = mamba2_conv_channels(p), U = mamba2_in_cols(p);
    const int ptiles = (P + SCAN_COLS - 1) / SCAN_COLS;
    const int h = blockIdx.x / ptiles, pt = blockIdx.x - h * ptiles, e = blockIdx.y;
    const int g = h / (p.heads / p.groups);
    const int tid = threadIdx.x, pl = tid >> 3, ng = tid & 7;
    const int pcol = pt * SCAN_COLS + pl, pcol1 = pcol + 16;
    const bool pok = pcol < P, pok1 = pcol1 < P;
    float * Bs = sm;                              // [SCAN_CHUNK][N]
    float * Cs = Bs + SCAN_CHUNK * N;             // [SCAN_CHUNK][N]
    float * xs = Cs + SCAN_CHUNK * N;             // [SCAN_CHUNK][SCAN_COLS]
    float * dts = xs + SCAN_CHUNK * SCAN_COLS;    // [SCAN_CHUNK] step sizes, then [SCAN_CHUNK] decays
    float * gst = ssm_state + (int64_t) slot[e] * slot_stride + (int64_t) h * N * P;
    float S[NREG], S1[NREG];
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int nn = ng + 8 * j;
        S[j] = (pok && nn < N) ? gst[(int64_t) nn * P + pcol] : 0.f;
        S1[j] = (pok1 && nn < N) ? gst[(int64_t) nn * P + pcol1] : 0.f;
    }
    const float A = -expf(A_log[h]), dtb = dt_bias[h], Dh = Dp[h];
    const int t0 = off[e], n = off[e + 1] - t0;
    for (int c0 = 0; c0 < n; c0 += SCAN_CHUNK) {
        const int nc = min(SCAN_CHUNK, n - c0);
        __syncthreads();
        for (int i = tid; i < nc * N; i += 128) {
            const int tt = i / N, nn = i - tt * N;
            const float * row = xbc + (int64_t) (t0 + c0 + tt) * CH + inner + g * N + nn;
            Bs[i] = row[0];
            Cs[i] = row[p.groups * N];
        }
        for (int i = tid; i < nc * SCAN_COLS; i += 128) {
            const int tt = i / SCAN_COLS, pp = i - tt * SCAN_COLS;
            xs[i] = pt * SCAN_COLS + pp < P ? xbc[(int64_t) (t0 + c0 + tt) * CH + h * P + pt * SCAN_COLS + pp] : 0.f;
        }
        if (tid < nc) {
            const float raw = u[(int64_t) (t0 + c0 + tid) * U + 2 * inner + 2 * p.groups * N + h] + dtb;
            const float dt = raw > 20.f ? raw : log1pf(expf(raw));
            dts[tid] = dt;
            dts[SCAN_CHUNK + tid] = expf(A * dt);
        }
        __syncthreads();
        for (int tt = 0; tt < nc; tt++) {
            const float dt = dts[tt], dec = dts[SCAN_CHUNK + tt], xv = xs[tt * SCAN_COLS + pl], xv1 = xs[tt * SCAN_COLS + pl + 16];
            const float dx = dt * xv, dx1 = dt * xv1;
            const float * Br = Bs + tt * N, * Cr = Cs + tt * N;
            float acc = 0.f, acc1 = 0.f;
#pragma unroll
            for (int j = 0; j < NREG; j++) {
                const int nn = ng + 8 * j;
                if (nn < N) {
                    const float bv = Br[nn], cv = Cr[nn];
                    S[j] = fmaf(dec, S[j], dx * bv);
                    S1[j] = fmaf(dec, S1[j], dx1 * bv);
                    acc = fmaf(S[j], cv, acc);
                    acc1 = fmaf(S1[j], cv, acc1);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 4);
            if (ng == 0 && pok) y[(int64_t) (t0 + c0 + tt) * inner + h * P + pcol] = acc + Dh * xv;
            if (ng == 0 && pok1) y[(int64_t) (t0 + c0 + tt) * inner + h * P + pcol1] = acc1 + Dh * xv1;
        }
    }
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int nn = ng + 8 * j;
        if (pok && nn < N) gst[(int64_t) nn * P + pcol] = S[j];
        if (pok1 && nn < N) gst[(int64_t) nn * P + pcol1] = S1[j];
    }
}

template <typename OT>
__global__ void __launch_bounds__(256) k_mamba2_gate_norm(const float * __restrict__ y, const float * __restrict__ u, Mamba2Params p, const float * __restrict__ w,
                                                          float eps, OT * __restrict__ out) {
    __shared__ float red[33];
    const int t = blockIdx.x, grp = blockIdx.y;
    const int inner = mamba2_inner(p), U = mamba2_in_cols(p), part = inner / p.norm_groups;
    const float * yr = y + (int64_t) t * inner + grp * part, * zr = u + (int64_t) t * U + grp * part;
    float q = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) { const float v = yr[i] * silu_f(zr[i]); q = fmaf(v, v, q); }
    const float inv = 1.f / sqrtf(block_sum(q, red) / (float) part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x)
        put(out, (int64_t) t * inner + grp * part + i, yr[i] * silu_f(zr[i]) * inv * w[grp * part + i]);
}

}  // namespace

int launch_embed(const void * table, int type, int width, const int32_t * tokens, int n_tokens, float * x, float * x_copy, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    return ck_launch([&] {
        if (type == T_BF16) k_embed<__nv_bfloat16><<<n_tokens, 128, 0, st>>>((const __nv_bfloat16 *) table, width, tokens, x, x_copy);
        else k_embed<float><<<n_tokens, 128, 0, st>>>((const float *) table, width, tokens, x, x_copy);
    });
}
int launch_cast(const float * x, void * y, int otype, int64_t n, cudaStream_t st) {
    if (n <= 0) return 0;
    const unsigned grid = (unsigned) ((n + 255) / 256);
    return ck_launch([&] {
        if (otype == T_BF16) k_cast<__nv_bfloat16><<<grid, 256, 0, st>>>(x, (__nv_bfloat16 *) y, n);
        else k_cast<float><<<grid, 256, 0, st>>>(x, (float *) y, n);
    });
}
int launch_layernorm(const float * x, const int32_t * rows, const float * w, float eps, void * y, int otype, int n_rows, int width, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    return ck_launch([&] {
        if (otype == T_BF16) k_layernorm<__nv_bfloat16, false><<<n_rows, 256, 0, st>>>(x, rows, w, nullptr, eps, (__nv_bfloat16 *) y, nullptr, width);
        else k_layernorm<float, false><<<n_rows, 256, 0, st>>>(x, rows, w, nullptr, eps, (float *) y, nullptr, width);
    });
}
int launch_layernorm_affine(const float * x, const int32_t * rows, const float * w, const float * bias, float eps, void * y, int otype, int n_rows, int width,
                            cudaStream_t st) {
    if (n_rows <= 0) return 0;
    return ck_launch([&] {
        if (otype == T_BF16) k_layernorm<__nv_bfloat16, false><<<n_rows, 256, 0, st>>>(x, rows, w, bias, eps, (__nv_bfloat16 *) y, nullptr, width);
        else k_layernorm<float, false><<<n_rows, 256, 0, st>>>(x, rows, w, bias, eps, (float *) y, nullptr, width);
    });
}
int launch_layernorm_affine_residual(const float * m, const float * w, const float * bias, float mult, float eps, float * x, void * xa, int otype, int n_rows,
                                     int width, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    return ck_launch([&] {
        if (otype == T_BF16) k_layernorm_affine_residual<__nv_bfloat16><<<n_rows, 256, 0, st>>>(m, w, bias, mult, eps, x, (__nv_bfloat16 *) xa, width);
        else k_layernorm_affine_residual<float><<<n_rows, 256, 0, st>>>(m, w, bias, mult, eps, x, (float *) xa, width);
    });
}
int launch_relu2(const float * u, void * y, int otype, int64_t n, cudaStream_t st) {
    if (n <= 0) return 0;
    const unsigned grid = (unsigned) ((n + 255) / 256);
    return ck_launch([&] {
        if (otype == T_BF16) k_relu2<__nv_bfloat16><<<grid, 256, 0, st>>>(u, (__nv_bfloat16 *) y, n);
        else k_relu2<float><<<grid, 256, 0, st>>>(u, (float *) y, n);
    });
}
int launch_softcap(float * x, int64_t n, float cap, cudaStream_t st) {
    if (n <= 0 || !(cap > 0.f)) return 0;
    return ck_launch([&] { k_softcap<<<(unsigned) ((n + 255) / 256), 256, 0, st>>>(x, n, cap); });
}
int launch_embed_pos(const void * table, const void * pos_table, int type, int width, const int32_t * tokens, const BatchView & b, float * x, void * xa,
                     int otype, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if ((xa && otype != type) || !pos_table) return (int) cudaErrorInvalidValue;
    return ck_launch([&] {
        if (type == T_BF16)
            k_embed_pos<__nv_bfloat16, __nv_bfloat16><<<b.n_tokens, 128, 0, st>>>((const __nv_bfloat16 *) table, (const __nv_bfloat16 *) pos_table, width, tokens,
                                                                                   b.off, b.pos0, b.entry_of, x, (__nv_bfloat16 *) xa);
        else
            k_embed_pos<float, float><<<b.n_tokens, 128, 0, st>>>((const float *) table, (const float *) pos_table, width, tokens, b.off, b.pos0, b.entry_of, x,
                                                                   (float *) xa);
    });
}
int launch_layernorm_residual(const float * m, const float * w, float eps, float * x, int n_rows, int width, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    return ck_launch([&] { k_layernorm<float, true><<<n_rows, 256, 0, st>>>(m, nullptr, w, nullptr, eps, nullptr, x, width); });
}
int launch_layernorm_residual_next(const float * m, const float * wa, const float * wb, float eps, float * x, void * y, int otype, int n_rows, int width,
                                   cudaStream_t st) {
    if (n_rows <= 0) return 0;
    return ck_launch([&] {
        if (otype == T_BF16) k_layernorm_residual_next<__nv_bfloat16><<<n_rows, 256, 0, st>>>(m, wa, wb, eps, x, (__nv_bfloat16 *) y, width);
        else k_layernorm_residual_next<float><<<n_rows, 256, 0, st>>>(m, wa, wb, eps, x, (float *) y, width);
    });
}
int launch_gelu_mul(const float * gu, void * y, int otype, int n_tokens, int ff, cudaStream_t st) {
    const int64_t n = (int64_t) n_tokens * ff;
    if (n <= 0) return 0;
    const unsigned grid = (unsigned) ((n + 255) / 256);
    return ck_launch([&] {
        if (otype == T_BF16) k_gelu_mul<__nv_bfloat16><<<grid, 256, 0, st>>>(gu, (__nv_bfloat16 *) y, n_tokens, ff);
        else k_gelu_mul<float><<<grid, 256, 0, st>>>(gu, (float *) y, n_tokens, ff);
    });
}
int launch_argmax_rows(const float * logits, int n, int n_rows, int32_t * out, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    return ck_launch([&] { k_argmax_rows<<<n_rows, n >= 8192 ? 1024 : 256, 0, st>>>(logits, n, out); });
}

int launch_attn_kv_store(const float * qkvg, const BatchView & b, const AttnParams & a, float * kcache, float * vcache, int64_t slot_stride, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    return ck_launch([&] { k_attn_kv_store<<<b.n_tokens, 128, 0, st>>>(qkvg, b.slot, b.off, b.pos0, b.entry_of, a, kcache, vcache, slot_stride); });
}

int launch_attn_qknorm_kv_store(float * qkvg, const BatchView & b, const AttnParams & a, const float * wq, const float * wk, float eps, float * kcache,
                                float * vcache, int64_t slot_stride, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (!wq || !wk) return (int) cudaErrorInvalidValue;
    return ck_launch([&] {
        k_attn_qknorm_kv_store<<<b.n_tokens, 256, 0, st>>>(qkvg, b.slot, b.off, b.pos0, b.entry_of, a, wq, wk, eps, kcache, vcache, slot_stride);
    });
}

#define PB_NV_DISPATCH(NVV, CALL)                                  \
    do {                                                           \
        if ((NVV) <= 1) { constexpr int NV = 1; CALL; }            \
        else if ((NVV) <= 2) { constexpr int NV = 2; CALL; }       \
        else if ((NVV) <= 4) { constexpr int NV = 4; CALL; }       \
        else if ((NVV) <= 8) { constexpr int NV = 8; CALL; }       \
        else if ((NVV) <= 16) { constexpr int NV = 16; CALL; }     \
        else return (int) cudaErrorInvalidValue;                   \
    } while (0)

template <typename OT, int NVC>
static int attn_prefill_tiled_typed(const AttnIO & io, const BatchView & b, const AttnParams & a, OT * out, cudaStream_t st) {
    const size_t smem = attn_tiled_smem(a.dim, a.vdim);
    int rc = raise_smem(k_attn_window_prefill_tiled<OT, NVC>, smem);
    if (rc) return rc;
    const dim3 grid((unsigned) ((b.max_n + PQ - 1) / PQ), (unsigned) a.heads, (unsigned) b.n_entries);
    return ck_launch([&] { k_attn_window_prefill_tiled<OT, NVC><<<grid, 256, smem, st>>>(io, b.off, a, out); });
}
template <typename OT, int NV>
static int attn_prefill_typed(const AttnIO & io, const BatchView & b, const AttnParams & a, OT * out, cudaStream_t st) {
    const size_t smem = ((size_t) AQ * a.dim + (size_t) AKT * (a.dim + 1) + (size_t) AKT * a.vdim) * sizeof(float);
    int rc = raise_smem(k_attn_window_prefill<OT, NV>, smem);
    if (rc) return rc;
    const dim3 grid((unsigned) ((b.max_n + AQ - 1) / AQ), (unsigned) a.heads, (unsigned) b.n_entries);
    return ck_launch([&] { k_attn_window_prefill<OT, NV><<<grid, AQ * 32, smem, st>>>(io, b.off, a, out); });
}
int launch_attn_prefill_io(const AttnIO & io, const BatchView & b, const AttnParams & a, void * out, int otype, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads != 0 || a.dim <= 0 || a.vdim <= 0 || a.shared_dim < 0 || a.shared_dim > a.dim ||
        (a.shared_dim > 0 && !io.ks))
        return (int) cudaErrorInvalidValue;
    static const bool no_tiled = getenv("PB200_ATTN_ROWWISE") != nullptr;   // A/B: the one-warp-per-query kernel for every length
    const size_t tiled_smem = attn_tiled_smem(a.dim, a.vdim);
    if (b.max_n > 16 && !no_tiled && tiled_smem <= 220 * 1024) {   // long entries: 64-query tiles; the same numbers up to fp32 summation order
        const int nvc = (a.vdim + 15) / 16;
        if (nvc <= 16) {
            if (otype == T_BF16) {
                if (nvc <= 2) return attn_prefill_tiled_typed<__nv_bfloat16, 2>(io, b, a, (__nv_bfloat16 *) out, st);
                if (nvc <= 4) return attn_prefill_tiled_typed<__nv_bfloat16, 4>(io, b, a, (__nv_bfloat16 *) out, st);
                if (nvc <= 8) return attn_prefill_tiled_typed<__nv_bfloat16, 8>(io, b, a, (__nv_bfloat16 *) out, st);
                return attn_prefill_tiled_typed<__nv_bfloat16, 16>(io, b, a, (__nv_bfloat16 *) out, st);
            }
            if (nvc <= 2) return attn_prefill_tiled_typed<float, 2>(io, b, a, (float *) out, st);
            if (nvc <= 4) return attn_prefill_tiled_typed<float, 4>(io, b, a, (float *) out, st);
            if (nvc <= 8) return attn_prefill_tiled_typed<float, 8>(io, b, a, (float *) out, st);
            return attn_prefill_tiled_typed<float, 16>(io, b, a, (float *) out, st);
        }
    }
    const int nv = (a.vdim + 31) / 32;
    if (otype == T_BF16) PB_NV_DISPATCH(nv, return (attn_prefill_typed<__nv_bfloat16, NV>(io, b, a, (__nv_bfloat16 *) out, st)));
    else PB_NV_DISPATCH(nv, return (attn_prefill_typed<float, NV>(io, b, a, (float *) out, st)));
    return 0;
}
template <typename OT, int NV>
static int attn_decode_typed(const AttnIO & io, const BatchView & b, const AttnParams & a, const float * kc, const float * vc, int64_t stride, OT * out,
                             float * part, cudaStream_t st) {
    const int splits = part ? attn_decode_splits(a.cache_rows) : 1;
    const int nw = splits > 1 ? DEC_SPLIT_WARPS : DEC_WARPS;
    const size_t smem = ((size_t) ((a.dim + 3) & ~3) + 2 * nw + (size_t) nw * NV * 32) * sizeof(float);
    int rc = raise_smem(k_attn_window_decode<OT, NV>, ((size_t) ((a.dim + 3) & ~3) + 2 * DEC_WARPS + (size_t) DEC_WARPS * NV * 32) * sizeof(float));
    if (rc) return rc;
    const dim3 grid((unsigned) a.heads, (unsigned) b.n_entries, (unsigned) splits);
    rc = ck_launch([&] {
        k_attn_window_decode<OT, NV><<<grid, nw * 32, smem, st>>>(io, b.slot, b.off, b.pos0, a, kc, vc, stride, out, part, attn_decode_chunk(a.cache_rows));
    });
    if (rc || splits == 1) return rc;
    const dim3 mgrid((unsigned) a.heads, (unsigned) b.n_entries);
    return ck_launch([&] { k_attn_decode_merge<OT><<<mgrid, 128, 0, st>>>(io, b.off, a, part, splits, out); });
}
int launch_attn_decode_io(const AttnIO & io, const BatchView & b, const AttnParams & a, const float * kcache, const float * vcache, int64_t slot_stride,
                          void * out, int otype, cudaStream_t st, float * part) {
    if (b.n_tokens <= 0) return 0;
    if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads != 0 || a.dim <= 0 || a.vdim <= 0) return (int) cudaErrorInvalidValue;
    const int nv = (a.vdim + 31) / 32;
    if (otype == T_BF16) PB_NV_DISPATCH(nv, return (attn_decode_typed<__nv_bfloat16, NV>(io, b, a, kcache, vcache, slot_stride, (__nv_bfloat16 *) out, part, st)));
    else PB_NV_DISPATCH(nv, return (attn_decode_typed<float, NV>(io, b, a, kcache, vcache, slot_stride, (float *) out, part, st)));
    return 0;
}

// the fused q | k | v | gate projection of the windowed-attention mixer as the kernels' inputs
static AttnIO attn_io_fused(const float * qkvg, const AttnParams & a) {
    AttnIO io;
    const int64_t C = attn_qkvg_cols(a);
    io.q = qkvg; io.ldq = C;
    io.k = qkvg + (int64_t) a.heads * a.dim; io.ldk = C;
    io.v = io.k + (int64_t) a.kv_heads * a.dim; io.ldv = C;
    io.gate = io.v + (int64_t) a.kv_heads * a.vdim; io.ldg = C; io.gate_mode = a.gated ? 1 : 0;
    io.k_row = (int64_t) a.kv_heads * a.dim; io.v_row = (int64_t) a.kv_heads * a.vdim;
    return io;
}
int launch_attn_window_prefill(const float * qkvg, const BatchView & b, const AttnParams & a, void * out, int otype, cudaStream_t st) {
    if (a.shared_dim != 0) return (int) cudaErrorInvalidValue;
    return launch_attn_prefill_io(attn_io_fused(qkvg, a), b, a, out, otype, st);
}
int launch_attn_window_decode(const float * qkvg, const BatchView & b, const AttnParams & a, const float * kcache, const float * vcache, int64_t slot_stride,
                              void * out, int otype, cudaStream_t st, float * part) {
    return launch_attn_decode_io(attn_io_fused(qkvg, a), b, a, kcache, vcache, slot_stride, out, otype, st, part);
}

int launch_mamba2_conv(const float * u, const BatchView & b, const Mamba2Params & p, const float * w, const float * bias, float * conv_state,
                       int64_t slot_stride, float * xbc, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (p.conv < 1) return (int) cudaErrorInvalidValue;
    // few tokens (decode): spread the channels of a token over several CTAs
    const int CHn = mamba2_conv_channels(p);
    const dim3 cgrid((unsigned) b.n_tokens, (unsigned) (b.n_tokens >= 64 ? 1 : std::min(16, (CHn + 255) / 256)));
    int rc = ck_launch([&] { k_mamba2_conv<<<cgrid, 256, 0, st>>>(u, b.slot, b.off, b.entry_of, p, w, bias, conv_state, slot_stride, xbc); });
    if (rc || p.conv < 2) return rc;
    const dim3 grid((unsigned) ((mamba2_conv_channels(p) + 127) / 128), (unsigned) b.n_entries);
    return ck_launch([&] { k_mamba2_conv_state<<<grid, 128, 0, st>>>(u, b.slot, b.off, p, conv_state, slot_stride); });
}
int launch_mamba2_scan(const float * u, const float * xbc, const BatchView & b, const Mamba2Params & p, const float * dt_bias, const float * A_log,
                       const float * D, float * ssm_state, int64_t slot_stride, float * y, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (p.heads <= 0 || p.groups <= 0 || p.heads % p.groups != 0) return (int) cudaErrorInvalidValue;
    if (p.state <= 128) {
        const size_t sm2 = ((size_t) 2 * SCAN_CHUNK * p.state + SCAN_CHUNK * SCAN_COLS + 2 * SCAN_CHUNK) * sizeof(float);
        const dim3 grid2((unsigned) (p.heads * ((p.vdim + SCAN_COLS - 1) / SCAN_COLS)), (unsigned) b.n_entries);
        const int nreg = (p.state + 7) / 8;
#define PB_SCAN(NR) return ck_launch([&] { k_mamba2_scan_reg<NR><<<grid2, 128, sm2, st>>>(u, xbc, b.slot, b.off, p, dt_bias, A_log, D, ssm_state, slot_stride, y); })
        if (nreg <= 1) PB_SCAN(1);
        if (nreg <= 2) PB_SCAN(2);
        if (nreg <= 4) PB_SCAN(4);
        if (nreg <= 8) PB_SCAN(8);
        PB_SCAN(16);
#undef PB_SCAN
    }
    const size_t smem = ((size_t) p.state * p.vdim + 2 * (size_t) p.state + p.vdim) * sizeof(float);
    int rc = raise_smem(k_mamba2_scan, smem);
    if (rc) return rc;
    const dim3 grid((unsigned) p.heads, (unsigned) b.n_entries);
    return ck_launch([&] { k_mamba2_scan<<<grid, 256, smem, st>>>(u, xbc, b.slot, b.off, p, dt_bias, A_log, D, ssm_state, slot_stride, y); });
}
int launch_mamba2_gate_norm(const float * y, const float * u, const Mamba2Params & p, const float * w, float eps, void * out, int otype, int n_tokens,
                            cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (p.norm_groups <= 0 || mamba2_inner(p) % p.norm_groups != 0) return (int) cudaErrorInvalidValue;
    const dim3 grid((unsigned) n_tokens, (unsigned) p.norm_groups);
    return ck_launch([&] {
        if (otype == T_BF16) k_mamba2_gate_norm<__nv_bfloat16><<<grid, 256, 0, st>>>(y, u, p, w, eps, (__nv_bfloat16 *) out);
        else k_mamba2_gate_norm<float><<<grid, 256, 0, st>>>(y, u, p, w, eps, (float *) out);
    });
}

}  // namespace pb
