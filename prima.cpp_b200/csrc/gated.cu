// prima.cpp_b200/csrc/gated.cu — mechanisms of a dual mixer (an attention branch and a recurrent branch over the same input) and of the
// stream around it (declarations and semantics: layers.h): hashed bigram embedding; a short causal convolution over a range of projection
// channels with the slot's last inputs as history; the preparation of attention inputs (RMS norm over a whole projection or per head,
// partial rotation by position in either pair layout, values turned by their position) with the cache store; turning an attention
// result back + gate; gated linear recurrences whose decay comes with every token (gated delta rule, HGRN2) with the state in registers;
// two normed branch results joined onto the stream with the next norm in the same pass.  Everything here is fp32: positions, angles,
// norms, decays, the recurrent state and what enters it; only a value written for a dense product takes its operand type.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include <algorithm>

#include "layers.h"
#include "mixers.cuh"

namespace pb {
namespace {

// ---------------------------------------------------------------------------------------------------------------
template <typename WT>
__global__ void k_embed_bigram(const WT * __restrict__ table, const WT * __restrict__ bigram, int width, float scale, BigramParams bg,
                               const int32_t * __restrict__ tokens, const int32_t * __restrict__ off, const int32_t * __restrict__ entry_of,
                               const int32_t * __restrict__ prev, float * __restrict__ x, float * __restrict__ x0) {
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int tok = tokens[t];
    const int pv = t == off[e] ? prev[e] : tokens[t - 1];
    const int64_t brow = (pv < 0 || bg.buckets <= 0) ? bg.buckets : ((int64_t) pv * bg.mul_prev + (int64_t) tok * bg.mul_cur) % bg.buckets;
    const WT * er = table + (int64_t) tok * width;
    const WT * br = bigram ? bigram + brow * width : nullptr;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = ld_f(er, i) * scale;
        if (br) v += ld_f(br, i);
        x[(int64_t) t * width + i] = v;
        if (x0) x0[(int64_t) t * width + i] = v;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// grid (tokens, channel tiles): a thread owns one channel of one token
__global__ void k_causal_conv(const float * __restrict__ u, int64_t ldu, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                              const int32_t * __restrict__ entry_of, int channels, int taps, const float * __restrict__ w, int silu_from,
                              float * __restrict__ conv_state, int64_t slot_stride, float * __restrict__ out, int64_t ldo, int advance) {
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int lt = t - off[e];
    float * st = conv_state + (int64_t) slot[e] * slot_stride;   // [taps - 1][channels], row taps - 2 = the input just before this entry
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int d = taps - 1; d >= 0; d--) {                          // oldest input first
            const int l2 = lt - d;
            const float in = l2 >= 0 ? u[(int64_t) (t - d) * ldu + c] : st[(int64_t) (taps - 1 + l2) * channels + c];
            acc = fmaf(w[(int64_t) c * taps + (taps - 1 - d)], in, acc);
        }
        out[(int64_t) t * ldo + c] = c >= silu_from ? silu_f(acc) : acc;
        if (advance) {   // entries of one token: this thread is the only reader and writer of its channel's state
            for (int k = 0; k + 1 < taps - 1; k++) st[(int64_t) k * channels + c] = st[(int64_t) (k + 1) * channels + c];
            if (taps > 1) st[(int64_t) (taps - 2) * channels + c] = u[(int64_t) t * ldu + c];
        }
    }
}
__global__ void k_causal_conv_state(const float * __restrict__ u, int64_t ldu, const int32_t * __restrict__ slot, const int32_t * __restrict__ off, int channels,
                                    int taps, float * __restrict__ conv_state, int64_t slot_stride) {
    const int e = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int n = off[e + 1] - off[e];
    float * st = conv_state + (int64_t) slot[e] * slot_stride;
    for (int k = 0; k < taps - 1; k++) {     // ascending: row k + n is read before a later iteration overwrites it
        const int l2 = n - (taps - 1) + k;   // index within the entry of the input that becomes state row k
        st[(int64_t) k * channels + c] = l2 >= 0 ? u[(int64_t) (off[e] + l2) * ldu + c] : st[(int64_t) (k + n) * channels + c];
    }
}

// ---------------------------------------------------------------------------------------------------------------
// turns the pair (a, b) by angle: (a cos - b sin, b cos + a sin)
__device__ __forceinline__ void turn(float & a, float & b, float angle) {
    float sn, cs;
    sincosf(angle, &sn, &cs);
    const float u = a, v = b;
    a = u * cs - v * sn;
    b = v * cs + u * sn;
}
// indices of pair i of a vector whose leading `dims` entries turn
__device__ __forceinline__ void pair_of(int i, int dims, int layout, int & ia, int & ib) {
    if (layout == ROT_INTERLEAVED) { ia = 2 * i; ib = 2 * i + 1; }
    else { ia = i; ib = i + dims / 2; }
}

// One CTA per token.  (1) RMS norm over the whole query projection and over the whole key projection with weights; (2) rotation of the
// leading entries of every query and key head; (3) every head divided by its own root mean square; (4) rotation of the value heads;
// (5) the K / V rows later tokens can still see go to the cache.  Steps that the design does not have are skipped.
// cs: scratch of rot_dims + vdim floats in shared memory: the token's cosines and sines, computed once for all heads
__device__ __forceinline__ void attn_prep_rows(float * qr, float * kr, float * vr, float fp, const AttnParams & a, const AttnPrep & pr, float * red, float * cs) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int QD = a.heads * a.dim, KD = a.kv_heads * a.dim;
    const int hq = pr.rot_dims / 2, hv2 = pr.v_rot ? a.vdim / 2 : 0;
    float * csv = cs + 2 * hq;
    for (int i = threadIdx.x; i < hq + hv2; i += blockDim.x) {
        if (i < hq) sincosf(fp * pr.rot_freq[i], &cs[2 * i + 1], &cs[2 * i]);
        else sincosf(fp * pr.v_freq[i - hq], &csv[2 * (i - hq) + 1], &csv[2 * (i - hq)]);
    }
    // the barrier after the whole-projection norm, or the one below, makes the table visible
    if (pr.norm == QKN_WHOLE_WEIGHT) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < QD; i += blockDim.x) sq = fmaf(qr[i], qr[i], sq);
        for (int i = threadIdx.x; i < KD; i += blockDim.x) sk = fmaf(kr[i], kr[i], sk);
        const float iq = 1.f / sqrtf(block_sum(sq, red) / (float) QD + pr.eps);
        const float ik = 1.f / sqrtf(block_sum(sk, red) / (float) KD + pr.eps);
        for (int i = threadIdx.x; i < QD; i += blockDim.x) qr[i] = qr[i] * iq * pr.wq[i];
        for (int i = threadIdx.x; i < KD; i += blockDim.x) kr[i] = kr[i] * ik * pr.wk[i];
    }
    __syncthreads();
    if (pr.rot_dims > 1) {
        const int hp = pr.rot_dims / 2, total = (a.heads + a.kv_heads) * hp;
        for (int j = threadIdx.x; j < total; j += blockDim.x) {
            const int hh = j / hp, i = j - hh * hp;
            float * hv = hh < a.heads ? qr + (int64_t) hh * a.dim : kr + (int64_t) (hh - a.heads) * a.dim;
            int ia, ib;
            pair_of(i, pr.rot_dims, pr.rot_layout, ia, ib);
            const float u = hv[ia], w = hv[ib], c = cs[2 * i], sn = cs[2 * i + 1];
            hv[ia] = u * c - w * sn;
            hv[ib] = w * c + u * sn;
        }
        __syncthreads();
    }
    if (pr.norm == QKN_HEAD_UNIT) {
        for (int hh = warp; hh < a.heads + a.kv_heads; hh += nw) {
            float * hv = hh < a.heads ? qr + (int64_t) hh * a.dim : kr + (int64_t) (hh - a.heads) * a.dim;
            float ss = 0.f;
            for (int i = lane; i < a.dim; i += 32) ss = fmaf(hv[i], hv[i], ss);
            const float inv = 1.f / sqrtf(wsum(ss) / (float) a.dim + pr.eps);
            for (int i = lane; i < a.dim; i += 32) hv[i] *= inv;
        }
    }
    if (pr.v_rot && a.vdim > 1) {
        const int hp = a.vdim / 2, total = a.kv_heads * hp;
        for (int j = threadIdx.x; j < total; j += blockDim.x) {
            const int hh = j / hp, i = j - hh * hp;
            float * hv = vr + (int64_t) hh * a.vdim;
            int ia, ib;
            pair_of(i, 2 * hp, pr.v_layout, ia, ib);
            const float u = hv[ia], w = hv[ib], c = csv[2 * i], sn = csv[2 * i + 1];
            hv[ia] = u * c - w * sn;
            hv[ib] = w * c + u * sn;
        }
    }
}
// the inputs of a recurrent branch that ride along in the same launch (launch_dual_prep_store)
struct RecPrep {
    int kind = -1;            // 0: gated delta rule (launch_delta_prep), 1: HGRN2 (launch_hgrn2_prep), -1: nothing
    float * q = nullptr;      int64_t ldq = 0;
    float * k = nullptr;      int64_t ldk = 0;     // HGRN2: the forget-gate logits
    float * beta = nullptr;   int64_t ldb = 0;
    float * a = nullptr;      int64_t lda = 0;
    const float * p0 = nullptr, * p1 = nullptr;    // A_log, dt_bias  |  f_bias, lower
    int qk_heads = 0, heads = 0, dim = 0;
};
__device__ __forceinline__ void delta_prep_rows(float * qr, float * kr, float * bp, float * ap, const float * __restrict__ A_log,
                                                const float * __restrict__ dt_bias, int qk_heads, int heads, int dim) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const float qs = 1.f / sqrtf((float) dim);
    for (int hh = warp; hh < 2 * qk_heads; hh += nw) {
        const bool isq = hh < qk_heads;
        float * hv = isq ? qr + (int64_t) hh * dim : kr + (int64_t) (hh - qk_heads) * dim;
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) ss = fmaf(hv[i], hv[i], ss);
        const float inv = (1.f / sqrtf(wsum(ss) + 1e-6f)) * (isq ? qs : 1.f);
        for (int i = lane; i < dim; i += 32) hv[i] *= inv;
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        bp[h] = sigmoid_f(bp[h]);
        const float z = ap[h] + dt_bias[h];
        const float sp = z > 20.f ? z : log1pf(expf(z));
        ap[h] = expf(-expf(A_log[h]) * sp);
    }
}
__device__ __forceinline__ void hgrn2_prep_rows(float * qr, float * fr, const float * __restrict__ f_bias, const float * __restrict__ lower, int n) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        qr[i] = silu_f(qr[i]);
        const float lo = lower[i];
        fr[i] = lo + (1.f - lo) * sigmoid_f(fr[i] + f_bias[i]);
    }
}

// One CTA per token prepares everything the token's branches need before their kernels.  With `staged` the token's q, k, v rows (and the
// recurrence's q and k rows) are copied into shared memory once, every step runs there, and the rows go back to global memory (and the
// K / V rows later tokens can still see to the cache) once: two passes over global memory instead of one per step.
__global__ void __launch_bounds__(256) k_dual_prep_store(RecPrep rc, float * __restrict__ q, int64_t ldq, float * __restrict__ k, int64_t ldk,
                                                         float * __restrict__ v, int64_t ldv, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                                         const int32_t * __restrict__ pos0, const int32_t * __restrict__ entry_of, AttnParams a, AttnPrep pr,
                                                         float * __restrict__ kcache, float * __restrict__ vcache, int64_t slot_stride, int staged) {
    extern __shared__ float sm[];
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int n = off[e + 1] - off[e];
    const int p = pos0[e] + (t - off[e]), pend = pos0[e] + n;
    const int QD = a.heads * a.dim, KD = a.kv_heads * a.dim, VD = a.kv_heads * a.vdim, RQ = rc.kind >= 0 ? rc.qk_heads * rc.dim : 0;
    float * gq = q + (int64_t) t * ldq, * gk = k + (int64_t) t * ldk, * gv = v + (int64_t) t * ldv;
    float * grq = rc.kind >= 0 ? rc.q + (int64_t) t * rc.ldq : nullptr, * grk = rc.kind >= 0 ? rc.k + (int64_t) t * rc.ldk : nullptr;
    float * qr = gq, * kr = gk, * vr = gv, * rqr = grq, * rkr = grk;
    float * cs = sm;                                 // the token's cosines and sines: [rot_dims] for q / k, [vdim] for v
    float * rows = sm + ((pr.rot_dims + a.vdim + 3) & ~3);
    if (staged) {
        qr = rows; kr = qr + QD; vr = kr + KD; rqr = vr + VD; rkr = rqr + RQ;
        for (int i = threadIdx.x; i < QD; i += blockDim.x) qr[i] = gq[i];
        for (int i = threadIdx.x; i < KD; i += blockDim.x) kr[i] = gk[i];
        for (int i = threadIdx.x; i < VD; i += blockDim.x) vr[i] = gv[i];
        for (int i = threadIdx.x; i < RQ; i += blockDim.x) { rqr[i] = grq[i]; rkr[i] = grk[i]; }
        __syncthreads();
    }
    if (rc.kind == 0) delta_prep_rows(rqr, rkr, rc.beta + (int64_t) t * rc.ldb, rc.a + (int64_t) t * rc.lda, rc.p0, rc.p1, rc.qk_heads, rc.heads, rc.dim);
    else if (rc.kind == 1) hgrn2_prep_rows(rqr, rkr, rc.p0, rc.p1, RQ);
    attn_prep_rows(qr, kr, vr, (float) p, a, pr, red, cs);
    __syncthreads();
    if (staged) {
        for (int i = threadIdx.x; i < QD; i += blockDim.x) gq[i] = qr[i];
        for (int i = threadIdx.x; i < KD; i += blockDim.x) gk[i] = kr[i];
        for (int i = threadIdx.x; i < VD; i += blockDim.x) gv[i] = vr[i];
        for (int i = threadIdx.x; i < RQ; i += blockDim.x) { grq[i] = rqr[i]; grk[i] = rkr[i]; }
    }
    const int keep = min(a.keep_first, a.cache_rows), ring = a.cache_rows - keep;
    // of the positions that share a ring row only the last one of this entry is stored
    if (p >= keep && (ring <= 0 || p < pend - ring)) return;
    const int crow = p < keep ? p : keep + (p - keep) % max(ring, 1);
    float * kd = kcache + (int64_t) slot[e] * slot_stride + (int64_t) crow * KD;
    float * vd = vcache + (int64_t) slot[e] * slot_stride + (int64_t) crow * VD;
    for (int i = threadIdx.x; i < KD; i += blockDim.x) kd[i] = kr[i];
    for (int i = threadIdx.x; i < VD; i += blockDim.x) vd[i] = vr[i];
}

// grid (tokens, heads): one thread per pair of the head's result
template <typename OT>
__global__ void k_attn_unrotate_gate(const float * __restrict__ o, const int32_t * __restrict__ off, const int32_t * __restrict__ pos0,
                                     const int32_t * __restrict__ entry_of, int heads, int vdim, int v_layout, const float * __restrict__ v_freq,
                                     const float * __restrict__ gate, int64_t ldg, int gate_mode, float out_scale, OT * __restrict__ out, int64_t ldo) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int e = entry_of[t];
    const float fp = (float) (pos0[e] + (t - off[e]));
    const float * src = o + ((int64_t) t * heads + h) * vdim;
    const int hp = vdim / 2;
    const float gh = gate_mode == 1 ? sigmoid_f(gate[(int64_t) t * ldg + h]) * out_scale : out_scale;
    for (int i = threadIdx.x; i < hp + (vdim & 1); i += blockDim.x) {
        if (i == hp) {   // an odd last entry has no partner
            const float gg = gate_mode == 2 ? sigmoid_f(gate[(int64_t) t * ldg + (int64_t) h * vdim + vdim - 1]) : 1.f;
            put(out, (int64_t) t * ldo + (int64_t) h * vdim + vdim - 1, src[vdim - 1] * gh * gg);
            continue;
        }
        int ia, ib;
        pair_of(i, 2 * hp, v_layout, ia, ib);
        float va = src[ia], vb = src[ib];
        if (v_freq) turn(va, vb, -fp * v_freq[i]);
        float ga = gh, gb = gh;
        if (gate_mode == 2) {
            ga *= sigmoid_f(gate[(int64_t) t * ldg + (int64_t) h * vdim + ia]);
            gb *= sigmoid_f(gate[(int64_t) t * ldg + (int64_t) h * vdim + ib]);
        }
        put(out, (int64_t) t * ldo + (int64_t) h * vdim + ia, va * ga);
        put(out, (int64_t) t * ldo + (int64_t) h * vdim + ib, vb * gb);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// the two preparations as kernels of their own (one CTA per token)
__global__ void __launch_bounds__(256) k_delta_prep(float * __restrict__ q, int64_t ldq, float * __restrict__ k, int64_t ldk, float * __restrict__ beta,
                                                    int64_t ldb, float * __restrict__ a, int64_t lda, const float * __restrict__ A_log,
                                                    const float * __restrict__ dt_bias, int qk_heads, int heads, int dim) {
    const int64_t t = blockIdx.x;
    delta_prep_rows(q + t * ldq, k + t * ldk, beta + t * ldb, a + t * lda, A_log, dt_bias, qk_heads, heads, dim);
}
__global__ void k_hgrn2_prep(float * __restrict__ q, int64_t ldq, float * __restrict__ f, int64_t ldf, const float * __restrict__ f_bias,
                             const float * __restrict__ lower, int n) {
    const int64_t t = blockIdx.x;
    hgrn2_prep_rows(q + t * ldq, f + t * ldf, f_bias, lower, n);
}

// ---- C: both branches' results into the operand of the one output product.  grid (tokens, left heads + right heads): a CTA of the first
// kind turns an attention head back and gates it; one of the second kind divides a recurrence head by its root mean square, applies the
// weight and the gate ----
template <typename OT>
__global__ void __launch_bounds__(128) k_dual_post(const float * __restrict__ o, const int32_t * __restrict__ off, const int32_t * __restrict__ pos0,
                                                   const int32_t * __restrict__ entry_of, int heads, int vdim, int v_layout, const float * __restrict__ v_freq,
                                                   const float * __restrict__ gate, int64_t ldg, int gate_mode, float left_scale, const float * __restrict__ y,
                                                   int r_heads, int r_vdim, const float * __restrict__ r_gate, int64_t ldrg, const float * __restrict__ r_w,
                                                   int r_gate_act, float eps, float right_scale, OT * __restrict__ out, int64_t ldo) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    if ((int) blockIdx.y < heads) {
        const int h = blockIdx.y;
        const int e = entry_of[t];
        const float fp = (float) (pos0[e] + (t - off[e]));
        const float * src = o + ((int64_t) t * heads + h) * vdim;
        const int hp = vdim / 2;
        const float gh = gate_mode == 1 ? sigmoid_f(gate[(int64_t) t * ldg + h]) * left_scale : left_scale;
        for (int i = threadIdx.x; i < hp + (vdim & 1); i += blockDim.x) {
            if (i == hp) {
                const float gg = gate_mode == 2 ? sigmoid_f(gate[(int64_t) t * ldg + (int64_t) h * vdim + vdim - 1]) : 1.f;
                put(out, (int64_t) t * ldo + (int64_t) h * vdim + vdim - 1, src[vdim - 1] * gh * gg);
                continue;
            }
            int ia, ib;
            pair_of(i, 2 * hp, v_layout, ia, ib);
            float va = src[ia], vb = src[ib];
            if (v_freq) turn(va, vb, -fp * v_freq[i]);
            float ga = gh, gb = gh;
            if (gate_mode == 2) {
                ga *= sigmoid_f(gate[(int64_t) t * ldg + (int64_t) h * vdim + ia]);
                gb *= sigmoid_f(gate[(int64_t) t * ldg + (int64_t) h * vdim + ib]);
            }
            put(out, (int64_t) t * ldo + (int64_t) h * vdim + ia, va * ga);
            put(out, (int64_t) t * ldo + (int64_t) h * vdim + ib, vb * gb);
        }
        return;
    }
    const int h = blockIdx.y - heads;
    const float * yr = y + ((int64_t) t * r_heads + h) * r_vdim;
    const float * gr = r_gate_act >= 0 ? r_gate + (int64_t) t * ldrg + (int64_t) h * r_vdim : nullptr;
    float q = 0.f;
    for (int i = threadIdx.x; i < r_vdim; i += blockDim.x) q = fmaf(yr[i], yr[i], q);
    const float inv = 1.f / sqrtf(block_sum(q, red) / (float) r_vdim + eps);
    for (int i = threadIdx.x; i < r_vdim; i += blockDim.x) {
        float v = yr[i] * inv;
        if (r_w) v *= r_w[h * r_vdim + i];
        if (gr) v *= r_gate_act == 0 ? sigmoid_f(gr[i]) : silu_f(gr[i]);
        put(out, (int64_t) t * ldo + (int64_t) heads * vdim + (int64_t) h * r_vdim + i, v * right_scale);
    }
}

// A CTA owns one head and 16 value columns.  LN lanes share a column: thread (pl = tid / LN, ng = tid % LN) keeps S[n][column pl] for
// n = NREG ng .. NREG ng + NREG - 1 (consecutive, so that a token's k and q entries come out of shared memory as 16-byte loads).  Tokens are walked in chunks of 16 whose q, k (or per-channel decay) rows, v columns and per-head
// numbers go through registers into shared memory; the loads of the next chunk are in flight while the current one runs.  A token costs a
// thread NREG fused steps and the column ONE shuffle reduction: for the delta rule the products of the OLD state with k and with q are
// reduced together (with k . q), and  u = beta (v - g S_old^T k),  y = g S_old^T q + u (k . q)  follow without a second pass.
constexpr int GCHUNK = 16, GCOLS = 16;
template <int NREG, int LN, bool DELTA, bool CHAN>
__global__ void __launch_bounds__(GCOLS * LN) k_gated_linattn_reg(GatedLinIO io, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                                                  GatedLinParams p, float * __restrict__ state, int64_t slot_stride, float * __restrict__ y) {
    extern __shared__ float sm[];
    constexpr int NT = GCOLS * LN;
    constexpr int NV = (GCHUNK * GCOLS + NT - 1) / NT;
    const int N = p.dim, P = p.vdim, inner = p.heads * p.vdim;
    const int ptiles = (P + GCOLS - 1) / GCOLS;
    const int h = blockIdx.x / ptiles, pt = blockIdx.x - h * ptiles, e = blockIdx.y;
    const int hk = h / (p.heads / p.qk_heads);
    const int tid = threadIdx.x, pl = tid / LN, ng = tid % LN;
    const int pcol = pt * GCOLS + pl;
    const bool pok = pcol < P;
    float * Ks = sm;                        // [GCHUNK][N]  key, or the per-channel decay when the key is tied to it
    float * Qs = Ks + GCHUNK * N;           // [GCHUNK][N]
    float * Vs = Qs + GCHUNK * N;           // [GCHUNK][GCOLS]
    float * Gs = Vs + GCHUNK * GCOLS;       // [GCHUNK] decay per token (one per head), [GCHUNK] beta
    float * gst = state + (int64_t) slot[e] * slot_stride + (int64_t) h * N * P;
    float S[NREG];
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int nn = ng * NREG + j;
        S[j] = (pok && nn < N) ? gst[(int64_t) nn * P + pcol] : 0.f;
    }
    const int t0 = off[e], n = off[e + 1] - t0;
    const bool vec4 = NREG % 4 == 0 && (N & 3) == 0;
    // this thread's NREG entries of a staged row (zeros beyond the key size)
    auto row_regs = [&](const float * row, float (&r)[NREG]) {
        if (vec4) {
#pragma unroll
            for (int j = 0; j < NREG; j += 4) {
                const int nn = ng * NREG + j;
                const float4 v = nn < N ? *reinterpret_cast<const float4 *>(row + nn) : make_float4(0.f, 0.f, 0.f, 0.f);
                r[j] = v.x; r[(j + 1) % NREG] = v.y; r[(j + 2) % NREG] = v.z; r[(j + 3) % NREG] = v.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < NREG; j++) {
                const int nn = ng * NREG + j;
                r[j] = nn < N ? row[nn] : 0.f;
            }
        }
    };
    float rk[NREG], rq[NREG], rv[NV], rg = 0.f;
    auto fetch = [&](int c0) {
        const int nc = min(GCHUNK, n - c0);
#pragma unroll
        for (int k = 0; k < NREG; k++) {
            const int i = tid + NT * k;
            if (i < nc * N) {
                const int tt = i / N, nn = i - tt * N;
                const int64_t tok = t0 + c0 + tt;
                rk[k] = CHAN ? io.decay[tok * io.ldd + hk * N + nn] : io.k[tok * io.ldk + hk * N + nn];
                rq[k] = io.q[tok * io.ldq + hk * N + nn];
            }
        }
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int i = tid + NT * k, tt = i / GCOLS, pp = i - tt * GCOLS;
            rv[k] = (tt < nc && pt * GCOLS + pp < P) ? io.v[(int64_t) (t0 + c0 + tt) * io.ldv + h * P + pt * GCOLS + pp] : 0.f;
        }
        if (tid < 2 * GCHUNK) {
            const int tt = tid & (GCHUNK - 1);
            rg = 0.f;
            if (tt < nc) {
                if (tid < GCHUNK) { if (!CHAN) rg = io.decay[(int64_t) (t0 + c0 + tt) * io.ldd + h]; }
                else if (DELTA) rg = io.beta[(int64_t) (t0 + c0 + tt) * io.ldb + h];
            }
        }
    };
    if (n > 0) fetch(0);
    for (int c0 = 0; c0 < n; c0 += GCHUNK) {
        const int nc = min(GCHUNK, n - c0);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < NREG; k++) {
            const int i = tid + NT * k;
            if (i < nc * N) { Ks[i] = rk[k]; Qs[i] = rq[k]; }
        }
#pragma unroll
        for (int k = 0; k < NV; k++)
            if (tid + NT * k < GCHUNK * GCOLS) Vs[tid + NT * k] = rv[k];
        if (tid < 2 * GCHUNK) Gs[tid] = rg;
        __syncthreads();
        if (c0 + GCHUNK < n) fetch(c0 + GCHUNK);
        for (int tt = 0; tt < nc; tt++) {
            const float xv = Vs[tt * GCOLS + pl];
            float kk[NREG], qq[NREG];
            row_regs(Ks + tt * N, kk);
            row_regs(Qs + tt * N, qq);
            float out;
            if constexpr (DELTA) {
                // old state against k and q, and k . q, in one reduction (entries beyond the key size are zero on both sides)
                float sk = 0.f, sq = 0.f, kq = 0.f;
#pragma unroll
                for (int j = 0; j < NREG; j++) {
                    sk = fmaf(S[j], kk[j], sk);
                    sq = fmaf(S[j], qq[j], sq);
                    kq = fmaf(kk[j], qq[j], kq);
                }
#pragma unroll
                for (int o = 1; o < LN; o <<= 1) {
                    sk += __shfl_xor_sync(0xffffffffu, sk, o);
                    sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    kq += __shfl_xor_sync(0xffffffffu, kq, o);
                }
                const float g = Gs[tt], u = Gs[GCHUNK + tt] * (xv - g * sk);
#pragma unroll
                for (int j = 0; j < NREG; j++) S[j] = fmaf(kk[j], u, g * S[j]);
                out = fmaf(u, kq, g * sq);
            } else {
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < NREG; j++) {
                    if constexpr (CHAN) S[j] = fmaf(kk[j], S[j], (1.f - kk[j]) * xv);   // key tied to the decay
                    else S[j] = fmaf(Gs[tt], S[j], kk[j] * xv);
                    acc = fmaf(S[j], qq[j], acc);                                      // q is zero beyond the key size
                }
#pragma unroll
                for (int o = 1; o < LN; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                out = acc;
            }
            if (ng == 0 && pok) y[(int64_t) (t0 + c0 + tt) * inner + h * P + pcol] = out;
        }
    }
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int nn = ng * NREG + j;
        if (pok && nn < N) gst[(int64_t) nn * P + pcol] = S[j];
    }
}

// any key size: one CTA per (head, 64 value columns, entry), the state tile S [N][64] in shared memory for the whole entry; a thread owns
// a quarter of one column's rows.  The plain order of the recurrence: decay, (delta: read S^T k, write), read S^T q.
constexpr int GSCOLS = 64;
__global__ void __launch_bounds__(256) k_gated_linattn_smem(GatedLinIO io, const int32_t * __restrict__ slot, const int32_t * __restrict__ off, GatedLinParams p,
                                                            float * __restrict__ state, int64_t slot_stride, float * __restrict__ y) {
    extern __shared__ float sm[];
    const int N = p.dim, P = p.vdim, inner = p.heads * p.vdim;
    const int ptiles = (P + GSCOLS - 1) / GSCOLS;
    const int h = blockIdx.x / ptiles, pt = blockIdx.x - h * ptiles, e = blockIdx.y;
    const int hk = h / (p.heads / p.qk_heads);
    const int c0 = pt * GSCOLS, nc = min(GSCOLS, P - c0);
    float * S = sm;                 // [N][GSCOLS]
    float * ks = S + N * GSCOLS;    // [N]
    float * qs = ks + N;            // [N]
    float * fs = qs + N;            // [N] per-channel decay
    float * vs = fs + N;            // [GSCOLS]
    float * part = vs + GSCOLS;     // [4][GSCOLS]
    float * gst = state + (int64_t) slot[e] * slot_stride + (int64_t) h * N * P;
    for (int i = threadIdx.x; i < N * GSCOLS; i += blockDim.x) {
        const int nn = i / GSCOLS, cc = i - nn * GSCOLS;
        S[i] = cc < nc ? gst[(int64_t) nn * P + c0 + cc] : 0.f;
    }
    const int t0 = off[e], n = off[e + 1] - t0;
    const int cc = threadIdx.x & (GSCOLS - 1), q4 = threadIdx.x / GSCOLS;
    for (int lt = 0; lt < n; lt++) {
        const int64_t tok = t0 + lt;
        __syncthreads();
        for (int i = threadIdx.x; i < N; i += blockDim.x) {
            qs[i] = io.q[tok * io.ldq + hk * N + i];
            const float f = p.decay_per_channel ? io.decay[tok * io.ldd + hk * N + i] : io.decay[tok * io.ldd + h];
            fs[i] = f;
            ks[i] = p.tied_key ? 1.f - f : io.k[tok * io.ldk + hk * N + i];
        }
        for (int i = threadIdx.x; i < GSCOLS; i += blockDim.x) vs[i] = i < nc ? io.v[tok * io.ldv + h * P + c0 + i] : 0.f;
        __syncthreads();
        float u = vs[cc];
        if (p.delta) {
            float acc = 0.f;
            for (int nn = q4; nn < N; nn += 4) {
                const float s = fs[nn] * S[nn * GSCOLS + cc];
                S[nn * GSCOLS + cc] = s;
                acc = fmaf(s, ks[nn], acc);
            }
            part[q4 * GSCOLS + cc] = acc;
            __syncthreads();
            const float sk = (part[cc] + part[GSCOLS + cc]) + (part[2 * GSCOLS + cc] + part[3 * GSCOLS + cc]);
            u = io.beta[tok * io.ldb + h] * (u - sk);
            __syncthreads();
        }
        float acc = 0.f;
        for (int nn = q4; nn < N; nn += 4) {
            const float s = p.delta ? fmaf(ks[nn], u, S[nn * GSCOLS + cc]) : fmaf(fs[nn], S[nn * GSCOLS + cc], ks[nn] * u);
            S[nn * GSCOLS + cc] = s;
            acc = fmaf(s, qs[nn], acc);
        }
        part[q4 * GSCOLS + cc] = acc;
        __syncthreads();
        if (threadIdx.x < nc) y[tok * inner + h * P + c0 + threadIdx.x] =
            (part[threadIdx.x] + part[GSCOLS + threadIdx.x]) + (part[2 * GSCOLS + threadIdx.x] + part[3 * GSCOLS + threadIdx.x]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < N * GSCOLS; i += blockDim.x) {
        const int nn = i / GSCOLS, c2 = i - nn * GSCOLS;
        if (c2 < nc) gst[(int64_t) nn * P + c0 + c2] = S[i];
    }
}

// ---------------------------------------------------------------------------------------------------------------
// one CTA per token: both rows are normed, joined onto the stream, and the new stream row is normed for the next sublayer
template <typename OT>
__global__ void __launch_bounds__(256) k_rmsnorm_pair_residual(const float * __restrict__ a, int64_t lda, const float * __restrict__ bb, int64_t ldb,
                                                               const float * __restrict__ wa, const float * __restrict__ wb, float mult, float eps,
                                                               float * __restrict__ x, const float * __restrict__ wn, OT * __restrict__ y, int width) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const float * ar = a + (int64_t) t * lda, * br = bb + (int64_t) t * ldb;
    float * xr = x + (int64_t) t * width;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { sa = fmaf(ar[i], ar[i], sa); sb = fmaf(br[i], br[i], sb); }
    const float ia = 1.f / sqrtf(block_sum(sa, red) / (float) width + eps);
    const float ib = 1.f / sqrtf(block_sum(sb, red) / (float) width + eps);
    float sx = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i] + mult * (ar[i] * ia * wa[i] + br[i] * ib * wb[i]);
        xr[i] = v;                       // the same thread reads it back below
        sx = fmaf(v, v, sx);
    }
    if (!y) return;
    const float ix = 1.f / sqrtf(block_sum(sx, red) / (float) width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) put(y, (int64_t) t * width + i, xr[i] * ix * wn[i]);
}

template <typename OT>
__global__ void __launch_bounds__(256) k_stream_add_rmsnorm(float * __restrict__ x, const float * __restrict__ x0, const float * __restrict__ vec,
                                                            const float * __restrict__ w, float eps, OT * __restrict__ y, int width) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    float * xr = x + (int64_t) t * width;
    float sx = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = xr[i];
        if (x0) v += x0[(int64_t) t * width + i];
        if (vec) v += vec[i];
        xr[i] = v;
        sx = fmaf(v, v, sx);
    }
    const float ix = 1.f / sqrtf(block_sum(sx, red) / (float) width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) put(y, (int64_t) t * width + i, xr[i] * ix * w[i]);
}

}  // namespace

int launch_stream_add_rmsnorm(float * x, const float * x0, const float * vec, const float * w, float eps, void * y, int otype, int n_rows, int width,
                              cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (!x || !w || !y) return (int) cudaErrorInvalidValue;
    return ck_launch([&] {
        if (otype == T_BF16) k_stream_add_rmsnorm<__nv_bfloat16><<<n_rows, 256, 0, st>>>(x, x0, vec, w, eps, (__nv_bfloat16 *) y, width);
        else k_stream_add_rmsnorm<float><<<n_rows, 256, 0, st>>>(x, x0, vec, w, eps, (float *) y, width);
    });
}

int launch_embed_bigram(const void * table, const void * bigram, int type, int width, float scale, const BigramParams & bg, const int32_t * tokens,
                        const BatchView & b, float * x, float * x0, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (!b.prev || (bigram && bg.buckets <= 0)) return (int) cudaErrorInvalidValue;
    return ck_launch([&] {
        if (type == T_BF16)
            k_embed_bigram<__nv_bfloat16><<<b.n_tokens, 128, 0, st>>>((const __nv_bfloat16 *) table, (const __nv_bfloat16 *) bigram, width, scale, bg, tokens, b.off,
                                                                      b.entry_of, b.prev, x, x0);
        else k_embed_bigram<float><<<b.n_tokens, 128, 0, st>>>((const float *) table, (const float *) bigram, width, scale, bg, tokens, b.off, b.entry_of, b.prev, x, x0);
    });
}

int launch_causal_conv(const float * u, int64_t ldu, const BatchView & b, int channels, int taps, const float * w, int silu_from, float * conv_state,
                       int64_t slot_stride, float * out, int64_t ldo, cudaStream_t st) {
    if (b.n_tokens <= 0 || channels <= 0) return 0;
    if (taps < 1 || !w || (taps > 1 && !conv_state)) return (int) cudaErrorInvalidValue;
    const int tiles = b.n_tokens >= 512 ? 1 : std::min((channels + 127) / 128, 32);   // few tokens: a token's channels spread over CTAs
    const int advance = b.max_n == 1 && taps > 1;   // one-token entries: the same kernel moves the state on
    int rc = ck_launch([&] {
        k_causal_conv<<<dim3((unsigned) b.n_tokens, (unsigned) tiles), 128, 0, st>>>(u, ldu, b.slot, b.off, b.entry_of, channels, taps, w, silu_from, conv_state,
                                                                                     slot_stride, out, ldo, advance);
    });
    if (rc || taps == 1 || advance) return rc;
    return ck_launch([&] {
        k_causal_conv_state<<<dim3((unsigned) ((channels + 127) / 128), (unsigned) b.n_entries), 128, 0, st>>>(u, ldu, b.slot, b.off, channels, taps, conv_state, slot_stride);
    });
}

static int dual_prep_launch(const RecPrep & rc, float * q, int64_t ldq, float * k, int64_t ldk, float * v, int64_t ldv, const BatchView & b, const AttnParams & a,
                            const AttnPrep & pr, float * kcache, float * vcache, int64_t slot_stride, cudaStream_t st) {
    if (a.heads <= 0 || a.kv_heads <= 0 || a.dim <= 0 || a.vdim <= 0 || pr.rot_dims < 0 || pr.rot_dims > a.dim || (pr.rot_dims & 1) ||
        (pr.rot_dims > 0 && !pr.rot_freq) || (pr.v_rot && !pr.v_freq) || (pr.norm == QKN_WHOLE_WEIGHT && (!pr.wq || !pr.wk)))
        return (int) cudaErrorInvalidValue;
    // the token's rows in shared memory when they fit
    const size_t floats = (size_t) a.heads * a.dim + (size_t) a.kv_heads * (a.dim + a.vdim) + (rc.kind >= 0 ? 2 * (size_t) rc.qk_heads * rc.dim : 0);
    const size_t table = (size_t) ((pr.rot_dims + a.vdim + 3) & ~3);   // cosines and sines of the token's position
    const int staged = (floats + table) * sizeof(float) <= 160 * 1024;
    const size_t smem = (table + (staged ? floats : 0)) * sizeof(float);
    int e = raise_smem(k_dual_prep_store, smem);
    if (e) return e;
    return ck_launch([&] {
        k_dual_prep_store<<<b.n_tokens, 256, smem, st>>>(rc, q, ldq, k, ldk, v, ldv, b.slot, b.off, b.pos0, b.entry_of, a, pr, kcache, vcache, slot_stride, staged);
    });
}
int launch_attn_prep_store(float * q, int64_t ldq, float * k, int64_t ldk, float * v, int64_t ldv, const BatchView & b, const AttnParams & a,
                           const AttnPrep & pr, float * kcache, float * vcache, int64_t slot_stride, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    return dual_prep_launch(RecPrep(), q, ldq, k, ldk, v, ldv, b, a, pr, kcache, vcache, slot_stride, st);
}

int launch_attn_unrotate_gate(const float * o, const BatchView & b, int heads, int vdim, int v_layout, const float * v_freq, const float * gate, int64_t ldg,
                              int gate_mode, float out_scale, void * out, int64_t ldo, int otype, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || (gate_mode != 0 && !gate)) return (int) cudaErrorInvalidValue;
    const dim3 grid((unsigned) b.n_tokens, (unsigned) heads);
    const int threads = vdim / 2 >= 128 ? 128 : vdim / 2 >= 64 ? 64 : 32;
    return ck_launch([&] {
        if (otype == T_BF16)
            k_attn_unrotate_gate<__nv_bfloat16><<<grid, threads, 0, st>>>(o, b.off, b.pos0, b.entry_of, heads, vdim, v_layout, v_freq, gate, ldg, gate_mode, out_scale,
                                                                         (__nv_bfloat16 *) out, ldo);
        else k_attn_unrotate_gate<float><<<grid, threads, 0, st>>>(o, b.off, b.pos0, b.entry_of, heads, vdim, v_layout, v_freq, gate, ldg, gate_mode, out_scale,
                                                                   (float *) out, ldo);
    });
}

int launch_delta_prep(float * q, int64_t ldq, float * k, int64_t ldk, float * beta, int64_t ldb, float * a, int64_t lda, const float * A_log,
                      const float * dt_bias, int qk_heads, int heads, int dim, int n_tokens, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (qk_heads <= 0 || heads <= 0 || dim <= 0 || !A_log || !dt_bias) return (int) cudaErrorInvalidValue;
    return ck_launch([&] { k_delta_prep<<<n_tokens, 256, 0, st>>>(q, ldq, k, ldk, beta, ldb, a, lda, A_log, dt_bias, qk_heads, heads, dim); });
}
int launch_hgrn2_prep(float * q, int64_t ldq, float * f, int64_t ldf, const float * f_bias, const float * lower, int n, int n_tokens, cudaStream_t st) {
    if (n_tokens <= 0 || n <= 0) return 0;
    if (!f_bias || !lower) return (int) cudaErrorInvalidValue;
    return ck_launch([&] { k_hgrn2_prep<<<n_tokens, 256, 0, st>>>(q, ldq, f, ldf, f_bias, lower, n); });
}

int launch_gated_linattn(const GatedLinIO & io, const BatchView & b, const GatedLinParams & p, float * state, int64_t slot_stride, float * y, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (p.heads <= 0 || p.qk_heads <= 0 || p.heads % p.qk_heads || p.dim <= 0 || p.vdim <= 0 || !state || !io.q || !io.v || !io.decay || (p.delta && !io.beta) ||
        (p.tied_key && (!p.decay_per_channel || p.delta)) || (!p.tied_key && !io.k) || (p.decay_per_channel && !p.tied_key))
        return (int) cudaErrorInvalidValue;
    // the two register kernels: delta rule with one decay per head, tied key with a decay per channel
    if (p.dim <= 256 && ((p.delta && !p.decay_per_channel) || (p.tied_key && !p.delta))) {
        const int ln = p.dim <= 32 ? 8 : p.dim <= 64 ? 16 : 32;
        const int nreg = (p.dim + ln - 1) / ln;
        const size_t smem = ((size_t) 2 * GCHUNK * p.dim + GCHUNK * GCOLS + 2 * GCHUNK) * sizeof(float);
        const dim3 grid((unsigned) (p.heads * ((p.vdim + GCOLS - 1) / GCOLS)), (unsigned) b.n_entries);
#define PB_GL(NR, LNV)                                                                                                                               \
    do {                                                                                                                                             \
        if (p.delta) return ck_launch([&] { k_gated_linattn_reg<NR, LNV, true, false><<<grid, GCOLS * LNV, smem, st>>>(io, b.slot, b.off, p, state, slot_stride, y); }); \
        return ck_launch([&] { k_gated_linattn_reg<NR, LNV, false, true><<<grid, GCOLS * LNV, smem, st>>>(io, b.slot, b.off, p, state, slot_stride, y); });            \
    } while (0)
#define PB_GL_LN(LNV)                 \
    do {                              \
        if (nreg <= 1) PB_GL(1, LNV); \
        if (nreg <= 2) PB_GL(2, LNV); \
        if (nreg <= 4) PB_GL(4, LNV); \
        PB_GL(8, LNV);                \
    } while (0)
        if (ln == 8) PB_GL_LN(8);
        if (ln == 16) PB_GL_LN(16);
        PB_GL_LN(32);
#undef PB_GL_LN
#undef PB_GL
    }
    const size_t smem = ((size_t) p.dim * GSCOLS + 3 * (size_t) p.dim + 5 * GSCOLS) * sizeof(float);
    if (smem > 220 * 1024) return (int) cudaErrorInvalidValue;
    int rc = raise_smem(k_gated_linattn_smem, smem);
    if (rc) return rc;
    const dim3 grid((unsigned) (p.heads * ((p.vdim + GSCOLS - 1) / GSCOLS)), (unsigned) b.n_entries);
    return ck_launch([&] { k_gated_linattn_smem<<<grid, 256, smem, st>>>(io, b.slot, b.off, p, state, slot_stride, y); });
}

int launch_dual_prep_store(int rec_kind, float * rq, int64_t ldrq, float * rk, int64_t ldrk, float * beta, int64_t ldb, float * ra, int64_t lda, const float * p0,
                           const float * p1, int qk_heads, int r_heads, int r_dim, float * q, int64_t ldq, float * k, int64_t ldk, float * v, int64_t ldv,
                           const BatchView & b, const AttnParams & a, const AttnPrep & pr, float * kcache, float * vcache, int64_t slot_stride, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (rec_kind < 0 || rec_kind > 1 || !rq || !rk || !p0 || !p1 || qk_heads <= 0 || r_dim <= 0 || (rec_kind == 0 && (!beta || !ra || r_heads <= 0)))
        return (int) cudaErrorInvalidValue;
    RecPrep rc;
    rc.kind = rec_kind;
    rc.q = rq; rc.ldq = ldrq; rc.k = rk; rc.ldk = ldrk; rc.beta = beta; rc.ldb = ldb; rc.a = ra; rc.lda = lda;
    rc.p0 = p0; rc.p1 = p1; rc.qk_heads = qk_heads; rc.heads = r_heads; rc.dim = r_dim;
    return dual_prep_launch(rc, q, ldq, k, ldk, v, ldv, b, a, pr, kcache, vcache, slot_stride, st);
}

int launch_dual_post(const float * o, const BatchView & b, int heads, int vdim, int v_layout, const float * v_freq, const float * gate, int64_t ldg, int gate_mode,
                     float left_scale, const float * y, int r_heads, int r_vdim, const float * r_gate, int64_t ldrg, const float * r_w, int r_gate_act, float eps,
                     float right_scale, void * out, int64_t ldo, int otype, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || r_heads <= 0 || r_vdim <= 0 || (gate_mode != 0 && !gate) || !o || !y) return (int) cudaErrorInvalidValue;
    if (!r_gate) r_gate_act = -1;
    const dim3 grid((unsigned) b.n_tokens, (unsigned) (heads + r_heads));
    return ck_launch([&] {
        if (otype == T_BF16)
            k_dual_post<__nv_bfloat16><<<grid, 128, 0, st>>>(o, b.off, b.pos0, b.entry_of, heads, vdim, v_layout, v_freq, gate, ldg, gate_mode, left_scale, y, r_heads,
                                                            r_vdim, r_gate, ldrg, r_w, r_gate_act, eps, right_scale, (__nv_bfloat16 *) out, ldo);
        else
            k_dual_post<float><<<grid, 128, 0, st>>>(o, b.off, b.pos0, b.entry_of, heads, vdim, v_layout, v_freq, gate, ldg, gate_mode, left_scale, y, r_heads, r_vdim,
                                                    r_gate, ldrg, r_w, r_gate_act, eps, right_scale, (float *) out, ldo);
    });
}

int launch_rmsnorm_pair_residual(const float * a, int64_t lda, const float * bb, int64_t ldb, const float * wa, const float * wb, float mult, float eps,
                                 float * x, const float * wn, void * y, int otype, int n_rows, int width, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (!a || !bb || !wa || !wb || !x || (y && !wn)) return (int) cudaErrorInvalidValue;
    return ck_launch([&] {
        if (otype == T_BF16)
            k_rmsnorm_pair_residual<__nv_bfloat16><<<n_rows, 256, 0, st>>>(a, lda, bb, ldb, wa, wb, mult, eps, x, wn, (__nv_bfloat16 *) y, width);
        else k_rmsnorm_pair_residual<float><<<n_rows, 256, 0, st>>>(a, lda, bb, ldb, wa, wb, mult, eps, x, wn, (float *) y, width);
    });
}

}  // namespace pb
