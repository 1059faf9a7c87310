// prima.cpp_b200/csrc/layers.h — launchers of the dense (f32 / bf16 weight) products and of the sequence mixers that the layer-list
// engine (layers.cu) is built from: windowed attention with kept first tokens, soft-capped scores and a per-head output gate; the
// Mamba-2 state-space mixer (short causal convolution, selective scan, gated grouped RMS norm); weight-only layer norm with the
// residual add; tanh-GELU gating; RMS norm in groups, token shift and the depth average of layer results; linear attention with a
// fixed decay per head; softmax attention over a low-rank latent with a shared rotated key part; the clamped gated feed-forward, dense
// or as a routed mixture of experts; layer norm with weight and bias on a sublayer's result (post-norm frame), a learned position table,
// an RMS norm per query / key head, the squared-ReLU feed-forward, the router with sigmoid scores, a choice correction and expert groups,
// and the tanh soft-cap of the logits; a hashed bigram embedding, a short causal convolution over any range of projection channels, the
// preparation of attention inputs (RMS norm over a whole projection or per head, partial rotation in either pair layout, values rotated by
// their position), a sink in the softmax denominator, gated linear recurrences with a decay per token (gated delta rule, HGRN2), experts
// whose routing weight multiplies their input.  Every constant of a mechanism is a parameter, nothing is tied to one model.
// All launchers enqueue on `stream` and return a cudaError_t as int (0 = success).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pb {

enum : int { T_BF16 = 30 };   // enum ggml_type value of bfloat16

// ---- ragged batch: the tokens of all entries lie back to back; entry e owns tokens [off[e], off[e+1]) of sequence slot slot[e],
// at positions pos0[e] .. pos0[e] + n - 1 ----
struct BatchView {
    int n_entries = 0;
    int n_tokens = 0;
    int max_n = 0;                 // longest entry
    const int32_t * slot = nullptr;   // device [n_entries]
    const int32_t * off = nullptr;    // device [n_entries + 1]
    const int32_t * pos0 = nullptr;   // device [n_entries]
    const int32_t * entry_of = nullptr;   // device [n_tokens]
    const int32_t * prev = nullptr;       // device [n_entries]: the sequence's token before the entry's first one (-1: the entry starts the sequence)
};

// ---- dense products ----
// C[t][n] = alpha * sum_k A[t][k] * W[n][k] (+ bias[n]) (+ resid[t][n]);  A and W share `type` (T_F32: true fp32 multiply-add;
// T_BF16: bf16 operands, fp32 accumulation), C / bias / resid are f32.  resid may alias C.  lda / ldw / ldc / ldr in elements.
// The result of a row does not depend on the other rows of the call beyond the choice between the small-batch and the tiled kernel.
int launch_dense(int type, const void * A, int64_t lda, const void * W, int64_t ldw, float * C, int64_t ldc, int T, int N, int K,
                 const float * bias, const float * resid, int64_t ldr, float alpha, cudaStream_t stream);
// Grouped product in one launch: rows [start[g], start[g] + count[g]) of A times the g-th matrix of W (w_stride elements apart, [N][K]
// each) into the same rows of C, g < groups; start / count are device arrays and no group has more than max_rows rows.  Tensor-core
// kernel only (bf16, aligned shapes): dense_grouped_ok says whether it applies; otherwise the caller multiplies group by group.
int dense_grouped_ok(int type, int N, int K, int64_t lda, int64_t ldw, int64_t w_stride, const void * A, const void * W);
int launch_dense_grouped(int type, const void * A, int64_t lda, const void * W, int64_t ldw, int64_t w_stride, float * C, int64_t ldc, const int32_t * start,
                         const int32_t * count, int groups, int max_rows, int N, int K, cudaStream_t stream);
// 1: the tensor-core kernel takes this shape (bf16, aligned K / strides); informational (bench, tests)
int dense_uses_tensor_cores(int type, int T, int N, int K, int64_t lda, int64_t ldw);

// ---- element-wise / norms; `otype` (T_F32 | T_BF16) is the type of an activation that feeds a dense product ----
int launch_embed(const void * table, int type, int width, const int32_t * tokens, int n_tokens, float * x, float * x_copy, cudaStream_t stream);
// x[t] = table[tokens[t]] + pos_table[position of t] (fp32 sum; both tables in `type`); xa (if given) receives x in the operand type
int launch_embed_pos(const void * table, const void * pos_table, int type, int width, const int32_t * tokens, const BatchView & b, float * x, void * xa,
                     int otype, cudaStream_t stream);
// x[t] = table[tokens[t]] * scale + bigram[row], row = (previous token * mul_prev + tokens[t] * mul_cur) mod buckets, or row `buckets` for a
// sequence's first token (bigram == nullptr: no second table).  The previous token of an entry's first token is b.prev.  x0 (may be null)
// receives a copy.
struct BigramParams { int64_t buckets = 0, mul_prev = 0, mul_cur = 0; };
int launch_embed_bigram(const void * table, const void * bigram, int type, int width, float scale, const BigramParams & bg, const int32_t * tokens,
                        const BatchView & b, float * x, float * x0, cudaStream_t stream);
int launch_cast(const float * x, void * y, int otype, int64_t n, cudaStream_t stream);
// y[r] = (x[row] - mean) / sqrt(var + eps) * w, row = rows ? rows[r] : r; var = mean of squared deviations
int launch_layernorm(const float * x, const int32_t * rows, const float * w, float eps, void * y, int otype, int n_rows, int width, cudaStream_t stream);
// the same with a bias: y[r] = (x[row] - mean) / sqrt(var + eps) * w + bias   (bias may be null)
int launch_layernorm_affine(const float * x, const int32_t * rows, const float * w, const float * bias, float eps, void * y, int otype, int n_rows, int width,
                            cudaStream_t stream);
// x[t] += mult * (layernorm(m[t]) * w + bias), then xa[t] = x[t] in the operand type (xa may be null): the norm on a sublayer's result, the
// residual sum (fp32) and the next sublayer's operand in one pass
int launch_layernorm_affine_residual(const float * m, const float * w, const float * bias, float mult, float eps, float * x, void * xa, int otype, int n_rows,
                                     int width, cudaStream_t stream);
// y[i] = max(u[i], 0)^2 -> operand type
int launch_relu2(const float * u, void * y, int otype, int64_t n, cudaStream_t stream);
// x[i] <- cap * tanh(x[i] / cap), in place
int launch_softcap(float * x, int64_t n, float cap, cudaStream_t stream);
// x[t] += layernorm(m[t]) * w      (the post-norm of a sublayer and the residual sum, fp32)
int launch_layernorm_residual(const float * m, const float * w, float eps, float * x, int n_rows, int width, cudaStream_t stream);
// both at once: x[t] += layernorm(m[t]) * wa, then y[t] = layernorm(x[t]) * wb (the next sublayer's input)
int launch_layernorm_residual_next(const float * m, const float * wa, const float * wb, float eps, float * x, void * y, int otype, int n_rows, int width,
                                   cudaStream_t stream);
// y[t][j] = gelu_tanh(gu[t][j]) * gu[t][ff + j]       gu: [T][2 ff] f32
int launch_gelu_mul(const float * gu, void * y, int otype, int n_tokens, int ff, cudaStream_t stream);
// out[r] = first index of the maximum of logits[r][0..n)
int launch_argmax_rows(const float * logits, int n, int n_rows, int32_t * out, cudaStream_t stream);

// ---- attention with a sliding window and kept first tokens ----
struct AttnParams {
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
    float scale = 1.f;
    float softcap = 0.f;      // > 0: score <- softcap * tanh(score / softcap)
    int window = 0;           // position i sees j <= i with i - j < window ...   (<= 0: every earlier position)
    int keep_first = 0;       // ... or j < keep_first
    int cache_rows = 0;       // rows per slot: positions < keep_first at their own row, later ones in a ring over the rest
    int shared_dim = 0;       // prompt kernels: the last shared_dim of a key's dim entries come from one array all heads share
    int gated = 1;            // the fused projection ends with one gate logit per head (0: q | k | v only, the output is not gated)
    int sink = 0;             // 1: one is added to the softmax denominator (a key of score 0 that has no value)
};
// Where the attention kernels read their inputs (fp32 rows, strides in floats).  Prompt kernels read keys and values of the batch:
// k rows hold [kv_heads][dim - shared_dim], ks rows [shared_dim]; v rows [kv_heads][vdim].  Decode kernels read q and gate here and
// the keys / values from the cache, whose rows are k_row / v_row floats apart (kv head h at + h * dim / + h * vdim).
struct AttnIO {
    const float * q = nullptr;    int64_t ldq = 0;     // [heads][dim]
    const float * k = nullptr;    int64_t ldk = 0;
    const float * ks = nullptr;   int64_t ldks = 0;
    const float * v = nullptr;    int64_t ldv = 0;
    const float * gate = nullptr; int64_t ldg = 0;     // gate logits; the output is multiplied by their sigmoid
    int gate_mode = 0;                                  // 0: no gate, 1: one logit per head, 2: one per output element [heads][vdim]
    int64_t k_row = 0, v_row = 0;
};
__host__ __device__ inline int attn_qkvg_cols(const AttnParams & a) { return a.heads * a.dim + a.kv_heads * a.dim + a.kv_heads * a.vdim + (a.gated ? a.heads : 0); }
// rows of a slot's cache so that every position a later token may still see is present, capped at n_ctx
inline int attn_cache_rows(int window, int keep_first, int n_ctx) {
    if (window <= 0) return n_ctx;
    const int64_t need = (int64_t) keep_first + window;
    return (int) (need < n_ctx ? need : n_ctx);
}
// qkvg: [T][q | k | v | gate] f32 (one fused projection).  Stores the K / V rows that later tokens can still see.
// kcache / vcache: base of the layer run's cache, slot s at + s * slot_stride floats; rows of kv_heads*dim / kv_heads*vdim floats.
int launch_attn_kv_store(const float * qkvg, const BatchView & b, const AttnParams & a, float * kcache, float * vcache, int64_t slot_stride,
                         cudaStream_t stream);
// the same after an RMS norm of every query head (weight wq [dim]) and key head (wk [dim]) of the fused projection, in place:
// v <- v / sqrt(mean(v^2) + eps) * w per head; the cache receives the normed keys
int launch_attn_qknorm_kv_store(float * qkvg, const BatchView & b, const AttnParams & a, const float * wq, const float * wk, float eps, float * kcache,
                                float * vcache, int64_t slot_stride, cudaStream_t stream);
// entries that start at position 0: keys and values are read from the batch itself
int launch_attn_window_prefill(const float * qkvg, const BatchView & b, const AttnParams & a, void * out, int otype, cudaStream_t stream);
// one-token entries: keys and values come from the cache (the token's own row already stored).  part (may be null): scratch of
// attn_decode_part_floats floats; with it and a cache of 128 rows or more the rows are split over several CTAs per (head, entry) in chunks
// of attn_decode_chunk rows, and a second kernel merges the partial softmax states.  The split depends on the cache's row count alone.
inline int attn_decode_chunk(int cache_rows) {
    const int c = (cache_rows + 63) / 64;                 // at most 64 splits ...
    return c < 64 ? 64 : (c + 31) / 32 * 32;              // ... of at least 64 rows
}
inline int attn_decode_splits(int cache_rows) { return cache_rows < 128 ? 1 : (cache_rows + attn_decode_chunk(cache_rows) - 1) / attn_decode_chunk(cache_rows); }
inline size_t attn_decode_part_floats(const AttnParams & a, int n_entries) {
    return (size_t) n_entries * (size_t) a.heads * (size_t) attn_decode_splits(a.cache_rows) * (size_t) (a.vdim + 2);
}
int launch_attn_window_decode(const float * qkvg, const BatchView & b, const AttnParams & a, const float * kcache, const float * vcache,
                              int64_t slot_stride, void * out, int otype, cudaStream_t stream, float * part = nullptr);

// the same two kernels with every input given by an AttnIO
int launch_attn_prefill_io(const AttnIO & io, const BatchView & b, const AttnParams & a, void * out, int otype, cudaStream_t stream);
int launch_attn_decode_io(const AttnIO & io, const BatchView & b, const AttnParams & a, const float * kcache, const float * vcache, int64_t slot_stride,
                          void * out, int otype, cudaStream_t stream, float * part = nullptr);

// ---- Mamba-2 ----
struct Mamba2Params {
    int heads = 0, vdim = 0, state = 0, groups = 0, conv = 0, norm_groups = 0;
};
__host__ __device__ inline int mamba2_inner(const Mamba2Params & p) { return p.heads * p.vdim; }
__host__ __device__ inline int mamba2_conv_channels(const Mamba2Params & p) { return p.heads * p.vdim + 2 * p.groups * p.state; }
__host__ __device__ inline int mamba2_in_cols(const Mamba2Params & p) { return 2 * p.heads * p.vdim + 2 * p.groups * p.state + p.heads; }
// u: [T][z | x | B | C | dt] f32 (the input projection).  xbc[t][c] = silu(bias[c] + sum_d w[c][taps-1-d] * in(t - d)), inputs before
// the entry's first token come from the slot's convolution state [taps-1][channels] (zeros for a new sequence); then the state is
// advanced to the entry's last taps-1 inputs.
int launch_mamba2_conv(const float * u, const BatchView & b, const Mamba2Params & p, const float * w, const float * bias, float * conv_state,
                       int64_t slot_stride, float * xbc, cudaStream_t stream);
// selective scan per (entry, head) over the entry's tokens, state S [state][vdim] f32 per head carried in ssm_state:
//   dt = softplus(dt_raw + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x
int launch_mamba2_scan(const float * u, const float * xbc, const BatchView & b, const Mamba2Params & p, const float * dt_bias, const float * A_log,
                       const float * D, float * ssm_state, int64_t slot_stride, float * y, cudaStream_t stream);
// out[t] = rms_norm_by_group(y[t] * silu(z[t])) * w      (z = first inner columns of u)
int launch_mamba2_gate_norm(const float * y, const float * u, const Mamba2Params & p, const float * w, float eps, void * out, int otype, int n_tokens,
                            cudaStream_t stream);

// ---- RMS norm in groups, token shift, depth average ----
// y[r] = x[row] / sqrt(mean over the group (x^2) + eps) * w: the row is cut into `groups` equal consecutive parts, each with its own mean
int launch_group_rmsnorm(const float * x, const int32_t * rows, const float * w, int groups, float eps, void * y, int otype, int n_rows, int width,
                         cudaStream_t stream);
// h = group_rmsnorm(x);  y[t] = h[t] + (h[t-1] - h[t]) * mu, where the token before an entry's first one is the slot's shift state
// [width] (zeros for a new sequence); afterwards the state holds the h of the entry's last token.  mu == nullptr: y = h, no state.
int launch_group_rmsnorm_shift(const float * x, const BatchView & b, const float * w, int groups, float eps, const float * mu, float * shift_state,
                               int64_t slot_stride, void * y, int otype, int width, cudaStream_t stream);
// out[i] = sum_{j < n} coef[j] * planes[j * plane_stride + i],  i < count
int launch_depth_average(const float * planes, int64_t plane_stride, const float * coef, int n, float * out, int64_t count, cudaStream_t stream);

// batches of one-token entries only: x = the depth average above, then launch_group_rmsnorm_shift of x (the next layer's mixer input), one kernel
int launch_depth_average_norm_shift(const float * planes, int64_t plane_stride, const float * coef, int n, float * x, const BatchView & b, const float * w,
                                    int groups, float eps, const float * mu, float * shift_state, int64_t slot_stride, void * y, int otype, int width,
                                    cudaStream_t stream);

// ---- linear attention with a fixed decay per head ----
struct DecayAttnParams {
    int heads = 0, dim = 0, vdim = 0;
    int act = 0;              // 1: q, k, v <- silu(.) before the recurrence
    float k_scale = 1.f;      // factor on k
};
// qkv rows (stride ld floats) hold q [heads][dim] at q_off, k at k_off, v [heads][vdim] at v_off.  Per (entry, head), state S [dim][vdim]
// f32 carried in the slot:  S <- decay[h] S + k_t v_t^T,  y_t = S^T q_t.   y: [T][heads * vdim]
int launch_decay_attn(const float * qkv, int64_t ld, int q_off, int k_off, int v_off, const BatchView & b, const DecayAttnParams & p, const float * decay,
                      float * state, int64_t slot_stride, float * y, cudaStream_t stream);
// out[t] = y[t] / rms over each of `groups` consecutive parts (* w if w) * act(gate[t]);  act: 0 sigmoid, 1 silu;  gate rows ldg floats apart
// gate_act -1 (or gate == nullptr): no gate.  The result, times out_scale, goes to rows of ldo elements (0: inner).
int launch_norm_gate(const float * y, const float * gate, int64_t ldg, int groups, const float * w, int gate_act, float eps, void * out, int otype,
                     int n_tokens, int inner, cudaStream_t stream, int64_t ldo = 0, float out_scale = 1.f);

// ---- attention over a latent ----
struct LatentParams {
    int heads = 0, dim = 0, rot_dim = 0, vdim = 0, kv_rank = 0, q_rank = 0;
    int rot_dims = 0;         // leading entries of the rotated part that turn, in pairs (i, i + rot_dims / 2)
    float rot_mag = 1.f;      // factor on cos and sin
    float scale = 1.f;
    int cache_rows = 0;       // rows of kv_rank + rot_dim floats per slot: [normed latent | rotated shared key part] of every position
    int own_kv = 1;           // 0: the layer reads another layer's cache and has no down-projection of its own
};
__host__ __device__ inline int latent_proj_cols(const LatentParams & p) { return p.q_rank + p.heads * p.vdim + (p.own_kv ? p.kv_rank + p.rot_dim : 0); }
__host__ __device__ inline int latent_row(const LatentParams & p) { return p.kv_rank + p.rot_dim; }
// proj: [T][dq | gate | dkv] f32 (one fused projection; dkv only with own_kv).  cq[t] = rmsnorm(dq) * wq -> operand type;
// with own_kv: cache row of the token's position <- [rmsnorm(dkv[:kv_rank]) * wkv | rotate(dkv[kv_rank:], position)]
int launch_latent_prep(const float * proj, const BatchView & b, const LatentParams & p, const float * wq, const float * wkv, const float * freq, float eps,
                       void * cq, int otype, float * cache, int64_t slot_stride, cudaStream_t stream);
// rotates the last rot_dim entries of every head of q [T][heads][dim + rot_dim] in place by the token's position
int launch_latent_rope_q(float * q, const BatchView & b, const LatentParams & p, const float * freq, cudaStream_t stream);
// the batch's own cache rows: latent -> lat [T][kv_rank] (operand type), rotated key part -> kr [T][rot_dim] f32
int launch_latent_gather(const float * cache, int64_t slot_stride, const BatchView & b, const LatentParams & p, void * lat, int otype, float * kr,
                         cudaStream_t stream);
// decode: qa[t][h] = [ W_uk[h]^T q_unrotated[t][h]  (kv_rank) | rotate(q[t][h][dim:], position) (rot_dim) ]: the score against a cache row is
// one dot product.  q comes straight from the projection (not rotated yet).
int launch_latent_absorb_q(const float * q, const BatchView & b, const void * wuk, int wtype, const LatentParams & p, const float * freq, float * qa,
                           cudaStream_t stream);
// decode: out[t][h][:] = (W_uv[h] olat[t][h]) * sigmoid(gate[t][h][:])   olat: [T][heads][kv_rank] (the weighted sum of latents)
int launch_latent_up_v(const float * olat, const void * wuv, int wtype, const LatentParams & p, const float * gate, int64_t ldg, void * out, int otype,
                       int n_tokens, cudaStream_t stream);

// decode attention of one-token entries over the slot's rows, split over `splits` CTAs per (entry, 16 heads), then the merge, the
// value up-projection and the gate in a second kernel.  part: scratch of n_entries * splits * heads * (kv_rank + 2) floats.
inline int latent_decode_splits(int cache_rows) { return cache_rows >= 2048 ? 64 : cache_rows >= 64 ? cache_rows / 32 : 1; }
int launch_latent_decode(const float * qa, const BatchView & b, const LatentParams & p, const float * cache, int64_t slot_stride, int splits, float * part,
                         const void * wuv, int wtype, const float * gate, int64_t ldg, void * out, int otype, cudaStream_t stream);

// ---- clamped gated feed-forward, dense or a mixture of experts ----
// y[t][j] = g s(1.702 g) (u + 1),  g = min(gu[t][j], limit),  u = clamp(gu[t][ff + j], -limit, limit),  s = sigmoid     gu: [T][2 ff] f32
int launch_clamped_glu(const float * gu, void * y, int otype, int n_tokens, int ff, float limit, cudaStream_t stream);
struct MoeParams {
    int experts = 0, top = 0, ff = 0;
    float limit = 0.f;
    int act = 0;              // expert form: 0 = clamped gated unit (rows gate | up, 2 ff per expert), 1 = max(up, 0)^2 (rows up, ff per expert),
                              // 2 = SiLU gated unit silu(gate) * up (rows gate | up)
    int weight_on_input = 0;  // 1: a chosen expert's weight multiplies its INPUT (applied to the gate / up products, which are linear in it);
                              // the sum over the experts then takes no weights
    int norm_weights = 1;     // launch_moe_route_sigmoid: 1 = the chosen scores divided by their sum, 0 = the plain scores
    int groups = 1, keep_groups = 1;   // launch_moe_route_sigmoid: equal groups of neighbouring experts, of which the best keep_groups stay eligible
    float route_scale = 1.f;           // launch_moe_route_sigmoid: factor on the normalised weights
};
__host__ __device__ inline int moe_up_rows(const MoeParams & p) { return p.act == 1 ? p.ff : 2 * p.ff; }
// z = h W_r^T + bias in fp32 (h: the operand-type activations); idx[t][0..top) the experts with the largest z (ties: lower index),
// wt[t][..] the softmax over the chosen logits
int launch_moe_route(const void * h, int htype, const float * wr, const float * bias, const MoeParams & p, int width, int32_t * idx, float * wt,
                     int n_tokens, cudaStream_t stream);
// s = sigmoid(h W_r^T) in fp32; choice score c = s + correction; score of a group = its two largest c summed (its only one in a group of
// one); experts outside the keep_groups best groups are not eligible; idx[t][0..top) the eligible experts with the largest c (ties: lower
// index), wt[t][k] = s[idx] / (sum of the chosen s + 1e-20) * route_scale (norm_weights 0: s[idx] * route_scale).  correction may be null.
// shared_gate (may be null, then sg_out is not written):
// sg_out[t] = sigmoid(h . shared_gate), the factor on a shared expert's result.
int launch_moe_route_sigmoid(const void * h, int htype, const float * wr, const float * correction, const MoeParams & p, int width, const float * shared_gate,
                             int32_t * idx, float * wt, float * sg_out, int n_tokens, cudaStream_t stream);
// few tokens: every (token, chosen expert) streams its expert's rows.  y[t][k][ff] = act(expert idx[t][k] of gateup) -> operand type
// in_wt (weight_on_input): the pair's weight, a factor on its gate and up products
int launch_moe_gateup_rows(const void * h, int type, const void * gateup, const int32_t * idx, const MoeParams & p, int width, void * y, int n_tokens,
                           cudaStream_t stream, const float * in_wt = nullptr);
// y[r][j] = silu(s gu[r][j]) * (s gu[r][ff + j]),  s = in_wt ? in_wt[perm ? perm[r] : r] : 1      gu: [rows][2 ff] f32
int launch_silu_mul(const float * gu, void * y, int otype, int n_rows, int ff, const float * in_wt, const int32_t * perm, cudaStream_t stream);
// x[t] = base(x[t]) + sum_k wt[t][k] * down[idx[t][k]] y[t][k]      (k in the order of the choice)
// base: MOE_ADD x[t] itself, MOE_SET zero, MOE_SCALE x[t] * xscale[t] (a gated shared expert's result waits in x)
enum : int { MOE_ADD = 0, MOE_SET = 1, MOE_SCALE = 2 };
// wt == nullptr: every weight is one.  The sum is multiplied by out_scale before it meets the base.
int launch_moe_down_rows(const void * y, int type, const void * down, const int32_t * idx, const float * wt, const MoeParams & p, int width, float * x,
                         int n_tokens, cudaStream_t stream, int base = MOE_ADD, const float * xscale = nullptr, float out_scale = 1.f);
// many tokens: pairs (t, k) sorted by expert (stable).  count[e], start[e] (exclusive prefix), perm[r] = pair index t * top + k of sorted row r
int launch_moe_sort(const int32_t * idx, const MoeParams & p, int n_tokens, int32_t * count, int32_t * start, int32_t * perm, cudaStream_t stream);
// hs[r] = h[perm[r] / top]   (rows of `width` operand-type elements)
int launch_moe_gather(const void * h, int type, const int32_t * perm, int top, int width, void * hs, int n_rows, cudaStream_t stream);
// x[t] = base(x[t]) + sum_k wt[t][k] * ds[row_of[t * top + k]],  row_of = inverse of perm (computed by the kernel from perm)
int launch_moe_combine(const float * ds, const int32_t * perm, int32_t * row_of, const float * wt, int top, int width, float * x, int n_tokens,
                       cudaStream_t stream, int base = MOE_ADD, const float * xscale = nullptr, float out_scale = 1.f);

// ---- short causal convolution over a range of projection channels ----
// out[t][c] = act(sum_j w[c][j] * in(t - taps + 1 + j)[c]), c < channels, in(t) = u[t * ldu + c]; inputs before the entry's first token come
// from the slot's state [taps - 1][channels] (zeros for a new sequence), which then advances to the entry's last taps - 1 inputs.  No bias.
// act: channels >= silu_from pass SiLU, the ones below none.  w: [channels][taps].
int launch_causal_conv(const float * u, int64_t ldu, const BatchView & b, int channels, int taps, const float * w, int silu_from, float * conv_state,
                       int64_t slot_stride, float * out, int64_t ldo, cudaStream_t stream);

// ---- preparation of attention inputs, in place, and the cache store ----
enum : int { ROT_INTERLEAVED = 0, ROT_HALVES = 1 };   // pair (2i, 2i + 1), or (i, i + dims / 2)
enum : int { QKN_NONE = 0, QKN_HEAD_UNIT = 1, QKN_WHOLE_WEIGHT = 2 };
struct AttnPrep {
    int norm = QKN_NONE;          // QKN_HEAD_UNIT: every query / key head divided by its root mean square AFTER the rotation, no weight;
                                  // QKN_WHOLE_WEIGHT: RMS norm over all query rows at once (and all key rows) with weights wq / wk, BEFORE the rotation
    const float * wq = nullptr, * wk = nullptr;   // [heads * dim], [kv_heads * dim]
    float eps = 0.f;
    int rot_dims = 0;             // the leading rot_dims entries of every query / key head turn by position * rot_freq[i]
    int rot_layout = ROT_INTERLEAVED;
    const float * rot_freq = nullptr;   // [rot_dims / 2]
    int v_rot = 0;                // 1: every value head turns by its position over all vdim entries (pairs in v_layout, v_freq [vdim / 2]);
    int v_layout = ROT_INTERLEAVED;     // the cache holds the turned values and launch_attn_unrotate_gate turns a head's result back
    const float * v_freq = nullptr;
};
// q [T][heads][dim], k [T][kv_heads][dim], v [T][kv_heads][vdim] (rows ldq / ldk / ldv floats apart) are prepared in place; then the K / V
// rows that later tokens can still see go to the cache (layout as launch_attn_kv_store).
int launch_attn_prep_store(float * q, int64_t ldq, float * k, int64_t ldk, float * v, int64_t ldv, const BatchView & b, const AttnParams & a,
                           const AttnPrep & pr, float * kcache, float * vcache, int64_t slot_stride, cudaStream_t stream);
// o [T][heads][vdim] f32 (an attention result over values turned by their positions): every head is turned back by the token's position
// (v_freq == nullptr: not turned), multiplied by sigmoid of its gate logit (gate_mode as in AttnIO) and by out_scale -> out rows of ldo
// elements in the operand type
int launch_attn_unrotate_gate(const float * o, const BatchView & b, int heads, int vdim, int v_layout, const float * v_freq, const float * gate, int64_t ldg,
                              int gate_mode, float out_scale, void * out, int64_t ldo, int otype, cudaStream_t stream);

// the same with the preparation of a recurrent branch's inputs in front, one launch for both branches of a dual mixer: rec_kind 0 =
// launch_delta_prep(rq, rk, beta, ra, p0 = A_log, p1 = dt_bias), 1 = launch_hgrn2_prep(rq, rk = forget logits, p0 = f_bias, p1 = lower)
int launch_dual_prep_store(int rec_kind, float * rq, int64_t ldrq, float * rk, int64_t ldrk, float * beta, int64_t ldb, float * ra, int64_t lda, const float * p0,
                           const float * p1, int qk_heads, int r_heads, int r_dim, float * q, int64_t ldq, float * k, int64_t ldk, float * v, int64_t ldv,
                           const BatchView & b, const AttnParams & a, const AttnPrep & pr, float * kcache, float * vcache, int64_t slot_stride, cudaStream_t stream);
// launch_attn_unrotate_gate of the attention result o and launch_norm_gate (one group per head) of the recurrence's result y in one launch:
// out[t] = [ left_scale * gated, turned-back attention heads | right_scale * normed, weighted, gated recurrence heads ], rows of ldo elements
int launch_dual_post(const float * o, const BatchView & b, int heads, int vdim, int v_layout, const float * v_freq, const float * gate, int64_t ldg, int gate_mode,
                     float left_scale, const float * y, int r_heads, int r_vdim, const float * r_gate, int64_t ldrg, const float * r_w, int r_gate_act, float eps,
                     float right_scale, void * out, int64_t ldo, int otype, cudaStream_t stream);

// ---- gated linear recurrences: a state S [dim][vdim] f32 per (sequence slot, head) with a decay that every token brings ----
//   decay_per_channel 0: S <- g S (g [T][heads]);  1: S <- diag(f) S (f [T][qk_heads][dim])
//   delta 0: S <- S + k v^T;   1 (delta rule): u = beta (v - S^T k), S <- S + k u^T (beta [T][heads]), after the decay
//   tied_key 1: k = 1 - f (needs decay_per_channel; io.k unused)
//   y = S^T q, after the token's write.        Head h reads q / k head h / (heads / qk_heads).
struct GatedLinParams {
    int heads = 0, qk_heads = 0, dim = 0, vdim = 0;
    int decay_per_channel = 0, delta = 0, tied_key = 0;
};
struct GatedLinIO {
    const float * q = nullptr;      int64_t ldq = 0;    // [qk_heads][dim]
    const float * k = nullptr;      int64_t ldk = 0;
    const float * v = nullptr;      int64_t ldv = 0;    // [heads][vdim]
    const float * decay = nullptr;  int64_t ldd = 0;
    const float * beta = nullptr;   int64_t ldb = 0;
};
int launch_gated_linattn(const GatedLinIO & io, const BatchView & b, const GatedLinParams & p, float * state, int64_t slot_stride, float * y,
                         cudaStream_t stream);
// inputs of the gated delta rule, in place: every q / k head (qk_heads of each, dim wide) becomes x / sqrt(sum x^2 + 1e-6), q also times
// dim^-1/2;  beta <- sigmoid(beta);  a <- exp(-exp(A_log[h]) * softplus(a + dt_bias[h]))    (beta, a: [T][heads])
int launch_delta_prep(float * q, int64_t ldq, float * k, int64_t ldk, float * beta, int64_t ldb, float * a, int64_t lda, const float * A_log,
                      const float * dt_bias, int qk_heads, int heads, int dim, int n_tokens, cudaStream_t stream);
// inputs of HGRN2, in place: q <- silu(q);  f <- lower + (1 - lower) * sigmoid(f + f_bias)      (n = heads * dim entries per token)
int launch_hgrn2_prep(float * q, int64_t ldq, float * f, int64_t ldf, const float * f_bias, const float * lower, int n, int n_tokens, cudaStream_t stream);

// x[t] += (x0 ? x0[t] : 0) + (vec ? vec : 0), then y[t] = rmsnorm(x[t]) * w in the operand type: what opens a pass of a repeated block whose
// passes add the embedding output and a step vector, with the first layer's norm
int launch_stream_add_rmsnorm(float * x, const float * x0, const float * vec, const float * w, float eps, void * y, int otype, int n_rows, int width,
                              cudaStream_t stream);
// x[t] += mult * (rmsnorm(a[t]) * wa + rmsnorm(b[t]) * wb), then y[t] = rmsnorm(x[t]) * wn in the operand type (y may be null): two branch
// results joined after a norm each, the residual sum and the next sublayer's input in one pass.  a, b rows lda / ldb floats apart.
int launch_rmsnorm_pair_residual(const float * a, int64_t lda, const float * bb, int64_t ldb, const float * wa, const float * wb, float mult, float eps,
                                 float * x, const float * wn, void * y, int otype, int n_rows, int width, cudaStream_t stream);

}  // namespace pb
