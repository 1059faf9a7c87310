// prima.cpp_b200/csrc/dense.cu — products with dense f32 / bf16 weight matrices stored [out][in]:
//   C[t][n] = alpha * sum_k A[t][k] W[n][k] (+ bias[n]) (+ resid[t][n])
// Three kernels behind one launcher:
//   k_dense_rows   up to 4 tokens (decode): one warp streams one weight row with 16-byte loads and keeps one fp32 accumulator per token;
//                  the launch is bound by the HBM read of W
//   k_dense_tc     bf16, 5 tokens and more (decode batches, prompts): tcgen05.mma with the accumulator in TMEM (dense_tc.cu)
//   k_dense_tile   everything else (true-fp32 products, ragged shapes): shared-memory tiles, fp32 fused multiply-add
// No kernel splits K across CTAs or uses atomics: an output element is one fixed-order sum, whatever else is in the batch.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>

#include "layers.h"

extern std::atomic<uint64_t> g_launches;

namespace pb {

int launch_dense_tc(const __nv_bfloat16 * A, int64_t lda, const __nv_bfloat16 * W, int64_t ldw, float * C, int64_t ldc, int T, int N, int K,
                    const float * bias, const float * resid, int64_t ldr, float alpha, cudaStream_t stream);   // dense_tc.cu
bool dense_tc_ok(int T, int N, int K, int64_t lda, int64_t ldw, const void * A, const void * W);
int launch_dense_tc_grouped(const __nv_bfloat16 * A, int64_t lda, const __nv_bfloat16 * W, int64_t ldw, int64_t w_stride, float * C, int64_t ldc,
                            const int32_t * start, const int32_t * count, int groups, int max_rows, int N, int K, cudaStream_t st);

namespace {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }

// ---------------------------------------------------------------------------------------------------------------
// tiled kernel: 64 tokens x 64 outputs per CTA, K in steps of 16, 256 threads with a 4 x 4 register tile each
constexpr int TM = 64, TN = 64, TK = 16;

template <typename WT>
__global__ void __launch_bounds__(256) k_dense_tile(const WT * __restrict__ A, int64_t lda, const WT * __restrict__ W, int64_t ldw, float * C, int64_t ldc,
                                                    int T, int N, int K, const float * __restrict__ bias, const float * resid, int64_t ldr, float alpha) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Ws[TK][TN + 4];
    const int t0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;   // outputs n0 + tx*4 .. +3, tokens t0 + ty*4 .. +3
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    const int lr = tid >> 2, lk = (tid & 3) * 4;   // this thread stages row lr, k offsets lk .. lk+3 of both tiles
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            const int t = t0 + lr, n = n0 + lr;
            As[lk + j][lr] = (t < T && k < K) ? to_f(A[(int64_t) t * lda + k]) : 0.f;
            Ws[lk + j][lr] = (n < N && k < K) ? to_f(W[(int64_t) n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; k++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = alpha * acc[i][j];
            if (bias) v += bias[n];
            if (resid) v += resid[(int64_t) t * ldr + n];
            C[(int64_t) t * ldc + n] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// few tokens: one warp per weight row.  VEC: the row is read with 16-byte loads (K a multiple of the vector, aligned rows).
template <typename WT> struct Vec16;
template <> struct Vec16<float> { static constexpr int n = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int n = 8; };

template <int N> __device__ __forceinline__ void unpack(const uint4 & raw, float (&f)[N], float) {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
}
template <int N> __device__ __forceinline__ void unpack(const uint4 & raw, float (&f)[N], __nv_bfloat16) {
    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(r[i] << 16);
        f[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
    }
}

// KS warps share a weight row (each takes a contiguous part of K, a multiple of the 16-byte load step; the parts are summed in order
// through shared memory): matrices with few, long rows keep more loads in flight that way.  KS comes from (N, K) alone.
template <typename WT, int TB, bool VEC>
__global__ void __launch_bounds__(256) k_dense_rows(const WT * __restrict__ A, int64_t lda, const WT * __restrict__ W, int64_t ldw, float * C, int64_t ldc,
                                                    int T, int N, int K, const float * __restrict__ bias, const float * resid, int64_t ldr, float alpha,
                                                    int KS) {
    __shared__ float parts[8][TB];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rows_per_cta = (blockDim.x >> 5) / KS;
    const int n = blockIdx.x * rows_per_cta + warp / KS, part = warp % KS;
    const bool live = n < N;
    constexpr int V = Vec16<WT>::n;
    const int Kc = KS == 1 ? K : ((K + KS - 1) / KS + 32 * V - 1) / (32 * V) * (32 * V);
    const int k_begin = part * Kc, k_end = min(K, k_begin + Kc);
    const WT * w = W + (int64_t) (live ? n : 0) * ldw;
    float acc[TB];
#pragma unroll
    for (int t = 0; t < TB; t++) acc[t] = 0.f;
    if (live) {
        if (VEC) {
            for (int k = k_begin + lane * V; k < k_end; k += 32 * V) {
                float wf[V];
                unpack<V>(__ldcs(reinterpret_cast<const uint4 *>(w + k)), wf, WT());   // streamed once: do not keep in L1
#pragma unroll
                for (int t = 0; t < TB; t++) {
                    if (t < T) {
                        float af[V];
                        unpack<V>(__ldg(reinterpret_cast<const uint4 *>(A + (int64_t) t * lda + k)), af, WT());
#pragma unroll
                        for (int i = 0; i < V; i++) acc[t] = fmaf(af[i], wf[i], acc[t]);
                    }
                }
            }
        } else {
            for (int k = k_begin + lane; k < k_end; k += 32) {
                const float wv = to_f(w[k]);
#pragma unroll
                for (int t = 0; t < TB; t++)
                    if (t < T) acc[t] = fmaf(to_f(A[(int64_t) t * lda + k]), wv, acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TB; t++) {
        float v = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[t] = v;
    }
    if (KS > 1) {
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < TB; t++) parts[warp][t] = acc[t];
        }
        __syncthreads();
        if (part != 0) return;
#pragma unroll
        for (int t = 0; t < TB; t++) {
            float v = 0.f;
            for (int j = 0; j < KS; j++) v += parts[warp + j][t];
            acc[t] = v;
        }
    }
    if (lane == 0 && live) {
#pragma unroll
        for (int t = 0; t < TB; t++) {
            if (t < T) {
                float v = acc[t] * alpha;
                if (bias) v += bias[n];
                if (resid) v += resid[(int64_t) t * ldr + n];
                C[(int64_t) t * ldc + n] = v;
            }
        }
    }
}

constexpr int ROWS_MAX_T = 8;
// Largest batch the weight-streaming kernel takes when the tensor-core kernel could run instead.  Measured on a B200 at 28672 x 4096 bf16:
// 8 tokens stream at 1.9 TB/s through this kernel (one L1 read of the activations per token and weight chunk) and at 3.3 TB/s through
// the tensor-core kernel's 64-token tile, so the hand-over is at 4.  PB200_DENSE_ROWS_MAX overrides for A/B runs.
int rows_max_t() {
    static const int v = [] {
        const char * e = getenv("PB200_DENSE_ROWS_MAX");
        const int n = e ? atoi(e) : 4;
        return n < 0 ? 0 : (n > ROWS_MAX_T ? ROWS_MAX_T : n);
    }();
    return v;
}

template <typename WT>
int dense_typed(const WT * A, int64_t lda, const WT * W, int64_t ldw, float * C, int64_t ldc, int T, int N, int K, const float * bias,
                const float * resid, int64_t ldr, float alpha, cudaStream_t st) {
    if (T <= ROWS_MAX_T) {
        constexpr int V = Vec16<WT>::n;
        const bool vec = K % V == 0 && lda % V == 0 && ldw % V == 0 && ((uintptr_t) A & 15) == 0 && ((uintptr_t) W & 15) == 0;
        // warps per row: few rows leave most of the machine's load slots empty, so 2, 4 or 8 warps split a long row
        int KS = 1;
        while (KS < 8 && (int64_t) N * KS < 6144 && K / (2 * KS) >= 1024) KS *= 2;
        const dim3 grid((unsigned) ((N + 8 / KS - 1) / (8 / KS))), block(256);
        g_launches++;
        if (T <= 1) {
            if (vec) k_dense_rows<WT, 1, true><<<grid, block, 0, st>>>(A, lda, W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, KS);
            else k_dense_rows<WT, 1, false><<<grid, block, 0, st>>>(A, lda, W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, KS);
        } else if (T <= 4) {
            if (vec) k_dense_rows<WT, 4, true><<<grid, block, 0, st>>>(A, lda, W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, KS);
            else k_dense_rows<WT, 4, false><<<grid, block, 0, st>>>(A, lda, W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, KS);
        } else {
            if (vec) k_dense_rows<WT, ROWS_MAX_T, true><<<grid, block, 0, st>>>(A, lda, W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, KS);
            else k_dense_rows<WT, ROWS_MAX_T, false><<<grid, block, 0, st>>>(A, lda, W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, KS);
        }
        return (int) cudaGetLastError();
    }
    const dim3 grid((unsigned) ((N + TN - 1) / TN), (unsigned) ((T + TM - 1) / TM)), block(256);
    g_launches++;
    k_dense_tile<WT><<<grid, block, 0, st>>>(A, lda, W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha);
    return (int) cudaGetLastError();
}

}  // namespace

int dense_uses_tensor_cores(int type, int T, int N, int K, int64_t lda, int64_t ldw) {
    return type == T_BF16 && T > rows_max_t() && dense_tc_ok(T, N, K, lda, ldw, nullptr, nullptr) ? 1 : 0;
}

int dense_grouped_ok(int type, int N, int K, int64_t lda, int64_t ldw, int64_t w_stride, const void * A, const void * W) {
    return type == T_BF16 && w_stride % 8 == 0 && dense_tc_ok(1, N, K, lda, ldw, A, W) ? 1 : 0;
}
int launch_dense_grouped(int type, const void * A, int64_t lda, const void * W, int64_t ldw, int64_t w_stride, float * C, int64_t ldc, const int32_t * start,
                         const int32_t * count, int groups, int max_rows, int N, int K, cudaStream_t st) {
    if (!dense_grouped_ok(type, N, K, lda, ldw, w_stride, A, W)) return (int) cudaErrorInvalidValue;
    return launch_dense_tc_grouped((const __nv_bfloat16 *) A, lda, (const __nv_bfloat16 *) W, ldw, w_stride, C, ldc, start, count, groups, max_rows, N, K, st);
}

int launch_dense(int type, const void * A, int64_t lda, const void * W, int64_t ldw, float * C, int64_t ldc, int T, int N, int K, const float * bias,
                 const float * resid, int64_t ldr, float alpha, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || !A || !W || !C) return (int) cudaErrorInvalidValue;
    if (type == 0 /* T_F32 */) return dense_typed<float>((const float *) A, lda, (const float *) W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, st);
    if (type != T_BF16) return (int) cudaErrorInvalidValue;
    if (T > rows_max_t() && dense_tc_ok(T, N, K, lda, ldw, A, W))
        return launch_dense_tc((const __nv_bfloat16 *) A, lda, (const __nv_bfloat16 *) W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, st);
    return dense_typed<__nv_bfloat16>((const __nv_bfloat16 *) A, lda, (const __nv_bfloat16 *) W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, st);
}

}  // namespace pb
