// out[t, n] (+)= sum_k x[t, k] * w[n, k] + bias[n] on the CUDA cores in float.
//
// This is the matrix product of the true 32-bit path, and the fallback of the bfloat16
// path for shapes the tensor-core kernel refuses. Every output element is one chain of
// fmaf over k = 0..K-1, so its value does not depend on T, on the tile it falls in, or on
// what else is in the batch (the reference keeps the same promise for its dot products:
// src/kernels.h:5-7, src/kernels.c:35-39).
#include <stdexcept>

#include "common.cuh"
#include "kernels.h"

namespace sm {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TX, typename TW, typename TB, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const TB* __restrict__ bias,
                 TO* __restrict__ out, int T, int N, int K, bool accumulate) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    int t0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    int tid = threadIdx.x;
    int ty = tid / 16, tx = tid % 16;  // this thread: rows ty*4.., columns tx*4..
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k of each operand: 1024 elements, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int idx = tid + e * 256;
            int r = idx / BK, kk = idx % BK;
            int k = k0 + kk;
            float xv = 0.f, wv = 0.f;
            if (k < K) {
                if (t0 + r < T) xv = to_float(x[(size_t)(t0 + r) * K + k]);
                if (n0 + r < N) wv = to_float(w[(size_t)(n0 + r) * K + k]);
            }
            xs[kk][r] = xv;
            ws[kk][r] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += to_float(bias[n]);
            size_t o = (size_t)t * N + n;
            if (accumulate) v += to_float(out[o]);
            out[o] = from_float<TO>(v);
        }
    }
}

// The same product for up to 16 tokens (decode steps of the 32-bit path): the tile above would leave all but a few SMs
// idle (one CTA per 64 weight rows, K walked by that one CTA). Here a CTA takes 16 weight rows and one thread one
// output, still as ONE chain of fmaf over k = 0..K-1 in the same operand order, so the bits are those of the tile
// above; the operands come through shared memory in blocks of 64 of K.
constexpr int SR = 16, ST = 16, SK = 64;

template <typename TX, typename TW, typename TB, typename TO>
__global__ void __launch_bounds__(SR * ST)
gemm_simt_small_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const TB* __restrict__ bias,
                       TO* __restrict__ out, int T, int N, int K, bool accumulate) {
    __shared__ float xs[ST][SK + 1];
    __shared__ float ws[SR][SK + 1];
    const int n0 = blockIdx.x * SR;
    const int tid = threadIdx.x, r = tid / ST, t = tid % ST;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += SK) {
#pragma unroll
        for (int e = 0; e < (SR * SK) / (SR * ST); ++e) {
            const int idx = tid + e * SR * ST;
            const int row = idx / SK, kk = idx % SK, k = k0 + kk;
            xs[row][kk] = (k < K && row < T) ? to_float(x[(size_t)row * K + k]) : 0.f;
            ws[row][kk] = (k < K && n0 + row < N) ? to_float(w[(size_t)(n0 + row) * K + k]) : 0.f;
        }
        __syncthreads();
        const int span = min(SK, K - k0);
        if (span == SK) {
#pragma unroll
            for (int kk = 0; kk < SK; ++kk) acc = fmaf(xs[t][kk], ws[r][kk], acc);
        } else {
            for (int kk = 0; kk < span; ++kk) acc = fmaf(xs[t][kk], ws[r][kk], acc);
        }
        __syncthreads();
    }
    const int n = n0 + r;
    if (t >= T || n >= N) return;
    float v = acc;
    if (bias) v += to_float(bias[n]);
    const size_t o = (size_t)t * N + n;
    if (accumulate) v += to_float(out[o]);
    out[o] = from_float<TO>(v);
}

template <typename TX, typename TW, typename TB>
static void launch_out(const void* x, const void* w, const void* bias, void* out, DType out_dt, int T, int N,
                       int K, bool accumulate, cudaStream_t stream) {
    if (T <= ST) {
        const unsigned blocks = (unsigned)((N + SR - 1) / SR);
        if (out_dt == F32)
            gemm_simt_small_kernel<TX, TW, TB, float><<<blocks, SR * ST, 0, stream>>>((const TX*)x, (const TW*)w, (const TB*)bias,
                                                                                     (float*)out, T, N, K, accumulate);
        else
            gemm_simt_small_kernel<TX, TW, TB, __nv_bfloat16><<<blocks, SR * ST, 0, stream>>>(
                (const TX*)x, (const TW*)w, (const TB*)bias, (__nv_bfloat16*)out, T, N, K, accumulate);
        return;
    }
    dim3 grid((N + BN - 1) / BN, (T + BM - 1) / BM);
    if (out_dt == F32)
        gemm_simt_kernel<TX, TW, TB, float><<<grid, 256, 0, stream>>>((const TX*)x, (const TW*)w, (const TB*)bias,
                                                                     (float*)out, T, N, K, accumulate);
    else
        gemm_simt_kernel<TX, TW, TB, __nv_bfloat16><<<grid, 256, 0, stream>>>(
            (const TX*)x, (const TW*)w, (const TB*)bias, (__nv_bfloat16*)out, T, N, K, accumulate);
}

template <typename TX, typename TW>
static void launch_bias(const void* x, const void* w, const void* bias, DType bias_dt, void* out, DType out_dt,
                        int T, int N, int K, bool accumulate, cudaStream_t stream) {
    if (bias_dt == F32) launch_out<TX, TW, float>(x, w, bias, out, out_dt, T, N, K, accumulate, stream);
    else launch_out<TX, TW, __nv_bfloat16>(x, w, bias, out, out_dt, T, N, K, accumulate, stream);
}

void gemm_simt(const void* x, DType x_dt, const void* w, DType w_dt, const void* bias, DType bias_dt, void* out,
               DType out_dt, int T, int N, int K, bool accumulate, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return;
    if (K <= 0) throw std::invalid_argument("gemm_simt: K must be positive");
    if ((T + BM - 1) / BM > 65535) throw std::invalid_argument("gemm_simt: more than 65535*64 rows in one call");
    note_launch();
    if (x_dt == F32 && w_dt == F32) launch_bias<float, float>(x, w, bias, bias_dt, out, out_dt, T, N, K, accumulate, stream);
    else if (x_dt == F32) launch_bias<float, __nv_bfloat16>(x, w, bias, bias_dt, out, out_dt, T, N, K, accumulate, stream);
    else if (w_dt == F32) launch_bias<__nv_bfloat16, float>(x, w, bias, bias_dt, out, out_dt, T, N, K, accumulate, stream);
    else launch_bias<__nv_bfloat16, __nv_bfloat16>(x, w, bias, bias_dt, out, out_dt, T, N, K, accumulate, stream);
}

}  // namespace sm
