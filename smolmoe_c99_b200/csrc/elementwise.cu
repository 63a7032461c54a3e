// Embedding gather, RMSNorm, SwiGLU, and the rotation of q and k with the cache write.
// Each works on float values; storage is float or bfloat16.
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace sm {

// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int32_t* __restrict__ tokens,
                                 float* __restrict__ out, int D, int V, int32_t* status) {
    pdl_launch_dependents();
    pdl_wait();   // the tokens may come from the sampler's kernel
    int t = blockIdx.x;
    int token = tokens[t];
    float* row = out + (size_t)t * D;
    if (token < 0 || token >= V) {
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        for (int d = threadIdx.x; d < D; d += blockDim.x) row[d] = 0.f;
        return;
    }
    const TW* src = table + (size_t)token * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) row[d] = to_float(src[d]);
}

void embedding(const void* table, DType table_dt, const int32_t* tokens, float* out, int T, int D,
               int V, int32_t* status, cudaStream_t stream) {
    if (T <= 0) return;
    note_launch();
    int threads = D >= 256 ? 256 : 128;
    if (table_dt == F32)
        launch_kernel("embedding", embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, 1, dependent_launch_enabled(),
                      (const float*)table, tokens, out, D, V, status);
    else
        launch_kernel("embedding", embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, 1,
                      dependent_launch_enabled(), (const __nv_bfloat16*)table, tokens, out, D, V, status);
}

// ---------------------------------------------------------------------------------------
// One block of kNormThreads per row. Every thread sums its strided elements in ascending
// order, the warp sums with a butterfly, and warp 0 adds the warps' sums in warp order: the
// order of additions depends only on D.
constexpr int kNormThreads = 256;

template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, float eps,
                               TO* __restrict__ out, const int32_t* __restrict__ rows, int D) {
    __shared__ float warp_part[kNormThreads / 32];
    __shared__ float inv_shared;
    int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float sq = 0.f;
    for (int d = threadIdx.x; d < D; d += kNormThreads) {
        float v = xr[d];
        sq = fmaf(v, v, sq);
    }
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
#pragma unroll
        for (int i = 0; i < kNormThreads / 32; ++i) total += warp_part[i];
        inv_shared = 1.0f / sqrtf(total / (float)D + eps);
    }
    __syncthreads();
    float inv = inv_shared;
    TO* o = out + (size_t)r * D;
    for (int d = threadIdx.x; d < D; d += kNormThreads) o[d] = from_float<TO>((xr[d] * inv) * to_float(w[d]));
}

void rmsnorm(const float* x, const void* w, DType w_dt, float eps, void* out, DType out_dt,
             const int32_t* rows, int n_rows, int D, cudaStream_t stream) {
    if (n_rows <= 0) return;
    note_launch();
#define SM_NORM(TW, TO) \
    rmsnorm_kernel<TW, TO><<<n_rows, kNormThreads, 0, stream>>>(x, (const TW*)w, eps, (TO*)out, rows, D)
    if (w_dt == F32 && out_dt == F32) SM_NORM(float, float);
    else if (w_dt == F32 && out_dt == BF16) SM_NORM(float, __nv_bfloat16);
    else if (w_dt == BF16 && out_dt == F32) SM_NORM(__nv_bfloat16, float);
    else SM_NORM(__nv_bfloat16, __nv_bfloat16);
#undef SM_NORM
}

// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gate_up, TO* __restrict__ out, int H, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t t = i / H;
    int j = (int)(i - t * H);
    float g = gate_up[t * 2 * H + j];
    float u = gate_up[t * 2 * H + H + j];
    out[i] = from_float<TO>(u * (g / (1.0f + expf(-g))));
}

void swiglu(const float* gate_up, void* out, DType out_dt, int T, int H, cudaStream_t stream) {
    size_t total = (size_t)T * H;
    if (!total) return;
    note_launch();
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dt == F32) swiglu_kernel<float><<<blocks, 256, 0, stream>>>(gate_up, (float*)out, H, total);
    else swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(gate_up, (__nv_bfloat16*)out, H, total);
}

// ---------------------------------------------------------------------------------------
// One block per token; one thread per pair of elements of one head (q heads, then k heads,
// then v heads).
template <typename TO>
__global__ void rope_store_kernel(RopeStoreArgs a) {
    int t = blockIdx.x;
    int hd = a.head_dim, half = hd / 2, rhalf = a.rotary_dim / 2;
    int n_heads = a.heads + 2 * a.kv_heads;
    int pos = a.positions[t];
    const float* row = a.qkv + (size_t)t * n_heads * hd;
    bool to_cache = a.k_pool != nullptr;
    int slot = 0;
    if (to_cache) {
        slot = a.token_slot[t];
        // a windowed group keeps `ring` positions: older tokens of a long prompt are not stored
        if (a.ring > 0 && pos < a.token_end[t] - a.ring) to_cache = false;
    }
    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};
    for (int j = threadIdx.x; j < n_heads * half; j += blockDim.x) {
        int head = j / half, i = j - head * half;
        const float* x = row + (size_t)head * hd;
        int d0, d1;
        float v0, v1;
        bool is_v = head >= a.heads + a.kv_heads;
        if (i < rhalf) { d0 = i; d1 = i + rhalf; } else { d0 = a.rotary_dim + 2 * (i - rhalf); d1 = d0 + 1; }
        v0 = x[d0];
        v1 = x[d1];
        if (!is_v && i < rhalf) {
            float c = a.cos_table[(size_t)pos * rhalf + i], s = a.sin_table[(size_t)pos * rhalf + i];
            float r0 = v0 * c - v1 * s;
            float r1 = v0 * s + v1 * c;
            v0 = r0;
            v1 = r1;
        }
        TO o0 = from_float<TO>(v0), o1 = from_float<TO>(v1);
        if (head < a.heads) {
            TO* q = (TO*)a.q_out + ((size_t)t * a.heads + head) * hd;
            q[d0] = o0;
            q[d1] = o1;
        } else {
            int kvh = is_v ? head - a.heads - a.kv_heads : head - a.heads;
            TO* packed = (TO*)(is_v ? a.v_packed : a.k_packed);
            if (packed) {
                TO* p = packed + ((size_t)t * a.kv_heads + kvh) * hd;
                p[d0] = o0;
                p[d1] = o1;
            }
            if (to_cache) {
                TO* c = (TO*)(is_v ? a.v_pool : a.k_pool) + paged.row_offset(slot, pos, kvh);
                c[d0] = o0;
                c[d1] = o1;
            }
        }
    }
}

void rope_store(const RopeStoreArgs& a, cudaStream_t stream) {
    if (a.T <= 0) return;
    if (a.head_dim % 2 || a.rotary_dim % 2 || a.rotary_dim > a.head_dim)
        throw std::invalid_argument("rope_store: head_dim " + std::to_string(a.head_dim) + " / rotary_dim " +
                                    std::to_string(a.rotary_dim) + " must be even, rotary_dim <= head_dim");
    note_launch();
    int work = (a.heads + 2 * a.kv_heads) * a.head_dim / 2;
    int threads = work >= 512 ? 256 : (work >= 128 ? 128 : 64);
    if (a.dt == F32) rope_store_kernel<float><<<a.T, threads, 0, stream>>>(a);
    else rope_store_kernel<__nv_bfloat16><<<a.T, threads, 0, stream>>>(a);
}

}  // namespace sm
