// Attention of one query against its visible keys, one CTA of eight warps per (token, head), for any
// head size that is a multiple of 8 up to 256 and any number of heads and groups.
//
// It is the attention of the true 32-bit path (whole prompts, prompts in portions, single
// tokens and any mix of them in one step) and the fallback of the bfloat16 path. Keys are visited in groups of 32 counted
// from the first visible key: warp w takes the groups w, w + 8, ... in ascending order with a running maximum and sum
// of its own, and the eight warps' results are put together in the order of the warps (the reference's two-pass softmax,
// src/kernels.c:1138-1176, gives the same value up to rounding). The number of warps is the same in every launch, so
// what a query's result depends on is the query, its visible keys and values, the scale and the window -- not the
// batch, not the step it came in, not where the keys lie in the cache. (One warp a query left a decode step of 8
// sequences over 2,048 positions with 112 warps on the whole GPU: 33 of the step's 46 ms.)
#include <math_constants.h>

#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"

namespace sm {

constexpr int kWarpsPerBlock = 8;      // the warps that share one query's keys
constexpr int kMaxHeadDim = 256;

template <typename T> struct Load8;
template <> struct Load8<float> {
    __device__ __forceinline__ static void load(const float* p, float (&v)[8]) {
        float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
template <> struct Load8<__nv_bfloat16> {
    __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
};

// SRC says where keys and values lie: 0 packed beside the queries (the step's own tokens), 1 in the cache, 2 both
// (positions before the first one the sequence brings in this step in the cache, the step's own packed).
template <typename T, int SRC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) attention_plain_kernel(AttentionArgs a) {
    __shared__ __align__(16) float q_shared[kMaxHeadDim];
    __shared__ float warp_m[kWarpsPerBlock], warp_l[kWarpsPerBlock];
    __shared__ float warp_acc[kWarpsPerBlock][kMaxHeadDim];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long item = blockIdx.x;
    int t = (int)(item / a.heads), h = (int)(item % a.heads);
    int hd = a.head_dim;
    int kvh = h / (a.heads / a.kv_heads);  // src/model.c:461
    int pos = a.positions[t];
    int start = (a.window > 0 && pos >= a.window) ? pos - a.window + 1 : 0;  // src/model.c:462

    const T* q = (const T*)a.q + ((size_t)t * a.heads + h) * hd;
    float* qs = q_shared;
    for (int d = threadIdx.x; d < hd; d += kWarpsPerBlock * 32) qs[d] = to_float(q[d]);
    __syncthreads();

    constexpr unsigned long long kPackedBit = 1ull << 63;   // marks a row offset into the packed tensors
    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};
    int slot = SRC != 0 ? a.token_slot[t] : 0;
    int seq_first = SRC != 1 ? a.token_seq_start[t] : 0;   // packed index of the sequence's first token of this step
    int pos0 = SRC != 1 ? pos - (t - seq_first) : 0;        // ... and its position

    float m = -CUDART_INF_F, l = 0.f;
    float acc[kMaxHeadDim / 32];
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.f;

    for (int base = start + 32 * warp; base <= pos; base += 32 * kWarpsPerBlock) {
        int p = base + lane;
        bool valid = p <= pos;
        unsigned long long row = 0;
        float s = -CUDART_INF_F;
        if (valid) {
            bool packed = SRC == 0 || (SRC == 2 && p >= pos0);
            row = packed ? (((unsigned long long)(seq_first + p - pos0) * a.kv_heads + kvh) * hd) | kPackedBit
                         : (unsigned long long)paged.row_offset(slot, p, kvh);
            const T* kr = (const T*)(packed ? a.k_packed : a.k_pool) + (row & ~kPackedBit);
            float dot = 0.f;
            for (int d = 0; d < hd; d += 8) {
                float kv[8];
                Load8<T>::load(kr + d, kv);
#pragma unroll
                for (int e = 0; e < 8; ++e) dot = fmaf(qs[d + e], kv[e], dot);
            }
            s = dot * a.scale;
        }
        float m_new = fmaxf(m, warp_max(s));
        float corr = expf(m - m_new);  // first group: exp(-inf) = 0
        float e = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(e);
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= corr;
        int n_valid = min(32, pos - base + 1);
        // the values of 8 keys at a time are asked for before they are used (one row a trip to memory otherwise); they are
        // still added in ascending key order, one fmaf chain per output dimension
        for (int j0 = 0; j0 < n_valid; j0 += 8) {
            float pj[8];
            float vv[8][kMaxHeadDim / 32];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int j = j0 + u;      // (lanes past n_valid hold e = 0 and row 0 of their source: harmless to read)
                pj[u] = __shfl_sync(0xffffffffu, e, j & 31);
                const unsigned long long rj = __shfl_sync(0xffffffffu, row, j & 31);
                const bool use = j < n_valid;
                const T* vr = (const T*)((rj & kPackedBit) ? a.v_packed : a.v_pool) + (rj & ~kPackedBit);
#pragma unroll
                for (int i = 0; i < kMaxHeadDim / 32; ++i) {
                    const int d = lane + 32 * i;
                    vv[u][i] = (use && d < hd) ? to_float(vr[d]) : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (j0 + u < n_valid) {
#pragma unroll
                    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = fmaf(pj[u], vv[u][i], acc[i]);
                }
            }
        }
        m = m_new;
    }
    // the warps' results, put together in the order of the warps (a warp without a group: m = -inf, weight 0)
    if (lane == 0) { warp_m[warp] = m; warp_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        int d = lane + 32 * i;
        if (d < hd) warp_acc[warp][d] = acc[i];
    }
    __syncthreads();
    float top = warp_m[0];          // (warp 0 always has the first group, which holds a visible key)
#pragma unroll
    for (int w = 1; w < kWarpsPerBlock; ++w) top = fmaxf(top, warp_m[w]);
    float weight[kWarpsPerBlock];
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsPerBlock; ++w) {
        weight[w] = expf(warp_m[w] - top);      // exp(-inf) = 0
        sum = fmaf(warp_l[w], weight[w], sum);
    }
    float inv = 1.0f / sum;
    T* o = (T*)a.out + ((size_t)t * a.heads + h) * hd;
    for (int d = threadIdx.x; d < hd; d += kWarpsPerBlock * 32) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsPerBlock; ++w) v = fmaf(warp_acc[w][d], weight[w], v);
        o[d] = from_float<T>(v * inv);
    }
}

void attention_plain(const AttentionArgs& a, cudaStream_t stream) {
    if (a.T <= 0) return;
    if (a.head_dim % 8 || a.head_dim > kMaxHeadDim || a.head_dim <= 0)
        throw std::invalid_argument("attention_plain: head_dim " + std::to_string(a.head_dim) +
                                    " must be a multiple of 8 between 8 and 256");
    if (a.heads % a.kv_heads)
        throw std::invalid_argument("attention_plain: kv_heads must divide heads");
    int src = a.k_packed == nullptr ? 1 : (a.k_pool == nullptr ? 0 : 2);
    if (src != 0 && (a.k_pool == nullptr || a.page_table == nullptr || a.token_slot == nullptr))
        throw std::invalid_argument("attention_plain: neither packed keys nor a cache were given");
    if (src != 1 && (a.v_packed == nullptr || a.token_seq_start == nullptr))
        throw std::invalid_argument("attention_plain: packed keys need packed values and each token's sequence start");
    note_launch();
    long long items = (long long)a.T * a.heads;
    if (items > 0x7fffffffll) throw std::invalid_argument("attention_plain: more than 2^31 - 1 (token, head) pairs in one step");
    unsigned blocks = (unsigned)items;
    int threads = kWarpsPerBlock * 32;
    if (a.dt == F32) {
        if (src == 0) attention_plain_kernel<float, 0><<<blocks, threads, 0, stream>>>(a);
        else if (src == 1) attention_plain_kernel<float, 1><<<blocks, threads, 0, stream>>>(a);
        else attention_plain_kernel<float, 2><<<blocks, threads, 0, stream>>>(a);
    } else {
        if (src == 0) attention_plain_kernel<__nv_bfloat16, 0><<<blocks, threads, 0, stream>>>(a);
        else if (src == 1) attention_plain_kernel<__nv_bfloat16, 1><<<blocks, threads, 0, stream>>>(a);
        else attention_plain_kernel<__nv_bfloat16, 2><<<blocks, threads, 0, stream>>>(a);
    }
}

}  // namespace sm
