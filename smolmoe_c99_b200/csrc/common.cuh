// Shared device helpers: element load/store for float and bfloat16 storage (all arithmetic
// is done in float), warp reductions with a fixed order, and the page arithmetic of the
// key/value cache.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm {

// Positions per cache page. The cache hands out storage in units of this many positions.
constexpr int kPageSize = 64;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// The activations of a gated feed-forward, act(gate) * up, in one place: a new one is added here (and named in
// kernels/ops.py); every kernel that folds the activation into a product's epilogue calls these.
enum Activation : int { ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_COUNT = 2 };
// exact library functions: the stand-alone kernel and the kernels of the 32-bit path
__device__ __forceinline__ float activate(int act, float g) {
    if (act == ACT_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + expf(-g));                       // x * sigmoid(x): src/vecmath.c:78-81 of the reference
}
// the hardware's exponential and reciprocal (a few ulp of float): epilogues whose result is stored as bfloat16
__device__ __forceinline__ float activate_fast(int act, float g) {
    if (act == ACT_GELU_TANH) {
        const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        const float e = __expf(2.0f * z);               // tanh(z) = 1 - 2 / (e^2z + 1)
        return 0.5f * g * (2.0f - __fdividef(2.0f, e + 1.0f));
    }
    return __fdividef(g, 1.0f + __expf(-g));
}

// Butterfly reductions: every lane ends with the same value, and the order of the
// additions depends on nothing but the lane numbers.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Where position `pos` of the sequence in `slot` lies inside one layer's page pool.
// `ring` > 0: the group keeps only the last `ring` positions (a multiple of kPageSize) and
// position p lives at ring index p % ring. Layout of a pool: [page][kv_head][kPageSize][head_dim].
struct PagedKV {
    const int32_t* page_table;  // [slots][table_stride]
    int table_stride;
    int ring;
    int kv_heads;
    int head_dim;

    __device__ __forceinline__ size_t row_offset(int slot, int pos, int kv_head) const {
        int idx = ring > 0 ? pos % ring : pos;
        int page = page_table[(size_t)slot * table_stride + idx / kPageSize];
        return (((size_t)page * kv_heads + kv_head) * kPageSize + (idx % kPageSize)) * (size_t)head_dim;
    }
};

}  // namespace sm
