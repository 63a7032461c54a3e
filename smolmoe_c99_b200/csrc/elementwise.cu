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
    pdl_launch_dependents();
    pdl_wait();   // x comes from the kernel before
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

// Many rows (prefill): one warp per row, the row held in registers (NV float4 a lane), one pass.
// The sum runs over a lane's elements in ascending order, then the butterfly: again a function
// of D alone.
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

constexpr int kRowWarps = 8;

template <typename TW, typename TO, int NV>
__global__ void __launch_bounds__(kRowWarps * 32)
rmsnorm_rows_kernel(const float* __restrict__ x, const TW* __restrict__ w, float eps, TO* __restrict__ out,
                    const int32_t* __restrict__ rows, int n_rows, int D) {
    const int r = blockIdx.x * kRowWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();   // x comes from the kernel before
    if (r >= n_rows) return;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float v[NV][4];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (i * 32 + lane) * 4;
        if (d < D) load4(xr + d, v[i]);
        else v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) sq = fmaf(v[i][e], v[i][e], sq);
    sq = warp_sum(sq);
    const float inv = 1.0f / sqrtf(sq / (float)D + eps);
    TO* o = out + (size_t)r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (i * 32 + lane) * 4;
        if (d < D) {
            float wv[4], y[4];
            load4(w + d, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = (v[i][e] * inv) * wv[e];
            store4(o + d, y);
        }
    }
}

template <typename TW, typename TO>
static void launch_norm(const float* x, const void* w, float eps, void* out, const int32_t* rows, int n_rows, int D,
                        cudaStream_t stream) {
    // rows whose length is a multiple of 4 and at most 2048 go to the warp-per-row kernel; a longer row is
    // worth a block of its own (at 3,584 a warp a row took 8 us for 64 rows). The choice depends on D alone,
    // never on the number of rows: a row's result must not depend on how many rows come with it
    if (D % 4 == 0 && D <= 2048) {
        const unsigned blocks = (unsigned)((n_rows + kRowWarps - 1) / kRowWarps);
        if (D <= 1024)
            launch_kernel("rmsnorm", rmsnorm_rows_kernel<TW, TO, 8>, dim3(blocks), dim3(kRowWarps * 32), 0, stream, 1,
                          dependent_launch_enabled(), x, (const TW*)w, eps, (TO*)out, rows, n_rows, D);
        else
            launch_kernel("rmsnorm", rmsnorm_rows_kernel<TW, TO, 16>, dim3(blocks), dim3(kRowWarps * 32), 0, stream, 1,
                          dependent_launch_enabled(), x, (const TW*)w, eps, (TO*)out, rows, n_rows, D);
        return;
    }
    launch_kernel("rmsnorm", rmsnorm_kernel<TW, TO>, dim3((unsigned)n_rows), dim3(kNormThreads), 0, stream, 1,
                  dependent_launch_enabled(), x, (const TW*)w, eps, (TO*)out, rows, D);
}

void rmsnorm(const float* x, const void* w, DType w_dt, float eps, void* out, DType out_dt,
             const int32_t* rows, int n_rows, int D, cudaStream_t stream) {
    if (n_rows <= 0) return;
    note_launch();
    if (w_dt == F32 && out_dt == F32) launch_norm<float, float>(x, w, eps, out, rows, n_rows, D, stream);
    else if (w_dt == F32 && out_dt == BF16) launch_norm<float, __nv_bfloat16>(x, w, eps, out, rows, n_rows, D, stream);
    else if (w_dt == BF16 && out_dt == F32) launch_norm<__nv_bfloat16, float>(x, w, eps, out, rows, n_rows, D, stream);
    else launch_norm<__nv_bfloat16, __nv_bfloat16>(x, w, eps, out, rows, n_rows, D, stream);
}

// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gate_up, TO* __restrict__ out, int H, size_t total, int act) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t t = i / H;
    int j = (int)(i - t * H);
    float g = gate_up[t * 2 * H + j];
    float u = gate_up[t * 2 * H + H + j];
    out[i] = from_float<TO>(u * activate(act, g));
}

void swiglu(const float* gate_up, void* out, DType out_dt, int T, int H, int act, cudaStream_t stream) {
    size_t total = (size_t)T * H;
    if (!total) return;
    if (act < 0 || act >= ACT_COUNT) throw std::invalid_argument("swiglu: unknown activation " + std::to_string(act));
    note_launch();
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dt == F32) swiglu_kernel<float><<<blocks, 256, 0, stream>>>(gate_up, (float*)out, H, total, act);
    else swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(gate_up, (__nv_bfloat16*)out, H, total, act);
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

// The common case (full rotation, head sizes that are multiples of 8): one thread per (token,
// head, 4 neighbouring pairs), 16-byte loads and 8-byte stores.
template <typename TO>
__global__ void rope_store_vec_kernel(RopeStoreArgs a, long long total) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();   // q, k and v come from the kernel before
    if (idx >= total) return;
    const int hd = a.head_dim, half = hd / 2, groups = half / 4;
    const int n_heads = a.heads + 2 * a.kv_heads;
    const int grp = (int)(idx % groups);
    const int head = (int)((idx / groups) % n_heads);
    const int t = (int)(idx / ((long long)groups * n_heads));
    const int pos = a.positions[t];
    const float* x = a.qkv + ((size_t)t * n_heads + head) * hd;
    const int i0 = grp * 4;
    float lo[4], hi[4];
    load4(x + i0, lo);
    load4(x + half + i0, hi);
    const bool is_v = head >= a.heads + a.kv_heads;
    if (!is_v) {
        float c[4], s[4];
        load4(a.cos_table + (size_t)pos * half + i0, c);
        load4(a.sin_table + (size_t)pos * half + i0, s);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float r0 = lo[e] * c[e] - hi[e] * s[e], r1 = lo[e] * s[e] + hi[e] * c[e];
            lo[e] = r0;
            hi[e] = r1;
        }
    }
    if (head < a.heads) {
        TO* q = (TO*)a.q_out + ((size_t)t * a.heads + head) * hd;
        store4(q + i0, lo);
        store4(q + half + i0, hi);
        return;
    }
    const int kvh = is_v ? head - a.heads - a.kv_heads : head - a.heads;
    TO* packed = (TO*)(is_v ? a.v_packed : a.k_packed);
    if (packed) {
        TO* p = packed + ((size_t)t * a.kv_heads + kvh) * hd;
        store4(p + i0, lo);
        store4(p + half + i0, hi);
    }
    if (a.k_pool != nullptr && !(a.ring > 0 && pos < a.token_end[t] - a.ring)) {
        PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};
        TO* c = (TO*)(is_v ? a.v_pool : a.k_pool) + paged.row_offset(a.token_slot[t], pos, kvh);
        store4(c + i0, lo);
        store4(c + half + i0, hi);
    }
}

// Small steps of a model that are no layer's: x *= scale; x = cap * tanh(x / cap); x[t, :] += table[rows[t], :].
__global__ void scale_kernel(float* x, size_t total, float scale) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] *= scale;
}
__global__ void softcap_kernel(float* x, size_t total, float cap) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = cap * tanhf(x[i] / cap);
}
template <typename TT>
__global__ void add_rows_kernel(float* x, const TT* __restrict__ table, const int32_t* __restrict__ rows, int D, int n_table_rows,
                                size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / D;
    const int r = rows[t];
    if (r >= 0 && r < n_table_rows) x[i] += to_float(table[(size_t)r * D + (i - t * D)]);
}

void scale_inplace(float* x, size_t total, float scale, cudaStream_t stream) {
    if (!total) return;
    note_launch();
    scale_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, total, scale);
}
void softcap_inplace(float* x, size_t total, float cap, cudaStream_t stream) {
    if (!total) return;
    if (!(cap > 0.f)) throw std::invalid_argument("softcap: the cap must be positive");
    note_launch();
    softcap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, total, cap);
}
void add_rows(float* x, const void* table, DType table_dt, const int32_t* rows, int T, int D, int n_table_rows, cudaStream_t stream) {
    const size_t total = (size_t)T * D;
    if (!total) return;
    note_launch();
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (table_dt == F32) add_rows_kernel<float><<<blocks, 256, 0, stream>>>(x, (const float*)table, rows, D, n_table_rows, total);
    else add_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(x, (const __nv_bfloat16*)table, rows, D, n_table_rows, total);
}

// Copies this step's packed keys and values into the cache: one thread per 16 bytes of a (token, kv head) row.
__global__ void kv_store_kernel(const uint4* __restrict__ k_packed, const uint4* __restrict__ v_packed, uint4* k_pool,
                                uint4* v_pool, int kv_heads, int chunks, const int32_t* positions,
                                const int32_t* page_table, int table_stride, int ring, const int32_t* token_slot,
                                const int32_t* token_end, long long total) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int c = (int)(idx % chunks);
    const int kvh = (int)((idx / chunks) % kv_heads);
    const int t = (int)(idx / ((long long)chunks * kv_heads));
    const int pos = positions[t];
    if (ring > 0 && pos < token_end[t] - ring) return;   // a later token of this step takes the same place
    PagedKV paged{page_table, table_stride, ring, kv_heads, chunks};   // offsets counted in 16-byte units
    const size_t dst = paged.row_offset(token_slot[t], pos, kvh) + c;
    const size_t src = ((size_t)t * kv_heads + kvh) * chunks + c;
    k_pool[dst] = k_packed[src];
    v_pool[dst] = v_packed[src];
}

void kv_store(const void* k_packed, const void* v_packed, DType dt, int T, int kv_heads, int head_dim, void* k_pool,
              void* v_pool, const int32_t* positions, const int32_t* page_table, int table_stride, int ring,
              const int32_t* token_slot, const int32_t* token_end, cudaStream_t stream) {
    if (T <= 0) return;
    const int elem = dt == F32 ? 4 : 2;
    if (head_dim <= 0 || (head_dim * elem) % 16)
        throw std::invalid_argument("kv_store: a row of head_dim " + std::to_string(head_dim) + " is no multiple of 16 bytes");
    note_launch();
    const int chunks = head_dim * elem / 16;
    const long long total = (long long)T * kv_heads * chunks;
    kv_store_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        (const uint4*)k_packed, (const uint4*)v_packed, (uint4*)k_pool, (uint4*)v_pool, kv_heads, chunks, positions,
        page_table, table_stride, ring, token_slot, token_end, total);
}

void rope_store(const RopeStoreArgs& a, cudaStream_t stream) {
    if (a.T <= 0) return;
    if (a.rotary_dim == a.head_dim && a.head_dim % 8 == 0 && a.head_dim > 0) {
        note_launch();
        const long long total = (long long)a.T * (a.heads + 2 * a.kv_heads) * (a.head_dim / 8);
        const unsigned blocks = (unsigned)((total + 255) / 256);
        if (a.dt == F32)
            launch_kernel("rope_store", rope_store_vec_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, dependent_launch_enabled(), a, total);
        else
            launch_kernel("rope_store", rope_store_vec_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, dependent_launch_enabled(), a, total);
        return;
    }
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
