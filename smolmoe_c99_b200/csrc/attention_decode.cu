// Decode attention over the paged cache for bfloat16: one new token per sequence attends
// to its sequence's keys, split along the positions so that one long sequence fills many
// SMs (the reference scans [start, pos] per head on one thread: src/kernels.c:1156-1176).
//
// Kernel 1, one CTA per (kv head, sequence, chunk of kChunk positions): the group's query
// heads share every key and value row that is read. Scores for the chunk, their running
// maximum and sum, and the unnormalised weighted values go to a workspace:
//   part_o [B, heads, splits, head_dim] float, part_ml [B, heads, splits, 2] float.
// The CTA that finishes last for its (sequence, kv head) -- known from a counter that it
// then resets -- merges the chunks that hold visible keys in ascending order and writes the
// normalised result, so the whole attention is one launch. Chunks without visible keys
// (beyond the sequence, or before the window) do no work and are not read by the merge.
#include <math_constants.h>

#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace sm {

namespace {

constexpr int kChunk = 128;       // positions per CTA
constexpr int kThreads = 128;
constexpr int kHeadPass = 8;      // query heads handled per pass over the keys
constexpr int kMaxHeadDim = 256;

struct DecodeArgs {
    const __nv_bfloat16* q;       // [B, heads, head_dim]
    __nv_bfloat16* out;           // [B, heads, head_dim]
    const __nv_bfloat16* k_pool;
    const __nv_bfloat16* v_pool;
    const int32_t* page_table;
    int table_stride, ring;
    const int32_t* slots;         // [B]
    const int32_t* positions;     // [B] position of the new token (its key is already in the cache)
    int B, heads, kv_heads, head_dim, window, splits;
    float scale;
    float* part_o;
    float* part_ml;
    int* counters;                // [B, kv_heads], zero between launches
};

// Phase timestamps of one CTA, for a timing probe built with -DSM_DECODE_TIMING.
#ifdef SM_DECODE_TIMING
__device__ unsigned long long g_decode_timing[32];
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define SM_STAMP(i) do { if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && (blockIdx.z == 0 || (i) >= 10)) g_decode_timing[i] = global_ns(); } while (0)
#else
#define SM_STAMP(i) do { } while (0)
#endif

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

__global__ void __launch_bounds__(kThreads) decode_partial_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SM_STAMP(0);
    pdl_launch_dependents();
    pdl_wait();   // q and the newest key and value come from the kernel before
    const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
    const int hd = a.head_dim, group = a.heads / a.kv_heads;
    const int pos = a.positions[b];
    const int start = (a.window > 0 && pos >= a.window) ? pos - a.window + 1 : 0;
    const int c0 = split * kChunk;
    if (c0 > pos || c0 + kChunk <= start) return;   // no visible key in this chunk
    const int lo = max(c0, start), hi = min(c0 + kChunk - 1, pos);   // visible keys [lo, hi]

    float* qs = reinterpret_cast<float*>(smem_raw);                    // [group][hd]
    float* sc = qs + group * hd;                                       // [group][kChunk] scores, then weights
    unsigned long long* rows = reinterpret_cast<unsigned long long*>(sc + group * kChunk);  // [kChunk]
    float* red = reinterpret_cast<float*>(rows + kChunk);              // [key groups][kHeadPass][hd]
    float* wts = red + (size_t)(kThreads / (hd / 8)) * kHeadPass * hd; // [warps][splits] merge weights
    __shared__ int is_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const __nv_bfloat16* qb = a.q + ((size_t)b * a.heads + (size_t)kvh * group) * hd;
    for (int i = tid * 8; i < group * hd; i += kThreads * 8) {   // hd is a multiple of 8
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(qb + i), v);
#pragma unroll
        for (int e = 0; e < 8; ++e) qs[i + e] = v[e];
    }
    const int slot = a.slots[b];
    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};
    const int p = c0 + tid;
    const bool valid = p >= lo && p <= hi;
    unsigned long long row = 0;
    if (valid) row = (unsigned long long)paged.row_offset(slot, p, kvh);
    rows[tid] = row;
    __syncthreads();
    SM_STAMP(1);

    // scores: one key per thread, kHeadPass heads at a time
    for (int g0 = 0; g0 < group; g0 += kHeadPass) {
        float s[kHeadPass];
#pragma unroll
        for (int g = 0; g < kHeadPass; ++g) s[g] = 0.f;
        if (valid) {
            const __nv_bfloat16* kr = a.k_pool + row;
            for (int d0 = 0; d0 < hd; d0 += 64) {
                // up to 64 dims of the key row at once: eight loads in flight, then the arithmetic
                uint4 raw[8];
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    raw[c] = d0 + c * 8 < hd ? *reinterpret_cast<const uint4*>(kr + d0 + c * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int d = d0 + c * 8;
                    if (d >= hd) break;
                    float kv[8];
                    unpack8(raw[c], kv);
#pragma unroll
                    for (int g = 0; g < kHeadPass; ++g) {
                        if (g0 + g < group) {
                            const float4 qa = *reinterpret_cast<const float4*>(qs + (g0 + g) * hd + d);
                            const float4 qc = *reinterpret_cast<const float4*>(qs + (g0 + g) * hd + d + 4);
                            s[g] = fmaf(qa.x, kv[0], s[g]); s[g] = fmaf(qa.y, kv[1], s[g]);
                            s[g] = fmaf(qa.z, kv[2], s[g]); s[g] = fmaf(qa.w, kv[3], s[g]);
                            s[g] = fmaf(qc.x, kv[4], s[g]); s[g] = fmaf(qc.y, kv[5], s[g]);
                            s[g] = fmaf(qc.z, kv[6], s[g]); s[g] = fmaf(qc.w, kv[7], s[g]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < kHeadPass; ++g)
            if (g0 + g < group) sc[(g0 + g) * kChunk + tid] = valid ? s[g] * a.scale : -CUDART_INF_F;
    }
    __syncthreads();
    SM_STAMP(2);

    // per head: maximum, weights exp(s - m) and their sum; warps take heads in turn
    for (int g = warp; g < group; g += kThreads / 32) {
        float m = -CUDART_INF_F;
        for (int i = lane; i < kChunk; i += 32) m = fmaxf(m, sc[g * kChunk + i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = lane; i < kChunk; i += 32) {
            float e = expf(sc[g * kChunk + i] - m);   // masked keys: exp(-inf) = 0
            sc[g * kChunk + i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) {
            float* ml = a.part_ml + (((size_t)b * a.heads + kvh * group + g) * a.splits + split) * 2;
            ml[0] = m;
            ml[1] = l;
        }
    }
    __syncthreads();
    SM_STAMP(3);

    // weighted values: a thread owns 8 neighbouring dims (16 bytes) of the rows of its key
    // group; the groups take keys in turn, four loads in flight each
    const int cpr = hd / 8;                       // 16-byte chunks per row
    const int key_groups = kThreads / cpr;        // hd <= 256 -> at least 4
    const int kg = tid / cpr, ch = tid - kg * cpr;
    const int first = lo - c0, last = hi - c0;
    for (int g0 = 0; g0 < group; g0 += kHeadPass) {
        float acc[kHeadPass][8];
#pragma unroll
        for (int g = 0; g < kHeadPass; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
        if (kg < key_groups) {
            for (int j0 = first + kg; j0 <= last; j0 += 8 * key_groups) {
                uint4 raw[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int j = j0 + u * key_groups;
                    raw[u] = j <= last ? *reinterpret_cast<const uint4*>(a.v_pool + rows[j] + 8 * ch) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int j = j0 + u * key_groups;
                    if (j > last) break;
                    float v[8];
                    unpack8(raw[u], v);
#pragma unroll
                    for (int g = 0; g < kHeadPass; ++g) {
                        if (g0 + g < group) {
                            const float w = sc[(g0 + g) * kChunk + j];
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(w, v[e], acc[g][e]);
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < kHeadPass; ++g)
#pragma unroll
                for (int e = 0; e < 8; ++e) red[((size_t)kg * kHeadPass + g) * hd + 8 * ch + e] = acc[g][e];
        }
        __syncthreads();
        for (int i = tid; i < kHeadPass * hd; i += kThreads) {
            int g = i / hd, d = i - g * hd;
            if (g0 + g < group) {
                float sum = 0.f;
                for (int k = 0; k < key_groups; ++k) sum += red[((size_t)k * kHeadPass + g) * hd + d];
                a.part_o[(((size_t)b * a.heads + kvh * group + g0 + g) * a.splits + split) * hd + d] = sum;
            }
        }
        __syncthreads();
    }

    SM_STAMP(4);
    // the last CTA of this (sequence, kv head) merges the chunks
    const int s_lo = start / kChunk, s_hi = pos / kChunk, n_active = s_hi - s_lo + 1;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = a.counters + b * a.kv_heads + kvh;
        int arrived = atomicAdd(counter, 1);
        is_last = arrived == n_active - 1;
        if (is_last) *counter = 0;
    }
    __syncthreads();
    SM_STAMP(5);
    if (!is_last) return;
    __threadfence();
    SM_STAMP(10);
    float* my_w = wts + (size_t)warp * a.splits;
    for (int g = warp; g < group; g += kThreads / 32) {
        const size_t head = (size_t)b * a.heads + kvh * group + g;
        const float* ml = a.part_ml + head * a.splits * 2;
        const float* po = a.part_o + head * a.splits * hd;
        float m = -CUDART_INF_F;
        for (int s = s_lo + lane; s <= s_hi; s += 32) m = fmaxf(m, __ldcg(ml + 2 * s));
        m = warp_max(m);
        float l = 0.f;
        for (int s = s_lo + lane; s <= s_hi; s += 32) {
            float w = expf(__ldcg(ml + 2 * s) - m);
            my_w[s - s_lo] = w;
            l = fmaf(__ldcg(ml + 2 * s + 1), w, l);
        }
        l = warp_sum(l);
        __syncwarp();
        SM_STAMP(11);
        float acc[kMaxHeadDim / 32];
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.f;
        for (int s0 = s_lo; s0 <= s_hi; s0 += 16) {
            // sixteen chunks' partial results in flight per dim, then the sums in chunk order
#pragma unroll
            for (int i = 0; i < kMaxHeadDim / 32; ++i) {
                const int d = lane + 32 * i;
                if (d >= hd) break;
                float v[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) v[u] = s0 + u <= s_hi ? __ldcg(po + (size_t)(s0 + u) * hd + d) : 0.f;
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (s0 + u <= s_hi) acc[i] = fmaf(v[u], my_w[s0 + u - s_lo], acc[i]);
            }
        }
        const float inv = 1.0f / l;
        __nv_bfloat16* o = a.out + head * hd;
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) {
            int d = lane + 32 * i;
            if (d < hd) o[d] = __float2bfloat16_rn(acc[i] * inv);
        }
        __syncwarp();
        SM_STAMP(12);
    }
}

}  // namespace

int attention_decode_splits(int max_len) { return (max_len + kChunk - 1) / kChunk; }

size_t attention_decode_workspace_floats(int B, int heads, int head_dim, int splits) {
    return (size_t)B * heads * splits * (head_dim + 2);
}

void attention_decode(const void* q, void* out, int B, int heads, int kv_heads, int head_dim, float scale, int window,
                      const int32_t* positions, const int32_t* slots, const void* k_pool, const void* v_pool,
                      const int32_t* page_table, int table_stride, int ring, int splits, float* workspace,
                      int* counters, cudaStream_t stream) {
    if (B <= 0) return;
    if (head_dim % 8 || head_dim <= 0 || head_dim > kMaxHeadDim)
        throw std::invalid_argument("attention_decode: head_dim " + std::to_string(head_dim) +
                                    " must be a multiple of 8 between 8 and 256");
    if (heads % kv_heads) throw std::invalid_argument("attention_decode: kv_heads must divide heads");
    if (splits <= 0 || splits > 65535) throw std::invalid_argument("attention_decode: splits out of range");
    int group = heads / kv_heads;
    int key_groups = kThreads / (head_dim / 8);
    size_t smem = (size_t)group * head_dim * 4 + (size_t)group * kChunk * 4 + kChunk * 8 +
                  (size_t)key_groups * kHeadPass * head_dim * 4 + (size_t)(kThreads / 32) * splits * 4;
    if (B * kv_heads > 65536) throw std::invalid_argument("attention_decode: more than 65536 (sequence, kv head) pairs");
    if (smem > 200 * 1024)
        throw std::invalid_argument("attention_decode: " + std::to_string(group) + " heads per kv head with head_dim " +
                                    std::to_string(head_dim) + " need more shared memory than one SM has");
    DecodeArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pool,
                 (const __nv_bfloat16*)v_pool, page_table, table_stride, ring, slots, positions,
                 B, heads, kv_heads, head_dim, window, splits, scale,
                 workspace, workspace + (size_t)B * heads * splits * head_dim, counters};
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(decode_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    note_launch();
    dim3 grid(kv_heads, B, splits);
    launch_kernel("attention_decode", decode_partial_kernel, grid, dim3(kThreads), smem, stream, 1,
                  dependent_launch_enabled(), a);
}

}  // namespace sm
