// Decode attention over the paged cache for bfloat16: one new token per sequence attends to
// its sequence's keys (the reference scans [start, pos] per head on one thread:
// src/kernels.c:1156-1176).
//
// A thread-block cluster of 1 to 16 CTAs serves one (sequence, kv head); its CTAs split the
// visible positions. The group's query heads are the 16 rows of the tensor-core tile (mma.sync
// m16n8k16, operands by ldmatrix), so every key and value row that is read serves all of them. A
// warp keeps a running maximum, sum and weighted values over its tiles; the warps of a CTA merge
// through shared memory, the CTAs of the cluster through distributed shared memory in rank order.
// There is no workspace in global memory and nothing depends on the order in which CTAs finish.
//
// Two kernels, by how long a CTA's share is at the largest cluster whose clusters are all
// resident at once:
//  - up to about 100 KB of keys and values (decode_attention_kernel): the step is bound by the
//    latency of one trip to memory, so the whole share is asked for at once (16-byte asynchronous
//    copies) and as early as possible: the rows of all earlier positions do not depend on the
//    kernel before (only the newest position's row was written by it), so they are requested
//    BEFORE the wait for that kernel. Eight warps take tiles of 32 positions.
//  - longer shares (decode_attention_stream_kernel) are bound by bandwidth: every warp streams
//    tiles of its own through a ring of shared memory filled by the TMA engine.
#include <cooperative_groups.h>
#include <math_constants.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "tcgen05.cuh"

namespace sm {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kTile = 32;           // positions per warp tile
constexpr int kMaxCluster = 16;      // above 8 a kernel has to allow "non-portable" cluster sizes

// the most positions of a CTA's share that are held in one buffer (about 96 KB); longer shares are streamed
constexpr int single_buffer_keys(int hdb) { return 96 * 1024 / ((hdb * 32 + 8) * 4) / kTile * kTile; }

struct DecodeArgs {
    const __nv_bfloat16* q;       // [B, heads, head_dim]
    __nv_bfloat16* out;           // [B, heads, head_dim]
    const __nv_bfloat16* k_pool;
    const __nv_bfloat16* v_pool;
    const int32_t* page_table;
    int table_stride, ring;
    const int32_t* slots;         // [B]
    const int32_t* positions;     // [B] position of the new token (its key is already in the cache)
    int B, heads, kv_heads, head_dim, window, cluster;
    float scale_log2;             // scale * log2(e)
    int buf_keys;                 // one-buffer kernel: positions the buffer holds (a multiple of the tile)
    int own_bytes;                // shared memory a CTA uses for itself: the buffers, later the warps' results
    int stages;                   // streaming kernel: tiles a warp keeps in flight
    int* error;                   // streaming kernel: where a wait that ran out is recorded
    int late;                     // rows of one sequence at several new positions: the kernel before wrote more than the
                                  // newest row of a sequence, so nothing of the cache is read before the wait for it
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// The 8 x 8 matrix of 16-bit elements that the warp holds as an MMA fragment (row lane / 4, columns 2 * (lane % 4) and
// + 1 in one register), transposed.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
    uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    int bytes = pred ? 16 : 0;   // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// The end of both kernels. Every warp has left what it holds after its tiles in shared memory, from smem_raw on:
// [WARPS][16] running maxima, [WARPS][16] sums, [WARPS][16][HDP] weighted values, per head of the group. They are
// merged over the CTA's warps, then over the cluster's CTAs through the leader's shared memory, in warp and rank
// order; the leader writes the output.
template <int WARPS>
__device__ __forceinline__ float* warp_maxima(unsigned char* smem_raw) { return reinterpret_cast<float*>(smem_raw); }
template <int WARPS>
__device__ __forceinline__ float* warp_sums(unsigned char* smem_raw) { return reinterpret_cast<float*>(smem_raw) + WARPS * 16; }
template <int WARPS>
__device__ __forceinline__ float* warp_values(unsigned char* smem_raw) { return reinterpret_cast<float*>(smem_raw) + 2 * WARPS * 16; }

template <int HDB, int WARPS>
__device__ __forceinline__ void merge_and_store(const DecodeArgs& a, unsigned char* smem_raw, float* part, int rank, int kvh, int b) {
    constexpr int HDP = HDB * 32;
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int hd = a.head_dim, group = a.heads / a.kv_heads;
    constexpr int kThreadsHere = WARPS * 32;
    const float* wm = warp_maxima<WARPS>(smem_raw);
    const float* wl = warp_sums<WARPS>(smem_raw);
    const float* wo = warp_values<WARPS>(smem_raw);
    __syncthreads();
    const int pstride = HDP + 2;
    float* dst = a.cluster > 1 ? cluster.map_shared_rank(part, 0) : part;
    for (int idx = threadIdx.x; idx < group * HDP; idx += kThreadsHere) {
        const int r = idx / HDP, d = idx - r * HDP;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, wm[w * 16 + r]);
        float l = 0.f, o = 0.f;
        if (m != -CUDART_INF_F) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float f = exp2f(wm[w * 16 + r] - m);   // a warp without tiles: exp2(-inf) = 0
                l = fmaf(wl[w * 16 + r], f, l);
                o = fmaf(wo[((size_t)w * 16 + r) * HDP + d], f, o);
            }
        }
        float* p = dst + ((size_t)rank * group + r) * pstride;
        p[2 + d] = o;
        if (d == 0) { p[0] = m; p[1] = l; }
    }
    if (a.cluster > 1) {
        cluster.sync();
        if (rank != 0) return;
    } else {
        __syncthreads();
    }
    // ---- the CTAs of the cluster, in rank order ---------------------------------------------------
    for (int idx = threadIdx.x; idx < group * hd; idx += kThreadsHere) {
        const int r = idx / hd, d = idx - r * hd;
        float m = -CUDART_INF_F;
        for (int c = 0; c < a.cluster; ++c) m = fmaxf(m, part[((size_t)c * group + r) * pstride]);
        float l = 0.f, o = 0.f;
        for (int c = 0; c < a.cluster; ++c) {
            const float* p = part + ((size_t)c * group + r) * pstride;
            const float f = exp2f(p[0] - m);   // a CTA without keys: exp2(-inf) = 0
            l = fmaf(p[1], f, l);
            o = fmaf(p[2 + d], f, o);
        }
        a.out[((size_t)b * a.heads + (size_t)kvh * group + r) * hd + d] = __float2bfloat16_rn(o / l);
    }
}

// A warp whose tiles had the heads as the 16 rows of the tensor-core tile (heads g and g + 8 per thread, NT tiles
// of 8 dimensions) leaves its state for the merge. The shared memory must be free (a barrier after its last use).
template <int HDB, int WARPS>
__device__ __forceinline__ void leave_rows_state(unsigned char* smem_raw, const float (&o_acc)[HDB * 4][4], float m0, float m1,
                                                 float l0, float l1) {
    constexpr int HDP = HDB * 32, NT = HDP / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q4 = lane & 3;
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* wm = warp_maxima<WARPS>(smem_raw);
    float* wl = warp_sums<WARPS>(smem_raw);
    float* wo = warp_values<WARPS>(smem_raw);
    if (q4 == 0) {
        wm[warp * 16 + g] = m0; wm[warp * 16 + g + 8] = m1;
        wl[warp * 16 + g] = l0; wl[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        float* r0 = wo + ((size_t)warp * 16 + g) * HDP + i * 8 + q4 * 2;
        float* r1 = wo + ((size_t)warp * 16 + g + 8) * HDP + i * 8 + q4 * 2;
        r0[0] = o_acc[i][0]; r0[1] = o_acc[i][1];
        r1[0] = o_acc[i][2]; r1[1] = o_acc[i][3];
    }
}

// HDB: blocks of 32 of the head dimension (head_dim <= 32 * HDB, a multiple of 16).
template <int HDB>
__global__ void __launch_bounds__(kThreads) decode_attention_kernel(DecodeArgs a) {
    constexpr int HDP = HDB * 32;            // padded head dimension
    constexpr int LD = HDP + 8;              // row in shared memory: conflict-free ldmatrix
    constexpr int NT = HDP / 8;              // dim tiles of the output
    constexpr int CPR = HDP / 8;             // 16-byte pieces per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // the share's keys, then its values, [buf_keys][LD] each; after the loop the same memory holds the warps'
    // results
    __nv_bfloat16* kv_all = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    const size_t buf_elems = (size_t)a.buf_keys * LD;
    const size_t kOwnBytes = (size_t)a.own_bytes;
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw + kOwnBytes);    // [16][LD], heads beyond the group zero
    // [cluster][group][HDP + 2], the leader's copy is used. It lies behind everything a CTA uses
    // for itself: other CTAs write here while this one may still be in its loop.
    float* part = reinterpret_cast<float*>(smem_raw + kOwnBytes + (size_t)16 * LD * sizeof(__nv_bfloat16));
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();

    const int rank = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q4 = lane & 3;
    const int hd = a.head_dim, group = a.heads / a.kv_heads;
    pdl_launch_dependents();
    // slots, positions and the page table are written before the step's first kernel
    const int slot = a.slots[b], pos = a.positions[b];
    const int start = (a.window > 0 && pos >= a.window) ? pos - a.window + 1 : 0;
    const int n_keys = pos - start + 1;
    const int per_cta = ((n_keys + a.cluster - 1) / a.cluster + kTile - 1) / kTile * kTile;
    const int cta_lo = start + rank * per_cta, cta_hi = min(pos + 1, cta_lo + per_cta);   // keys [cta_lo, cta_hi)
    const int cta_keys = cta_hi > cta_lo ? cta_hi - cta_lo : 0;
    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};

    // The whole share is asked for at once: thread -> (row, 16-byte piece) in turn, whole tiles (rows past the end
    // are zeros). The row of position `pos`, which the kernel before this one writes, is left out.
    const bool late = a.late != 0;
    if (late) pdl_wait();
    {
        __nv_bfloat16* kb = kv_all;
        __nv_bfloat16* vb = kv_all + buf_elems;
        const int rows = (cta_keys + kTile - 1) / kTile * kTile;
        for (int idx = threadIdx.x; idx < rows * CPR; idx += kThreads) {
            const int row = idx / CPR, col = (idx - row * CPR) * 8;
            const int key = cta_lo + row;
            if (key == pos && !late) continue;
            const bool in = key < cta_hi && col < hd;
            const size_t o = in ? paged.row_offset(slot, key, kvh) + col : 0;
            cp_async16(kb + (size_t)row * LD + col, a.k_pool + o, in);
            cp_async16(vb + (size_t)row * LD + col, a.v_pool + o, in);
        }
    }
    cp_async_commit();

    pdl_wait();   // q and the newest key and value come from the kernel before

    {
        // q of the group's heads, and the newest position's row: plain loads and stores, which the barrier
        // before the tiles' use makes visible
        const __nv_bfloat16* qrow = a.q + ((size_t)b * a.heads + (size_t)kvh * group) * hd;
        for (int idx = threadIdx.x; idx < 16 * CPR; idx += kThreads) {
            const int row = idx / CPR, col = (idx - row * CPR) * 8;
            const bool in = row < group && col < hd;
            *reinterpret_cast<uint4*>(qs + (size_t)row * LD + col) =
                in ? *reinterpret_cast<const uint4*>(qrow + (size_t)row * hd + col) : make_uint4(0, 0, 0, 0);
        }
        if (!late && pos >= cta_lo && pos < cta_hi) {
            const int row = pos - cta_lo;
            if (threadIdx.x < 2 * CPR) {
                const int which = threadIdx.x / CPR, col = (threadIdx.x - which * CPR) * 8;   // 0: key, 1: value
                const bool in = col < hd;
                const size_t o = in ? paged.row_offset(slot, pos, kvh) + col : 0;
                const __nv_bfloat16* src = (which ? a.v_pool : a.k_pool) + o;
                *reinterpret_cast<uint4*>(kv_all + (size_t)which * buf_elems + (size_t)row * LD + col) =
                    in ? *reinterpret_cast<const uint4*>(src) : make_uint4(0, 0, 0, 0);
            }
        }
    }

    float o_acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    {
        const __nv_bfloat16* kb = kv_all;
        const __nv_bfloat16* vb = kv_all + buf_elems;
        const int lo = cta_lo;
        const int tiles = (cta_keys + kTile - 1) / kTile;
        for (int tile = warp; tile < tiles; tile += kWarps) {
            const __nv_bfloat16* kt = kb + (size_t)tile * kTile * LD;
            const __nv_bfloat16* vt = vb + (size_t)tile * kTile * LD;
            // S = Q K^T: 16 heads x 32 keys
            float s[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kb32 = 0; kb32 < HDB; ++kb32) {
                uint32_t qa[4], qb[4];   // heads x dims [0, 16) and [16, 32) of this block of 32
                ldmatrix_x4(qa, qs + (size_t)(lane & 15) * LD + kb32 * 32 + (lane >> 4) * 8);
                ldmatrix_x4(qb, qs + (size_t)(lane & 15) * LD + kb32 * 32 + 16 + (lane >> 4) * 8);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t kf[4];      // keys 8j.. x dims 0-7, 8-15, 16-23, 24-31 of the block
                    ldmatrix_x4(kf, kt + (size_t)(j * 8 + (lane & 7)) * LD + kb32 * 32 + (lane >> 3) * 8);
                    mma_bf16(s[j], qa[0], qa[1], qa[2], qa[3], kf[0], kf[1]);
                    mma_bf16(s[j], qb[0], qb[1], qb[2], qb[3], kf[2], kf[3]);
                }
            }
            // scale, mask the keys beyond this CTA's range, running maximum
            const int kbase = lo + tile * kTile;
            float mx0 = m0, mx1 = m1;
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = kbase + j * 8 + q4 * 2 + (e & 1);
                    const float x = key < cta_hi ? s[j][e] * a.scale_log2 : -CUDART_INF_F;
                    s[j][e] = x;
                    if (e & 2) mx1 = fmaxf(mx1, x); else mx0 = fmaxf(mx0, x);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float c0 = exp2f(m0 - mx0), c1 = exp2f(m1 - mx1);   // a tile always holds a visible key: mx is finite
            m0 = mx0;
            m1 = mx1;
            uint32_t pf[2][4];
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p0 = exp2f(s[j][0] - mx0), p1 = exp2f(s[j][1] - mx0);
                const float p2 = exp2f(s[j][2] - mx1), p3 = exp2f(s[j][3] - mx1);
                sum0 += p0 + p1;
                sum1 += p2 + p3;
                pf[j / 2][(j & 1) * 2] = pack_bf16(p0, p1);
                pf[j / 2][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            l0 = l0 * c0 + sum0;
            l1 = l1 * c1 + sum1;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                o_acc[i][0] *= c0; o_acc[i][1] *= c0; o_acc[i][2] *= c1; o_acc[i][3] *= c1;
            }
            // O += P V: keys 16jj.. x two dim tiles per ldmatrix
#pragma unroll
            for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                for (int i = 0; i < NT; i += 2) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vt + (size_t)(jj * 16 + (lane & 15)) * LD + i * 8 + (lane >> 4) * 8);
                    mma_bf16(o_acc[i], pf[jj][0], pf[jj][1], pf[jj][2], pf[jj][3], vf[0], vf[1]);
                    mma_bf16(o_acc[i + 1], pf[jj][0], pf[jj][1], pf[jj][2], pf[jj][3], vf[2], vf[3]);
                }
        }
    }
    __syncthreads();   // the buffer is free for the warps' results
    leave_rows_state<HDB, kWarps>(smem_raw, o_acc, m0, m1, l0, l1);
    merge_and_store<HDB, kWarps>(a, smem_raw, part, rank, kvh, b);
}

// ---- shares that do not fit one buffer: every warp streams tiles of its own ------------------------------------
//
// A CTA of four warps; warp w takes the tiles w, w + 4, ... of the CTA's share (KT positions a tile) and keeps
// `stages` of them in flight in a ring of its own, each slot with an mbarrier that counts the bytes as they land.
// Nothing in the loop synchronises the CTA: a warp waits for its tile, uses it, and asks for the tile `stages`
// ahead into the same slot. The query fragments stay in registers for the whole share.
//
// How a tile comes in. A page of the cache holds 64 positions of one kv head as one contiguous block, so with
// head sizes of 64 and 128 (BOX) a tile that lies on a multiple of KT positions is one box of a 2-D tensor map over
// the pool [pages * kv heads * 64 rows, head_dim]: one TMA copy per 64 columns of keys and of values, written with
// the 128-byte swizzle that keeps ldmatrix free of bank conflicts. (Copies of single rows, the other way, are bound
// by the number of copies: a B200 takes about one per 16 cycles and SM, 2.3 to 3.8 TB/s at 128 to 256 bytes a row.)
// Other head sizes are copied row by row (cp.async.bulk, one lane a row) into rows padded by 16 bytes.
constexpr int kStreamWarps = 4;
constexpr int kStreamThreads = kStreamWarps * 32;

template <int HDB, int KT, bool BOX, int NHT>
__global__ void __launch_bounds__(kStreamThreads)
decode_attention_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, DecodeArgs a) {
    using namespace tc5;
    constexpr int HDP = HDB * 32;
    constexpr int LD = HDP + 8;                  // row by row: elements of a padded row
    constexpr int CPR = HDP / 8;                 // 16-byte pieces of a row
    constexpr int HALVES = BOX ? HDP / 64 : 1;   // BOX: blocks of 64 columns, each [KT][64] with rows of 128 bytes
    constexpr int kTileElems = BOX ? KT * HDP : KT * LD;                  // keys of a tile; as many values behind them
    constexpr int kTileBytes = 2 * kTileElems * (int)sizeof(__nv_bfloat16);
    static_assert(KT == 16 || KT == 32, "a tile is 16 or 32 positions");
    static_assert(!BOX || HDP % 64 == 0, "boxes are 64 columns wide");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // [warp][stage][keys | values] (on 1,024 bytes for the swizzle), later the warps' results from smem_raw on;
    // then q, the cluster's partial results, the barriers. (The partial results have memory of their own, although
    // they are written only when the rings are free: a CTA that is done hands its result to the leader at once,
    // while others still stream. Measured with them laid over the rings, which takes a cluster barrier after the
    // loop but leaves room for a third tile in flight: 16.6 -> 19.4 us at 8 x 16,384 positions.)
    const int group = a.heads / a.kv_heads, hd = a.head_dim, S = a.stages;
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw + a.own_bytes);
    float* part = reinterpret_cast<float*>(smem_raw + a.own_bytes + (size_t)16 * LD * sizeof(__nv_bfloat16));
    uint64_t* bars = reinterpret_cast<uint64_t*>(part + (size_t)a.cluster * group * (HDP + 2));   // [warp][stage]

    const int rank = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q4 = lane & 3;
    pdl_launch_dependents();
    // slots, positions and the page table are written before the step's first kernel
    const int slot = a.slots[b], pos = a.positions[b];
    const int start = (a.window > 0 && pos >= a.window) ? pos - a.window + 1 : 0;
    // BOX: tiles lie on multiples of KT positions, so that each is inside one page; what lies before `start` in
    // the first of them is masked
    const int base0 = BOX ? start / KT * KT : start;
    const int n_keys = pos - base0 + 1;
    const int per_cta = ((n_keys + a.cluster - 1) / a.cluster + kTile - 1) / kTile * kTile;
    const int cta_lo = base0 + rank * per_cta, cta_hi = min(pos + 1, cta_lo + per_cta);
    const int first_key = max(start, cta_lo);                                        // this CTA's keys: [first_key, cta_hi)
    const int n_tiles = cta_hi > cta_lo ? (cta_hi - cta_lo + KT - 1) / KT : 0;
    const int my_tiles = n_tiles > warp ? (n_tiles - warp + kStreamWarps - 1) / kStreamWarps : 0;
    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};
    unsigned char* ring_base = BOX ? reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023) : smem_raw;
    unsigned char* ring = ring_base + (size_t)warp * S * kTileBytes;
    uint64_t* my_bars = bars + warp * S;
    const uint32_t row_bytes = (uint32_t)hd * sizeof(__nv_bfloat16);

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&my_bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (!BOX && hd != HDP) {
        // the columns between head_dim and its padded size are never copied: zeros, so that they add nothing
        for (int i = lane; i < S * kTileBytes / 16; i += 32) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // Byte offset in a tile of the 16-byte piece `piece` of row `row`.
    auto piece_at = [&](int row, int piece) -> int {
        if (BOX) return (piece >> 3) * (KT * 128) + row * 128 + (((piece & 7) ^ (row & 7)) << 4);
        return (row * LD + piece * 8) * (int)sizeof(__nv_bfloat16);
    };
    // Whether this warp's tile number i holds the place of the newest position, whose row the kernel before this one
    // writes. In a ring that is the tile of the newest position and, where the window fills its ring and does not
    // start on a tile's boundary, also the first tile: its masked leading rows are the ring's places of the newest ones.
    auto holds_newest = [&](int i) -> bool {
        const int lo = cta_lo + (warp + kStreamWarps * i) * KT;
        const int place = a.ring > 0 ? pos % a.ring : pos, first = a.ring > 0 ? lo % a.ring : lo;
        return place >= first && place < first + KT;
    };
    // BOX: the page of this warp's tile number i (looked up ahead of the request, so that the trip to the table
    // is not waited for when the request is made)
    auto page_of = [&](int i) -> int {
        const int lo = cta_lo + (warp + kStreamWarps * i) * KT;
        const int idx = a.ring > 0 ? lo % a.ring : lo;
        return a.page_table[(size_t)slot * a.table_stride + idx / kPageSize];
    };
    int next_page = 0;
    // Asks for this warp's tile number i into slot s. Row by row: before the wait on the kernel before this one
    // the newest position's row is left out; rows behind the share's end are not copied, and the value rows among
    // them are zeroed, since they are multiplied (by zero weights).
    auto request = [&](int i, int s, bool before_wait) {
        const int lo = cta_lo + (warp + kStreamWarps * i) * KT;
        unsigned char* kt = ring + (size_t)s * kTileBytes;
        unsigned char* vt = kt + kTileBytes / 2;
        if (BOX) {
            if (lane == 0) mbar_expect_tx(&my_bars[s], (uint32_t)kTileBytes);
            __syncwarp();
            if (lane < 2 * HALVES) {
                const int which = lane / HALVES, half = lane - which * HALVES;   // 0: keys, 1: values
                const int idx = a.ring > 0 ? lo % a.ring : lo;
                const int page = before_wait || i < S ? page_of(i) : next_page;
                const int row = (page * a.kv_heads + kvh) * kPageSize + idx % kPageSize;
                tma_load_2d((which ? vt : kt) + half * (KT * 128), which ? &map_v : &map_k, half * 64, row, &my_bars[s]);
            }
            return;
        }
        const int rows = min(KT, cta_hi - lo);
        const bool without_newest = before_wait && pos >= lo && pos < lo + rows;
        if (lane == 0) mbar_expect_tx(&my_bars[s], (uint32_t)(rows - (without_newest ? 1 : 0)) * 2u * row_bytes);
        if (rows < KT) {
            for (int i16 = lane; i16 < (KT - rows) * (LD / 8); i16 += 32)
                reinterpret_cast<uint4*>(vt + (size_t)rows * LD * sizeof(__nv_bfloat16))[i16] = make_uint4(0, 0, 0, 0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
        const int row = KT == 32 ? lane : (lane & 15), key = lo + row;
        if (row < rows && !(before_wait && key == pos)) {
            const size_t o = paged.row_offset(slot, key, kvh);
            const int at = row * LD * (int)sizeof(__nv_bfloat16);
            if (KT == 32 || lane < 16) bulk_load(kt + at, a.k_pool + o, row_bytes, &my_bars[s]);
            if (KT == 32 || lane >= 16) bulk_load(vt + at, a.v_pool + o, row_bytes, &my_bars[s]);
        }
    };
    const int ahead = min(S, my_tiles);
    const bool late = a.late != 0;
    if (late) pdl_wait();
    for (int i = 0; i < ahead; ++i)
        if (late || !(BOX && holds_newest(i))) request(i, i, !late);

    pdl_wait();   // q and the newest key and value come from the kernel before

    {
        // q of the group's heads into shared memory (heads beyond the group zero): plain loads and stores
        const __nv_bfloat16* qrow = a.q + ((size_t)b * a.heads + (size_t)kvh * group) * hd;
        for (int idx = threadIdx.x; idx < 16 * CPR; idx += kStreamThreads) {
            const int row = idx / CPR, col = (idx - row * CPR) * 8;
            const bool in = row < group && col < hd;
            *reinterpret_cast<uint4*>(qs + (size_t)row * LD + col) =
                in ? *reinterpret_cast<const uint4*>(qrow + (size_t)row * hd + col) : make_uint4(0, 0, 0, 0);
        }
        // the newest position, if its tile is among those asked for above: as a whole tile now (BOX: every tile
        // that was left out above), else its row by plain loads and stores into the tile
        if (late) {
            // (every tile was asked for whole, after the wait)
        } else if (BOX) {
            for (int i = 0; i < ahead; ++i)
                if (holds_newest(i)) request(i, i, false);
        } else if (pos >= cta_lo && pos < cta_hi) {
            const int t = (pos - cta_lo) / KT, row = (pos - cta_lo) - t * KT;
            const int i = t / kStreamWarps;
            if (t % kStreamWarps == warp && i < ahead) {
                if (lane < 2 * CPR) {
                    const int which = lane / CPR, piece = lane - which * CPR;   // 0: key, 1: value
                    if (piece * 8 < hd) {
                        const size_t o = paged.row_offset(slot, pos, kvh) + piece * 8;
                        const __nv_bfloat16* src = (which ? a.v_pool : a.k_pool) + o;
                        unsigned char* tile = ring + (size_t)i * kTileBytes + which * (kTileBytes / 2);
                        *reinterpret_cast<uint4*>(tile + piece_at(row, piece)) = *reinterpret_cast<const uint4*>(src);
                    }
                }
            }
        }
    }
    __syncthreads();

    // The tiles are computed transposed: S^T = K Q^T has the tile's positions as the 16 rows of the tensor-core tile
    // and the group's heads as its 8 columns (NHT = 2 column tiles for groups of 9 to 16 heads), O^T = V^T P^T the
    // head dimension as rows. A group of up to 8 heads then costs half the MMAs of the untransposed form, where
    // the heads are padded to 16 rows; and with one warp a scheduler the MMAs are what a long share's time is.
    // A thread holds, per column tile, the heads 2 * q4 and 2 * q4 + 1 (of positions g and g + 8 in S^T, of
    // dimensions g and g + 8 in O^T).
    constexpr int MT = KT / 16;        // tiles of 16 positions
    constexpr int DT = HDP / 16;       // tiles of 16 dimensions
    const int g = lane >> 2;
    uint32_t qf[HDB][NHT][4];          // Q^T as the B operand: per block of 32 dimensions, two steps of 16
#pragma unroll
    for (int kb32 = 0; kb32 < HDB; ++kb32)
#pragma unroll
        for (int nh = 0; nh < NHT; ++nh)
            ldmatrix_x4(qf[kb32][nh], qs + (size_t)(nh * 8 + (lane & 7)) * LD + kb32 * 32 + (lane >> 3) * 8);
    float ot[DT][NHT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d)
#pragma unroll
        for (int nh = 0; nh < NHT; ++nh) ot[d][nh][0] = ot[d][nh][1] = ot[d][nh][2] = ot[d][nh][3] = 0.f;
    float run_m[NHT][2], run_l[NHT][2];   // per head: running maximum (the same in all lanes of a q4), this thread's part of the sum
#pragma unroll
    for (int nh = 0; nh < NHT; ++nh) { run_m[nh][0] = run_m[nh][1] = -CUDART_INF_F; run_l[nh][0] = run_l[nh][1] = 0.f; }

    int s = 0;
    uint32_t parity = 0;
    for (int i = 0; i < my_tiles; ++i) {
        if (!__all_sync(0xffffffffu, mbar_wait(&my_bars[s], parity))) {
            if (lane == 0 && a.error) atomicExch(a.error, 6);
            // the tiles asked for and not used (this one and up to S - 1 after it) may still land in the warp's ring:
            // one more bounded wait for each before the CTA leaves
            for (int j = i; j < my_tiles && j < i + S; ++j) mbar_wait(&my_bars[j % S], (uint32_t)(j / S) & 1u);
            break;
        }
        const unsigned char* kt = ring + (size_t)s * kTileBytes;
        unsigned char* vt = ring + (size_t)s * kTileBytes + kTileBytes / 2;
        const int lo = cta_lo + (warp + kStreamWarps * i) * KT;
        if (BOX && lane < 2 * HALVES && i + S < my_tiles) next_page = page_of(i + S);
        if (BOX && (lo < first_key || lo + KT > cta_hi)) {
            // a box brings whole rows of the page: the value rows outside the share are zeroed (zero weights times
            // whatever lies there must stay zero)
            for (int idx = lane; idx < KT * CPR; idx += 32) {
                const int row = idx / CPR, piece = idx - row * CPR;
                if (lo + row < first_key || lo + row >= cta_hi) *reinterpret_cast<uint4*>(vt + piece_at(row, piece)) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }
        // S^T = K Q^T
        float st[MT][NHT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nh = 0; nh < NHT; ++nh) st[mt][nh][0] = st[mt][nh][1] = st[mt][nh][2] = st[mt][nh][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HDP / 16; ++kk)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t kf[4];      // positions 16mt.. x dimensions 16kk..: rows g / g + 8, columns 0-7 / 8-15
                ldmatrix_x4(kf, kt + piece_at(mt * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
                for (int nh = 0; nh < NHT; ++nh)
                    mma_bf16(st[mt][nh], kf[0], kf[1], kf[2], kf[3], qf[kk / 2][nh][(kk & 1) * 2], qf[kk / 2][nh][(kk & 1) * 2 + 1]);
            }
        // scale, mask the positions outside this CTA's range, running maximum per head
        float mx[NHT][2];
#pragma unroll
        for (int nh = 0; nh < NHT; ++nh) { mx[nh][0] = run_m[nh][0]; mx[nh][1] = run_m[nh][1]; }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int key0 = lo + mt * 16 + g, key1 = key0 + 8;
            const bool in0 = key0 >= first_key && key0 < cta_hi, in1 = key1 >= first_key && key1 < cta_hi;
#pragma unroll
            for (int nh = 0; nh < NHT; ++nh)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float x = ((e & 2) ? in1 : in0) ? st[mt][nh][e] * a.scale_log2 : -CUDART_INF_F;
                    st[mt][nh][e] = x;
                    mx[nh][e & 1] = fmaxf(mx[nh][e & 1], x);
                }
        }
        float rescale[NHT][2];
#pragma unroll
        for (int nh = 0; nh < NHT; ++nh)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = mx[nh][e];
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
                mx[nh][e] = v;       // a tile always holds a visible key (the first one holds the window's start): finite
                rescale[nh][e] = exp2f(run_m[nh][e] - v);
                run_m[nh][e] = v;
            }
        // P^T as the B operand: an 8 x 8 block (positions x heads) of the accumulator is transposed among the lanes
        uint32_t pb[MT][NHT][2];
#pragma unroll
        for (int nh = 0; nh < NHT; ++nh) {
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const float p0 = exp2f(st[mt][nh][0] - mx[nh][0]), p1 = exp2f(st[mt][nh][1] - mx[nh][1]);
                const float p2 = exp2f(st[mt][nh][2] - mx[nh][0]), p3 = exp2f(st[mt][nh][3] - mx[nh][1]);
                sum0 += p0 + p2;
                sum1 += p1 + p3;
                pb[mt][nh][0] = movmatrix_trans(pack_bf16(p0, p1));
                pb[mt][nh][1] = movmatrix_trans(pack_bf16(p2, p3));
            }
            run_l[nh][0] = run_l[nh][0] * rescale[nh][0] + sum0;
            run_l[nh][1] = run_l[nh][1] * rescale[nh][1] + sum1;
        }
#pragma unroll
        for (int d = 0; d < DT; ++d)
#pragma unroll
            for (int nh = 0; nh < NHT; ++nh) {
                ot[d][nh][0] *= rescale[nh][0]; ot[d][nh][1] *= rescale[nh][1];
                ot[d][nh][2] *= rescale[nh][0]; ot[d][nh][3] *= rescale[nh][1];
            }
        // O^T += V^T P^T
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int d = 0; d < DT; ++d) {
                uint32_t vf[4];      // dimensions 16d.. x positions 16mt..: rows g / g + 8, columns 0-7 / 8-15, transposed on the way
                ldmatrix_x4_trans(vf, vt + piece_at(mt * 16 + (lane & 7) + ((lane >> 4) << 3), d * 2 + ((lane >> 3) & 1)));
#pragma unroll
                for (int nh = 0; nh < NHT; ++nh) mma_bf16(ot[d][nh], vf[0], vf[1], vf[2], vf[3], pb[mt][nh][0], pb[mt][nh][1]);
            }
        __syncwarp();   // every lane has read the slot
        if (i + S < my_tiles) request(i + S, s, false);
        if (++s == S) { s = 0; parity ^= 1u; }
    }

    // the warp's state for the merge: [16 heads] maxima and sums, [16 heads][HDP] weighted values
    __syncthreads();   // every warp is through its tiles: the rings are free
    {
        float* wm = warp_maxima<kStreamWarps>(smem_raw);
        float* wl = warp_sums<kStreamWarps>(smem_raw);
        float* wo = warp_values<kStreamWarps>(smem_raw);
#pragma unroll
        for (int nh = 0; nh < NHT; ++nh)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float l = run_l[nh][e];
                l += __shfl_xor_sync(0xffffffffu, l, 4);
                l += __shfl_xor_sync(0xffffffffu, l, 8);
                l += __shfl_xor_sync(0xffffffffu, l, 16);
                const int head = nh * 8 + q4 * 2 + e;
                if (g == 0) { wm[warp * 16 + head] = run_m[nh][e]; wl[warp * 16 + head] = l; }
#pragma unroll
                for (int d = 0; d < DT; ++d) {
                    float* row = wo + ((size_t)warp * 16 + head) * HDP + d * 16 + g;
                    row[0] = ot[d][nh][e];
                    row[8] = ot[d][nh][2 + e];
                }
            }
    }
    merge_and_store<HDB, kStreamWarps>(a, smem_raw, part, rank, kvh, b);
}

// Shared memory of a CTA and how it is cut, for a cluster size and the most positions a CTA can get.
struct DecodePlan {
    int cluster, buf_keys, own_bytes;
    size_t smem;
    bool fits;   // a CTA's share fits the buffer; else the share is streamed (StreamPlan)
};

DecodePlan make_plan(int hdb, int group, int cluster, int visible) {
    const int ld = hdb * 32 + 8;
    const int per_cta = ((visible + cluster - 1) / cluster + kTile - 1) / kTile * kTile;
    DecodePlan p{};
    p.cluster = cluster;
    p.fits = per_cta <= single_buffer_keys(hdb);
    p.buf_keys = p.fits ? per_cta : kTile;
    const size_t loop_bytes = (size_t)2 * p.buf_keys * ld * sizeof(__nv_bfloat16);
    const size_t local_bytes = ((size_t)kWarps * 32 + (size_t)kWarps * 16 * hdb * 32) * sizeof(float);
    p.own_bytes = (int)(((loop_bytes > local_bytes ? loop_bytes : local_bytes) + 15) / 16 * 16);
    p.smem = (size_t)p.own_bytes + (size_t)16 * ld * sizeof(__nv_bfloat16) +
             (size_t)cluster * group * (hdb * 32 + 2) * sizeof(float);
    return p;
}

template <int HDB>
void prepare(size_t smem) {
    // the largest size asked for so far is kept: the attribute is per kernel, not per launch
    static size_t allowed = 48 * 1024;
    static bool large_clusters = false;
    if (!large_clusters) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<HDB>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) throw std::runtime_error(std::string("attention_decode: ") + cudaGetErrorString(e));
        large_clusters = true;
    }
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<HDB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) throw std::runtime_error(std::string("attention_decode: ") + cudaGetErrorString(e));
        allowed = smem;
    }
}

// How many clusters of this shape the GPU holds at once (0 if the query fails).
template <int HDB>
int resident_clusters(const DecodePlan& p) {
    prepare<HDB>(p.smem);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(p.cluster, 1, 1);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = p.smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, decode_attention_kernel<HDB>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

// ---- the streaming kernel's plan -------------------------------------------------------------------------------
constexpr int stream_tile_keys(int hdb) { return hdb >= 3 ? 16 : 32; }
constexpr size_t kStreamSmemShared = 112 * 1024;   // two CTAs to an SM
constexpr size_t kStreamSmemAlone = 208 * 1024;    // one CTA to an SM: more tiles in flight when the CTAs are few

struct StreamPlan {
    int cluster, stages, own_bytes;
    size_t smem;
};

// Shared memory for a cluster size: as many tiles in flight per warp (2 to 6) as fit `target` bytes a CTA.
StreamPlan make_stream_plan(int hdb, bool box, int group, int cluster, size_t target) {
    const int hdp = hdb * 32, ld = hdp + 8;
    const size_t tile_bytes = (size_t)2 * stream_tile_keys(hdb) * (box ? hdp : ld) * sizeof(__nv_bfloat16);
    const size_t fixed = (size_t)16 * ld * sizeof(__nv_bfloat16) + (size_t)cluster * group * (hdp + 2) * sizeof(float) +
                         (size_t)kStreamWarps * 6 * sizeof(uint64_t) + (box ? 1024 : 0) /*the ring starts on 1,024 bytes*/;
    int stages = target > fixed ? (int)((target - fixed) / (kStreamWarps * tile_bytes)) : 2;
    stages = stages < 2 ? 2 : (stages > 6 ? 6 : stages);
    const size_t ring_bytes = (size_t)kStreamWarps * stages * tile_bytes + (box ? 1024 : 0);
    const size_t local_bytes = ((size_t)kStreamWarps * 32 + (size_t)kStreamWarps * 16 * hdp) * sizeof(float);
    StreamPlan p{};
    p.cluster = cluster;
    p.stages = stages;
    p.own_bytes = (int)(((ring_bytes > local_bytes ? ring_bytes : local_bytes) + 15) / 16 * 16);
    p.smem = (size_t)p.own_bytes + fixed - (box ? 1024 : 0);
    return p;
}

template <int HDB, bool BOX, int NHT>
void prepare_stream(size_t smem) {
    constexpr int KT = stream_tile_keys(HDB);
    static size_t allowed = 48 * 1024;
    static bool large_clusters = false;
    if (!large_clusters) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_stream_kernel<HDB, KT, BOX, NHT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) throw std::runtime_error(std::string("attention_decode: ") + cudaGetErrorString(e));
        large_clusters = true;
    }
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_stream_kernel<HDB, KT, BOX, NHT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) throw std::runtime_error(std::string("attention_decode: ") + cudaGetErrorString(e));
        allowed = smem;
    }
}

template <int HDB, bool BOX, int NHT>
int resident_stream_clusters(const StreamPlan& p) {
    prepare_stream<HDB, BOX, NHT>(p.smem);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(p.cluster, 1, 1);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = p.smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, decode_attention_stream_kernel<HDB, stream_tile_keys(HDB), BOX, NHT>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

// The largest cluster all of whose clusters are resident at once and every warp of which gets two tiles or more.
template <int HDB, bool BOX, int NHT>
StreamPlan choose_stream_plan(int pairs, int group, int visible) {
    struct Known { int pairs, group, visible; StreamPlan plan; };
    static std::mutex lock;
    static std::vector<Known> known;
    std::lock_guard<std::mutex> hold(lock);
    for (const Known& k : known)
        if (k.pairs == pairs && k.group == group && k.visible == visible) return k.plan;
    StreamPlan chosen = make_stream_plan(HDB, BOX, group, 1, kStreamSmemShared);
    for (int cluster = kMaxCluster; cluster > 1; cluster /= 2) {
        if (visible < cluster * kStreamWarps * 2 * stream_tile_keys(HDB)) continue;
        const StreamPlan p = make_stream_plan(HDB, BOX, group, cluster, kStreamSmemShared);
        if (pairs <= resident_stream_clusters<HDB, BOX, NHT>(p)) { chosen = p; break; }
    }
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (pairs * chosen.cluster <= sms) {
        // no SM gets a second CTA: each takes the shared memory of two
        const StreamPlan alone = make_stream_plan(HDB, BOX, group, chosen.cluster, kStreamSmemAlone);
        if (pairs <= resident_stream_clusters<HDB, BOX, NHT>(alone)) chosen = alone;
    }
    if (known.size() < 4096) known.push_back({pairs, group, visible, chosen});
    return chosen;
}

// Whether tiles can come in as boxes of a tensor map over the pool: whole blocks of 64 columns, a pool TMA can
// address (16-byte base, row numbers that fit 31 bits).
bool boxes_possible(int head_dim, int kv_heads, long long pool_pages, const void* k_pool, const void* v_pool) {
    return head_dim % 64 == 0 && pool_pages > 0 && pool_pages * kv_heads * kPageSize < (1ll << 31) &&
           (((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0;
}

// The pool [pages, kv heads, 64 positions, head_dim] as rows of head_dim, boxes of `rows` rows x 64 columns with
// the 128-byte swizzle.
CUtensorMap make_pool_map(const void* pool, long long pool_pages, int kv_heads, int head_dim, int rows) {
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)(pool_pages * kv_heads * kPageSize)};
    cuuint64_t strides[1] = {(cuuint64_t)head_dim * sizeof(__nv_bfloat16)};
    cuuint32_t box[2] = {64, (cuuint32_t)rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = tc5::tensor_map_encoder()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box,
                                           elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        throw std::runtime_error("attention_decode: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r) +
                                 " for a pool of " + std::to_string(pool_pages) + " pages");
    return map;
}

template <int HDB, bool BOX, int NHT>
void launch_stream(DecodeArgs a, int visible, long long pool_pages, cudaStream_t stream) {
    constexpr int KT = stream_tile_keys(HDB);
    const StreamPlan sp = choose_stream_plan<HDB, BOX, NHT>(a.B * a.kv_heads, a.heads / a.kv_heads, visible);
    a.cluster = sp.cluster;
    a.stages = sp.stages;
    a.own_bytes = sp.own_bytes;
    a.error = error_word();
    CUtensorMap map_k{}, map_v{};
    if (BOX) {
        map_k = make_pool_map(a.k_pool, pool_pages, a.kv_heads, a.head_dim, KT);
        map_v = make_pool_map(a.v_pool, pool_pages, a.kv_heads, a.head_dim, KT);
    }
    prepare_stream<HDB, BOX, NHT>(sp.smem);
    launch_kernel("attention_decode", decode_attention_stream_kernel<HDB, KT, BOX, NHT>, dim3(a.cluster, a.kv_heads, a.B),
                  dim3(kStreamThreads), sp.smem, stream, a.cluster, dependent_launch_enabled(), map_k, map_v, a);
}

// CTAs per (sequence, kv head): the largest cluster, of at most 16, all of whose clusters are resident at once
// (a second wave doubles the time), and every CTA of which gets a few tiles of positions.
template <int HDB>
DecodePlan choose_plan(int pairs, int group, int visible) {
    struct Known { int pairs, group, visible; DecodePlan plan; };
    static std::mutex lock;
    static std::vector<Known> known;
    std::lock_guard<std::mutex> hold(lock);
    for (const Known& k : known)
        if (k.pairs == pairs && k.group == group && k.visible == visible) return k.plan;
    DecodePlan chosen = make_plan(HDB, group, 1, visible);
    for (int cluster = kMaxCluster; cluster > 1; cluster /= 2) {
        if (visible <= (cluster / 2) * 4 * kTile) continue;
        const DecodePlan p = make_plan(HDB, group, cluster, visible);
        if (pairs <= resident_clusters<HDB>(p)) { chosen = p; break; }
    }
    if (known.size() < 4096) known.push_back({pairs, group, visible, chosen});
    return chosen;
}

template <int HDB>
void launch(DecodeArgs a, int visible, long long pool_pages, cudaStream_t stream) {
    const DecodePlan p = choose_plan<HDB>(a.B * a.kv_heads, a.heads / a.kv_heads, visible);
    if (!p.fits) {
        // a share that does not fit one buffer is streamed
        // (a group of up to 8 heads is one column tile of the transposed product, up to 16 heads two)
        const bool box = HDB % 2 == 0 && boxes_possible(a.head_dim, a.kv_heads, pool_pages, a.k_pool, a.v_pool);
        const bool wide = a.heads / a.kv_heads > 8;
        if (box && wide) launch_stream<HDB, HDB % 2 == 0, 2>(a, visible, pool_pages, stream);
        else if (box) launch_stream<HDB, HDB % 2 == 0, 1>(a, visible, pool_pages, stream);
        else if (wide) launch_stream<HDB, false, 2>(a, visible, pool_pages, stream);
        else launch_stream<HDB, false, 1>(a, visible, pool_pages, stream);
        return;
    }
    a.cluster = p.cluster;
    a.buf_keys = p.buf_keys;
    a.own_bytes = p.own_bytes;
    prepare<HDB>(p.smem);
    launch_kernel("attention_decode", decode_attention_kernel<HDB>, dim3(a.cluster, a.kv_heads, a.B), dim3(kThreads), p.smem,
                  stream, a.cluster, dependent_launch_enabled(), a);
}

}  // namespace

bool attention_decode_supports(int heads, int kv_heads, int head_dim) {
    return head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128 && kv_heads > 0 && heads % kv_heads == 0 &&
           heads / kv_heads <= 16;
}

void attention_decode_plan(int B, int heads, int kv_heads, int head_dim, int window, int max_len, int* plan) {
    if (!attention_decode_supports(heads, kv_heads, head_dim)) throw std::invalid_argument("attention_decode_plan: sizes outside the kernel");
    const int visible = window > 0 && window < max_len ? window : max_len;
    DecodePlan p{};
    switch ((head_dim + 31) / 32) {
        case 1: p = choose_plan<1>(B * kv_heads, heads / kv_heads, visible); break;
        case 2: p = choose_plan<2>(B * kv_heads, heads / kv_heads, visible); break;
        case 3: p = choose_plan<3>(B * kv_heads, heads / kv_heads, visible); break;
        default: p = choose_plan<4>(B * kv_heads, heads / kv_heads, visible); break;
    }
    plan[0] = p.cluster; plan[1] = p.buf_keys; plan[2] = 1; plan[3] = (int)p.smem;
    if (!p.fits) {   // streamed: the cluster, 0, the tiles a warp keeps in flight, the shared memory
        StreamPlan sp{};
        const int pairs = B * kv_heads, group = heads / kv_heads;
        const bool wide = group > 8;
        switch ((head_dim + 31) / 32) {
            case 1: sp = wide ? choose_stream_plan<1, false, 2>(pairs, group, visible) : choose_stream_plan<1, false, 1>(pairs, group, visible); break;
            case 2:
                if (head_dim == 64) sp = wide ? choose_stream_plan<2, true, 2>(pairs, group, visible) : choose_stream_plan<2, true, 1>(pairs, group, visible);
                else sp = wide ? choose_stream_plan<2, false, 2>(pairs, group, visible) : choose_stream_plan<2, false, 1>(pairs, group, visible);
                break;
            case 3: sp = wide ? choose_stream_plan<3, false, 2>(pairs, group, visible) : choose_stream_plan<3, false, 1>(pairs, group, visible); break;
            default:
                if (head_dim == 128) sp = wide ? choose_stream_plan<4, true, 2>(pairs, group, visible) : choose_stream_plan<4, true, 1>(pairs, group, visible);
                else sp = wide ? choose_stream_plan<4, false, 2>(pairs, group, visible) : choose_stream_plan<4, false, 1>(pairs, group, visible);
                break;
        }
        plan[0] = sp.cluster; plan[1] = 0; plan[2] = sp.stages; plan[3] = (int)sp.smem;
    }
}

void attention_decode(const void* q, void* out, int B, int heads, int kv_heads, int head_dim, float scale, int window,
                      const int32_t* positions, const int32_t* slots, const void* k_pool, const void* v_pool,
                      const int32_t* page_table, int table_stride, int ring, int max_len, long long pool_pages, bool late,
                      cudaStream_t stream) {
    if (B <= 0) return;
    if (!attention_decode_supports(heads, kv_heads, head_dim))
        throw std::invalid_argument("attention_decode: head_dim " + std::to_string(head_dim) + " with " +
                                    std::to_string(heads) + "/" + std::to_string(kv_heads) +
                                    " heads is outside this kernel (multiples of 16 up to 128, at most 16 heads per "
                                    "kv head); the plain kernel takes it");
    if (B > 65535 || kv_heads > 65535) throw std::invalid_argument("attention_decode: more than 65535 sequences or kv heads");
    const int visible = window > 0 && window < max_len ? window : max_len;
    DecodeArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
                 page_table, table_stride, ring, slots, positions, B, heads, kv_heads, head_dim, window, 1,
                 scale * 1.4426950408889634f, 0, 0, 0, nullptr, late ? 1 : 0};
    note_launch();
    switch ((head_dim + 31) / 32) {
        case 1: launch<1>(a, visible, pool_pages, stream); break;
        case 2: launch<2>(a, visible, pool_pages, stream); break;
        case 3: launch<3>(a, visible, pool_pages, stream); break;
        default: launch<4>(a, visible, pool_pages, stream); break;
    }
}

}  // namespace sm
