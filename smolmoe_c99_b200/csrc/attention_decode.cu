// Decode attention over the paged cache for bfloat16: one new token per sequence attends to
// its sequence's keys (the reference scans [start, pos] per head on one thread:
// src/kernels.c:1156-1176).
//
// A thread-block cluster of 1 to 16 CTAs serves one (sequence, kv head); its CTAs split the
// visible positions. A CTA brings its keys and values into shared memory with 16-byte
// asynchronous copies: all of them at once if its share fits a buffer of about 100 KB (two
// such CTAs fit an SM), else in chunks of a few hundred positions with two chunks in flight.
// The step is bound by the latency of that one trip to memory, so everything is asked for at
// once and as early as possible: the rows of all earlier positions do not depend on the kernel before (only the
// newest position's row was written by it), so they are requested BEFORE the wait for that
// kernel. Within a chunk the eight warps take tiles of 32 positions. The group's query heads
// are the 16 rows of the tensor-core tile (mma.sync m16n8k16, operands by ldmatrix), so every
// key and value row that is read serves all of them. A warp keeps a running maximum, sum and
// weighted values over its tiles; the warps of a CTA merge through shared memory, the CTAs of
// the cluster through distributed shared memory in rank order. There is no workspace in
// global memory and nothing depends on the order in which CTAs finish.
#include <cooperative_groups.h>
#include <math_constants.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace sm {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kTile = 32;           // positions per warp tile
constexpr int kMaxCluster = 16;      // above 8 a kernel has to allow "non-portable" cluster sizes

// positions per chunk for a head dimension of up to 32 * hdb when a share is read in chunks, two in
// flight: about 36 KB of keys and values each, so that two CTAs fit an SM
constexpr int chunk_keys(int hdb) { return hdb == 1 ? 224 : (hdb == 2 ? 128 : 64); }
// the most positions of a CTA's share that are held in one buffer instead (about 96 KB)
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
    int buf_keys, n_bufs;         // positions per buffer (a multiple of the tile) and buffers (1 or 2)
    int own_bytes;                // shared memory a CTA uses for itself: the buffers, later the warps' results
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
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
    uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    int bytes = pred ? 16 : 0;   // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// HDB: blocks of 32 of the head dimension (head_dim <= 32 * HDB, a multiple of 16).
template <int HDB>
__global__ void __launch_bounds__(kThreads) decode_attention_kernel(DecodeArgs a) {
    constexpr int HDP = HDB * 32;            // padded head dimension
    constexpr int LD = HDP + 8;              // row in shared memory: conflict-free ldmatrix
    constexpr int NT = HDP / 8;              // dim tiles of the output
    constexpr int CPR = HDP / 8;             // 16-byte pieces per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // n_bufs buffers of keys, then as many of values, [buf_keys][LD] each; after the loop the same memory holds
    // the warps' results
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
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q4 = lane & 3;
    const int hd = a.head_dim, group = a.heads / a.kv_heads;
    pdl_launch_dependents();
    // slots, positions and the page table are written before the step's first kernel
    const int slot = a.slots[b], pos = a.positions[b];
    const int start = (a.window > 0 && pos >= a.window) ? pos - a.window + 1 : 0;
    const int n_keys = pos - start + 1;
    const int per_cta = ((n_keys + a.cluster - 1) / a.cluster + kTile - 1) / kTile * kTile;
    const int cta_lo = start + rank * per_cta, cta_hi = min(pos + 1, cta_lo + per_cta);   // keys [cta_lo, cta_hi)
    const int cta_keys = cta_hi > cta_lo ? cta_hi - cta_lo : 0;
    const int n_chunks = (cta_keys + a.buf_keys - 1) / a.buf_keys;
    // chunks of equal length (a multiple of the tile), so that a short second chunk does not cost a whole pass
    const int chunk_len = n_chunks ? ((cta_keys + kTile - 1) / kTile + n_chunks - 1) / n_chunks * kTile : kTile;
    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};

    // Requests chunk `ch` into its buffer: thread -> (row, 16-byte piece) in turn. `skip_newest` leaves out
    // the row of position `pos`, which the kernel before this one writes.
    auto request_chunk = [&](int ch, bool skip_newest) {
        __nv_bfloat16* kb = kv_all + (size_t)(ch % a.n_bufs) * buf_elems;
        __nv_bfloat16* vb = kv_all + (size_t)(a.n_bufs + ch % a.n_bufs) * buf_elems;
        const int lo = cta_lo + ch * chunk_len;
        const int rows = min(chunk_len, (cta_hi - lo + kTile - 1) / kTile * kTile);   // whole tiles; rows past the end are zeros
        for (int idx = threadIdx.x; idx < rows * CPR; idx += kThreads) {
            const int row = idx / CPR, col = (idx - row * CPR) * 8;
            const int key = lo + row;
            if (skip_newest && key == pos) continue;
            const bool in = key < cta_hi && col < hd;
            const size_t o = in ? paged.row_offset(slot, key, kvh) + col : 0;
            cp_async16(kb + (size_t)row * LD + col, a.k_pool + o, in);
            cp_async16(vb + (size_t)row * LD + col, a.v_pool + o, in);
        }
    };
    if (n_chunks > 0) request_chunk(0, true);
    cp_async_commit();
    if (a.n_bufs > 1 && n_chunks > 1) request_chunk(1, true);
    cp_async_commit();

    pdl_wait();   // q and the newest key and value come from the kernel before

    {
        // q of the group's heads, and the newest position's row if its chunk has been asked for already: plain
        // loads and stores, which the barrier before the first chunk's use makes visible
        const __nv_bfloat16* qrow = a.q + ((size_t)b * a.heads + (size_t)kvh * group) * hd;
        for (int idx = threadIdx.x; idx < 16 * CPR; idx += kThreads) {
            const int row = idx / CPR, col = (idx - row * CPR) * 8;
            const bool in = row < group && col < hd;
            *reinterpret_cast<uint4*>(qs + (size_t)row * LD + col) =
                in ? *reinterpret_cast<const uint4*>(qrow + (size_t)row * hd + col) : make_uint4(0, 0, 0, 0);
        }
        if (pos >= cta_lo && pos < cta_hi) {
            const int ch = (pos - cta_lo) / chunk_len, row = (pos - cta_lo) - ch * chunk_len;
            if (ch < a.n_bufs && threadIdx.x < 2 * CPR) {
                const int which = threadIdx.x / CPR, col = (threadIdx.x - which * CPR) * 8;   // 0: key, 1: value
                const bool in = col < hd;
                const size_t o = in ? paged.row_offset(slot, pos, kvh) + col : 0;
                const __nv_bfloat16* src = (which ? a.v_pool : a.k_pool) + o;
                *reinterpret_cast<uint4*>(kv_all + (size_t)(which * a.n_bufs + ch) * buf_elems + (size_t)row * LD + col) =
                    in ? *reinterpret_cast<const uint4*>(src) : make_uint4(0, 0, 0, 0);
            }
        }
    }

    float o_acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

    for (int ch = 0; ch < n_chunks; ++ch) {
        // Groups of copies in the order they were committed: chunk 0, chunk 1 (or nothing), then one after every
        // chunk's use (chunk ch + n_bufs, or nothing). Chunk ch is in group ch; with two buffers one later group
        // may still be on its way.
        if (a.n_bufs == 1) asm volatile("cp.async.wait_group 0;" ::: "memory");
        else asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const __nv_bfloat16* kb = kv_all + (size_t)(ch % a.n_bufs) * buf_elems;
        const __nv_bfloat16* vb = kv_all + (size_t)(a.n_bufs + ch % a.n_bufs) * buf_elems;
        const int lo = cta_lo + ch * chunk_len;
        const int tiles = (min(chunk_len, cta_hi - lo) + kTile - 1) / kTile;
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
        __syncthreads();   // the buffer is free again
        if (ch + a.n_bufs < n_chunks) request_chunk(ch + a.n_bufs, false);
        cp_async_commit();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- the warps of this CTA, through shared memory (the chunk buffers are free now) -------
    __syncthreads();
    float* wm = reinterpret_cast<float*>(smem_raw);          // [kWarps][16] maxima
    float* wl = wm + kWarps * 16;                            // [kWarps][16] sums
    float* wo = wl + kWarps * 16;                            // [kWarps][16][HDP] weighted values
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
    __syncthreads();
    const int pstride = HDP + 2;
    float* dst = a.cluster > 1 ? cluster.map_shared_rank(part, 0) : part;
    for (int idx = threadIdx.x; idx < group * HDP; idx += kThreads) {
        const int r = idx / HDP, d = idx - r * HDP;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) m = fmaxf(m, wm[w * 16 + r]);
        float l = 0.f, o = 0.f;
        if (m != -CUDART_INF_F) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
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
    for (int idx = threadIdx.x; idx < group * hd; idx += kThreads) {
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

// Shared memory of a CTA and how it is cut, for a cluster size and the most positions a CTA can get.
struct DecodePlan {
    int cluster, buf_keys, n_bufs, own_bytes;
    size_t smem;
};

DecodePlan make_plan(int hdb, int group, int cluster, int visible) {
    const int ld = hdb * 32 + 8;
    const int per_cta = ((visible + cluster - 1) / cluster + kTile - 1) / kTile * kTile;
    DecodePlan p{};
    p.cluster = cluster;
    if (per_cta <= single_buffer_keys(hdb)) {
        p.n_bufs = 1;
        p.buf_keys = per_cta;
    } else {
        p.n_bufs = 2;
        p.buf_keys = chunk_keys(hdb);
    }
    const size_t loop_bytes = (size_t)2 * p.n_bufs * p.buf_keys * ld * sizeof(__nv_bfloat16);
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
void launch(DecodeArgs a, int visible, cudaStream_t stream) {
    const DecodePlan p = choose_plan<HDB>(a.B * a.kv_heads, a.heads / a.kv_heads, visible);
    a.cluster = p.cluster;
    a.buf_keys = p.buf_keys;
    a.n_bufs = p.n_bufs;
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
    plan[0] = p.cluster; plan[1] = p.buf_keys; plan[2] = p.n_bufs; plan[3] = (int)p.smem;
}

void attention_decode(const void* q, void* out, int B, int heads, int kv_heads, int head_dim, float scale, int window,
                      const int32_t* positions, const int32_t* slots, const void* k_pool, const void* v_pool,
                      const int32_t* page_table, int table_stride, int ring, int max_len, cudaStream_t stream) {
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
                 scale * 1.4426950408889634f, 0, 0, 0};
    note_launch();
    switch ((head_dim + 31) / 32) {
        case 1: launch<1>(a, visible, stream); break;
        case 2: launch<2>(a, visible, stream); break;
        case 3: launch<3>(a, visible, stream); break;
        default: launch<4>(a, visible, stream); break;
    }
}

}  // namespace sm
