// Decode attention over the paged cache for bfloat16: one new token per sequence attends to
// its sequence's keys (the reference scans [start, pos] per head on one thread:
// src/kernels.c:1156-1176).
//
// A thread-block cluster of 1 to 8 CTAs serves one (sequence, kv head); its CTAs split the
// visible positions, and within a CTA the eight warps take tiles of 32 positions in turn. The
// group's query heads are the 16 rows of the tensor-core tile (mma.sync m16n8k16), so every
// key and value row that is read serves all of them. A warp keeps a running maximum, sum and
// weighted values over its tiles (the next tile's keys and values are on their way while the
// current one is used); the warps of a CTA merge through shared memory, the CTAs of the
// cluster through distributed shared memory in rank order. There is no workspace in global
// memory and nothing depends on the order in which CTAs finish.
//
// Key rows are read straight from the cache into the B fragments (16 bytes a lane; the
// permutation of the head dimension inside a block of 32 is the same for q and k, so the
// dot products are unchanged); value rows go through shared memory to be read transposed.
#include <cooperative_groups.h>
#include <math_constants.h>

#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace sm {

namespace {

constexpr int kMaxWarps = 8;         // warps per CTA: 4 when CTAs are many, 8 when they are few
constexpr int kTile = 32;           // positions per warp tile
constexpr int kMaxCluster = 8;

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
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
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

// HDB: blocks of 32 of the head dimension (head_dim <= 32 * HDB, a multiple of 16).
template <int HDB, int kWarps>
__global__ void __launch_bounds__(kWarps * 32) decode_attention_kernel(DecodeArgs a) {
    constexpr int kThreads = kWarps * 32;
    constexpr int HDP = HDB * 32;            // padded head dimension
    constexpr int LDV = HDP + 8;             // value row in shared memory: conflict-free transposed reads
    constexpr int NT = HDP / 8;              // dim tiles of the output
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // per warp two value buffers [kTile][LDV]; after the loop the same memory holds the warps' results
    __nv_bfloat16* vs_all = reinterpret_cast<__nv_bfloat16*>(smem_raw);
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
    const int n_tiles = cta_hi > cta_lo ? (cta_hi - cta_lo + kTile - 1) / kTile : 0;
    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};
    __nv_bfloat16* vs = vs_all + (size_t)warp * 2 * kTile * LDV;

    // row offset of this lane's key of a tile (lane l <-> key l of the tile); ~0 marks "none"
    auto tile_offset = [&](int tile) -> unsigned long long {
        const int key = cta_lo + tile * kTile + lane;
        return key < cta_hi ? (unsigned long long)paged.row_offset(slot, key, kvh) : ~0ull;
    };
    int tile = warp;
    unsigned long long off = tile < n_tiles ? tile_offset(tile) : ~0ull;

    pdl_wait();   // q and the newest key and value come from the kernel before

    // Q fragments: rows g and g + 8 are heads kvh * group + g (+8); heads beyond the group are zero
    uint4 qa[HDB], qb[HDB];
    {
        const __nv_bfloat16* qrow = a.q + ((size_t)b * a.heads + (size_t)kvh * group) * hd;
#pragma unroll
        for (int kb = 0; kb < HDB; ++kb) {
            const int d = kb * 32 + q4 * 8;
            qa[kb] = (g < group && d < hd) ? *reinterpret_cast<const uint4*>(qrow + (size_t)g * hd + d) : make_uint4(0, 0, 0, 0);
            qb[kb] = (g + 8 < group && d < hd) ? *reinterpret_cast<const uint4*>(qrow + (size_t)(g + 8) * hd + d)
                                               : make_uint4(0, 0, 0, 0);
        }
    }
    uint4 kf[4][HDB];
    auto load_k = [&](unsigned long long my_off) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned long long o = __shfl_sync(0xffffffffu, my_off, 8 * j + g);   // key 8j + g of the tile
#pragma unroll
            for (int kb = 0; kb < HDB; ++kb) {
                const int d = kb * 32 + q4 * 8;
                kf[j][kb] = (o != ~0ull && d < hd) ? *reinterpret_cast<const uint4*>(a.k_pool + o + d) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    auto load_v = [&](unsigned long long my_off, int buf) {
        __nv_bfloat16* dst = vs + (size_t)buf * kTile * LDV;
        constexpr int CPR = HDP / 8;   // 16-byte chunks per row
#pragma unroll
        for (int c0 = 0; c0 < kTile * CPR; c0 += 32) {
            const int c = c0 + lane, row = c / CPR, col = (c % CPR) * 8;
            const unsigned long long o = __shfl_sync(0xffffffffu, my_off, row);
            const bool in = o != ~0ull && col < hd;
            cp_async16(dst + (size_t)row * LDV + col, a.v_pool + (in ? o + col : 0), in);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float o_acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

    if (tile < n_tiles) {
        load_k(off);
        load_v(off, 0);
    }
    int buf = 0;
    for (; tile < n_tiles; tile += kWarps, buf ^= 1) {
        const int next = tile + kWarps;
        const bool has_next = next < n_tiles;
        unsigned long long next_off = ~0ull;
        if (has_next) {
            next_off = tile_offset(next);
            __syncwarp();                 // the other buffer was read in the previous iteration
            load_v(next_off, buf ^ 1);
        }
        // S = Q K^T: 16 heads x 32 keys
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kb = 0; kb < HDB; ++kb) {
                mma_bf16(s[j], qa[kb].x, qb[kb].x, qa[kb].y, qb[kb].y, kf[j][kb].x, kf[j][kb].y);
                mma_bf16(s[j], qa[kb].z, qb[kb].z, qa[kb].w, qb[kb].w, kf[j][kb].z, kf[j][kb].w);
            }
        }
        if (has_next) load_k(next_off);   // the key registers are free again
        // scale, mask the keys beyond this CTA's range, running maximum
        const int kbase = cta_lo + tile * kTile;
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
        if (has_next) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        const __nv_bfloat16* vb = vs + (size_t)buf * kTile * LDV;
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                uint32_t b0, b1;
                ldmatrix_x2_trans(b0, b1, vb + (size_t)(jj * 16 + (lane & 15)) * LDV + i * 8);
                mma_bf16(o_acc[i], pf[jj][0], pf[jj][1], pf[jj][2], pf[jj][3], b0, b1);
            }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- the warps of this CTA, through shared memory (the value buffers are free now) -------
    __syncthreads();
    float* wm = reinterpret_cast<float*>(smem_raw);          // [kWarps][16] maxima
    float* wl = wm + kWarps * 16;                            // [kWarps][16] sums
    float* wo = wl + kWarps * 16;                            // [kWarps][16][HDP] weighted values
    // [cluster][group][HDP + 2], the leader's copy is used. It lies behind everything a CTA uses
    // for itself: other CTAs write here while this one may still be in its loop.
    constexpr size_t kLoopBytes = (size_t)kWarps * 2 * kTile * LDV * sizeof(__nv_bfloat16);
    constexpr size_t kLocalBytes = ((size_t)kWarps * 32 + (size_t)kWarps * 16 * HDP) * sizeof(float);
    float* part = reinterpret_cast<float*>(smem_raw + (kLoopBytes > kLocalBytes ? kLoopBytes : kLocalBytes));
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

template <int HDB, int kWarps>
void launch_w(const DecodeArgs& a, cudaStream_t stream) {
    constexpr int kThreads = kWarps * 32;
    constexpr int HDP = HDB * 32, LDV = HDP + 8;
    const int group = a.heads / a.kv_heads;
    const size_t loop_bytes = (size_t)kWarps * 2 * kTile * LDV * sizeof(__nv_bfloat16);
    const size_t local_bytes = ((size_t)kWarps * 32 + (size_t)kWarps * 16 * HDP) * sizeof(float);
    const size_t smem = (loop_bytes > local_bytes ? loop_bytes : local_bytes) +
                        (size_t)a.cluster * group * (HDP + 2) * sizeof(float);
    auto kernel = decode_attention_kernel<HDB, kWarps>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) throw std::runtime_error(std::string("attention_decode: ") + cudaGetErrorString(e));
    }
    launch_kernel("attention_decode", kernel, dim3(a.cluster, a.kv_heads, a.B), dim3(kThreads), smem, stream, a.cluster,
                  dependent_launch_enabled(), a);
}

template <int HDB>
void launch(const DecodeArgs& a, int warps, cudaStream_t stream) {
    if (warps == 8) launch_w<HDB, 8>(a, stream);
    else launch_w<HDB, 4>(a, stream);
}

}  // namespace

bool attention_decode_supports(int heads, int kv_heads, int head_dim) {
    return head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128 && kv_heads > 0 && heads % kv_heads == 0 &&
           heads / kv_heads <= 16;
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
    // CTAs per (sequence, kv head): fill the machine, but give every warp of every CTA a tile
    const int visible = window > 0 && window < max_len ? window : max_len;
    // measured on a B200 (14 heads on 2 kv heads, 2,100 keys): 8 warps win while the CTAs are few
    // (5.9 against 7.1 us at one sequence), 4 warps when they are many (8.5 against 11.2 us at 8)
    int cluster = 1;
    while (cluster < kMaxCluster && B * kv_heads * cluster < 296 && visible > cluster * 4 * kTile) cluster *= 2;
    const int warps = B * kv_heads * cluster <= 64 ? kMaxWarps : 4;
    DecodeArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
                 page_table, table_stride, ring, slots, positions, B, heads, kv_heads, head_dim, window, cluster,
                 scale * 1.4426950408889634f};
    note_launch();
    switch ((head_dim + 31) / 32) {
        case 1: launch<1>(a, warps, stream); break;
        case 2: launch<2>(a, warps, stream); break;
        case 3: launch<3>(a, warps, stream); break;
        default: launch<4>(a, warps, stream); break;
    }
}

}  // namespace sm
