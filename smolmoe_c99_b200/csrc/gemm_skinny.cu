// out[t, n] = sum_k x[t, k] * w[n, k] for a handful of tokens (decode: T <= 64) and
// bfloat16 weights: the step is bound by reading w once, so the kernel is built around
// streaming weight rows from HBM with nothing in the way, and everything that surrounds
// the product in a layer is folded into it so that a layer is five launches:
//   * prologue: x is either bfloat16 rows, or the float residual normalised on the fly
//     (RMSNorm: x * inv_rms * weight, rounded to bfloat16 as the stand-alone kernel does);
//   * epilogues: store (+bias), add into the float residual, act(gate) * up from two row
//     sets, or q/k/v with bias, rotation and the cache write (src/model.c:506-526).
//
// 16 output rows (two sets of 16 for gate/up) belong to a thread-block cluster of 1 to 8
// CTAs; the CTAs and their 8 warps each split K, so that even a small matrix has thousands
// of loads in flight. A CTA adds its warps' partial sums through its shared memory in warp
// order; the other CTAs then write theirs into the first CTA's shared memory (distributed
// shared memory) and it adds them in rank order and runs the epilogue. No workspace is
// needed and the result does not depend on timing. The products run on the tensor cores
// (mma.sync m16n8k16, float accumulate) with the weight rows as the 16-row operand and up
// to 8 tokens per instruction. Each lane loads 16 contiguous bytes of a row; the same
// permutation of k inside a 32-wide block is used for both operands, which leaves the dot
// products unchanged.
#include <cooperative_groups.h>
#include <math_constants.h>

#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace sm {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

enum SkinnyMode : int { SK_STORE = 0, SK_RESIDUAL = 1, SK_SWIGLU = 2, SK_QKV_ROPE = 3 };

struct SkinnyArgs {
    const void* x;              // bf16 [T, K], or float [T, K] when norm_w is set
    const void* norm_w;         // [K] or null
    int norm_w_dt;
    float eps;
    const __nv_bfloat16* w;     // [rows, K]
    int T, N, K;
    int mode;
    const void* bias;
    int bias_dt;
    void* out;
    int out_dt;
    int up_offset;
    // SK_QKV_ROPE
    int heads, kv_heads, head_dim;
    const int32_t* positions;
    const float* cos_table;
    const float* sin_table;
    void* q_out;
    int dt;
    void* k_pool;
    void* v_pool;
    const int32_t* page_table;
    int table_stride, ring;
    const int32_t* token_slot;
    int cluster;                // CTAs that share a tile (1..8)
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// weights are read once: do not keep them in L1
__device__ __forceinline__ uint4 ldg16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Which global row of w the tile's row r (0..15) is, for set s (0: gate or the only set, 1: up).
__device__ __forceinline__ int tile_row(const SkinnyArgs& a, int tile, int r, int set, bool* valid) {
    if (a.mode == SK_QKV_ROPE) {
        // tiles: for every q and k head half/8 tiles of 8 pairs (rows 0-7: dims i0.., rows 8-15:
        // dims i0 + half..), then for every v head head_dim/16 tiles of 16 dims
        const int hd = a.head_dim, half = hd / 2, per_rot = half / 8, per_v = hd / 16;
        const int rot_tiles = (a.heads + a.kv_heads) * per_rot;
        *valid = true;
        if (tile < rot_tiles) {
            int head = tile / per_rot, i0 = (tile - head * per_rot) * 8;
            return head * hd + (r < 8 ? i0 + r : half + i0 + (r - 8));
        }
        int vt = tile - rot_tiles, head = vt / per_v, d0 = (vt - head * per_v) * 16;
        return (a.heads + a.kv_heads + head) * hd + d0 + r;
    }
    int n = tile * 16 + r;
    *valid = n < a.N;
    return (*valid ? n : a.N - 1) + (set ? a.up_offset : 0);
}

// k blocks (of 32) a warp holds in registers at once, and a CTA stages of x per round
template <bool DUAL> struct Round { static constexpr int kPre = DUAL ? 2 : 4; };

template <int NT, bool NORM, bool DUAL>
__global__ void __launch_bounds__(kThreads, 2) gemm_skinny_kernel(SkinnyArgs a) {
    constexpr int SETS = DUAL ? 2 : 1, COLS = NT * 8 + 1;
    constexpr int kPre = Round<DUAL>::kPre;
    constexpr int kRoundK = kWarps * kPre * 32;          // k covered by one round of the CTA
    constexpr int kXStride = kRoundK + 32;               // bf16 elements; 64 bytes of padding: conflict-free fragment reads
    extern __shared__ __align__(16) float smem_f[];
    float (*red)[SETS][16][COLS] = reinterpret_cast<float (*)[SETS][16][COLS]>(smem_f);                 // [kWarps]
    float (*across)[SETS][16][COLS] = reinterpret_cast<float (*)[SETS][16][COLS]>(smem_f + kWarps * SETS * 16 * COLS);  // [cluster]
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_f + (size_t)(kWarps + a.cluster) * SETS * 16 * COLS);  // [NT*8][kXStride]
    __shared__ float inv_rms[NT * 8];
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = a.cluster > 1 ? (int)cluster.block_rank() : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;       // row (or token) within 8, 16-byte column within the 32-wide k block
    const int tile = blockIdx.x / a.cluster;
    const int K = a.K, kblocks = (K + 31) / 32;
    // this CTA's contiguous share of the k blocks
    const int per_cta = (kblocks + a.cluster - 1) / a.cluster;
    const int cta0 = rank * per_cta, cta1 = min(kblocks, cta0 + per_cta);

    bool v0, v1, vu;
    const __nv_bfloat16* row_lo = a.w + (size_t)tile_row(a, tile, g, 0, &v0) * K;
    const __nv_bfloat16* row_hi = a.w + (size_t)tile_row(a, tile, g + 8, 0, &v1) * K;
    const __nv_bfloat16* up_lo = DUAL ? a.w + (size_t)tile_row(a, tile, g, 1, &vu) * K : nullptr;
    const __nv_bfloat16* up_hi = DUAL ? a.w + (size_t)tile_row(a, tile, g + 8, 1, &vu) * K : nullptr;

    float acc[SETS][NT][4];
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.f;

    bool norms_done = !NORM;
    for (int round0 = cta0; round0 < cta1; round0 += kWarps * kPre) {
        const int round_blocks = min(kWarps * kPre, cta1 - round0);
        const int per_warp = (round_blocks + kWarps - 1) / kWarps;       // <= kPre
        const int wb0 = round0 + warp * per_warp, wb1 = min(round0 + round_blocks, wb0 + per_warp);
        // every weight chunk of this warp's share of the round is requested before anything waits
        uint4 wl[kPre], wh[kPre], ul[kPre], uh[kPre];
#pragma unroll
        for (int i = 0; i < kPre; ++i) {
            const int k = (wb0 + i) * 32 + q * 8;
            const bool in = wb0 + i < wb1 && k < K;
            wl[i] = in ? ldg16_stream(row_lo + k) : make_uint4(0, 0, 0, 0);
            wh[i] = in ? ldg16_stream(row_hi + k) : make_uint4(0, 0, 0, 0);
            if (DUAL) {
                ul[i] = in ? ldg16_stream(up_lo + k) : make_uint4(0, 0, 0, 0);
                uh[i] = in ? ldg16_stream(up_hi + k) : make_uint4(0, 0, 0, 0);
            }
        }
        if (round0 == cta0) {
            // the weights are on their way: let the next kernel in, then wait for the previous one,
            // whose output x is
            pdl_launch_dependents();
            pdl_wait();
        }
        if (!norms_done) {
            // inverse RMS of every token's row: warps take tokens in turn
            const float* xf = (const float*)a.x;
            for (int t = warp; t < NT * 8; t += kWarps) {
                float sq = 0.f;
                if (t < a.T)
                    for (int k0 = lane * 4; k0 < K; k0 += 8 * 128) {
                        // eight loads in flight, then the sums: one trip to L2 per 1024 elements
                        float4 v[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const int k = k0 + u * 128;
                            v[u] = k < K ? *reinterpret_cast<const float4*>(xf + (size_t)t * K + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            sq = fmaf(v[u].x, v[u].x, sq); sq = fmaf(v[u].y, v[u].y, sq);
                            sq = fmaf(v[u].z, v[u].z, sq); sq = fmaf(v[u].w, v[u].w, sq);
                        }
                    }
                sq = warp_sum(sq);
                if (lane == 0) inv_rms[t] = 1.0f / sqrtf(sq / (float)K + a.eps);
            }
            norms_done = true;
        }
        __syncthreads();   // inv_rms is ready; the previous round's x has been read
        // x of this round's k range, normalised if asked, as bfloat16 rows in shared memory
        const int k_lo = round0 * 32, chunks = round_blocks * 4;          // 16-byte chunks per row
        for (int idx = threadIdx.x; idx < a.T * chunks; idx += kThreads) {
            const int t = idx / chunks, c = idx - t * chunks;
            const int k = k_lo + c * 8;
            uint4 xb = make_uint4(0, 0, 0, 0);
            if (k < K) {
                if (NORM) {
                    const float* xp = (const float*)a.x + (size_t)t * K + k;
                    const float4 p0 = *reinterpret_cast<const float4*>(xp), p1 = *reinterpret_cast<const float4*>(xp + 4);
                    float nw[8];
                    if (a.norm_w_dt == F32) {
                        const float4 n0 = *reinterpret_cast<const float4*>((const float*)a.norm_w + k);
                        const float4 n1 = *reinterpret_cast<const float4*>((const float*)a.norm_w + k + 4);
                        nw[0] = n0.x; nw[1] = n0.y; nw[2] = n0.z; nw[3] = n0.w; nw[4] = n1.x; nw[5] = n1.y; nw[6] = n1.z; nw[7] = n1.w;
                    } else {
                        const uint4 raw = ldg16((const __nv_bfloat16*)a.norm_w + k);
                        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                        for (int e = 0; e < 4; ++e) { float2 f = __bfloat1622float2(h[e]); nw[2 * e] = f.x; nw[2 * e + 1] = f.y; }
                    }
                    const float inv = inv_rms[t];
                    xb.x = pack2((p0.x * inv) * nw[0], (p0.y * inv) * nw[1]);
                    xb.y = pack2((p0.z * inv) * nw[2], (p0.w * inv) * nw[3]);
                    xb.z = pack2((p1.x * inv) * nw[4], (p1.y * inv) * nw[5]);
                    xb.w = pack2((p1.z * inv) * nw[6], (p1.w * inv) * nw[7]);
                } else {
                    xb = ldg16((const __nv_bfloat16*)a.x + (size_t)t * K + k);
                }
            }
            *reinterpret_cast<uint4*>(xs + (size_t)t * kXStride + c * 8) = xb;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kPre; ++i) {
            if (wb0 + i >= wb1) break;
            const int c = (wb0 + i - round0) * 4 + q;                    // this lane's chunk within the staged row
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int t = j * 8 + g;
                const uint4 xb = t < a.T ? *reinterpret_cast<const uint4*>(xs + (size_t)t * kXStride + c * 8)
                                         : make_uint4(0, 0, 0, 0);
                mma16816(acc[0][j], wl[i].x, wh[i].x, wl[i].y, wh[i].y, xb.x, xb.y);
                mma16816(acc[0][j], wl[i].z, wh[i].z, wl[i].w, wh[i].w, xb.z, xb.w);
                if (DUAL) {
                    mma16816(acc[1][j], ul[i].x, uh[i].x, ul[i].y, uh[i].y, xb.x, xb.y);
                    mma16816(acc[1][j], ul[i].z, uh[i].z, ul[i].w, uh[i].w, xb.z, xb.w);
                }
            }
        }
    }
    if (cta0 >= cta1) {   // a CTA without k blocks
        pdl_launch_dependents();
        pdl_wait();
    }
    // partial sums of this warp: rows g and g + 8, tokens 2q and 2q + 1 of each group of 8
#pragma unroll
    for (int s = 0; s < (DUAL ? 2 : 1); ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            red[warp][s][g][j * 8 + 2 * q] = acc[s][j][0];
            red[warp][s][g][j * 8 + 2 * q + 1] = acc[s][j][1];
            red[warp][s][g + 8][j * 8 + 2 * q] = acc[s][j][2];
            red[warp][s][g + 8][j * 8 + 2 * q + 1] = acc[s][j][3];
        }
    __syncthreads();
    // this CTA's sums over its warps, in warp order, into `across[rank]` of the first CTA
    {
        float (*dst)[SETS][16][COLS] = a.cluster > 1 ? cluster.map_shared_rank(across, 0) : across;
        for (int idx = threadIdx.x; idx < SETS * 16 * NT * 8; idx += kThreads) {
            const int s = idx / (16 * NT * 8), r = (idx / (NT * 8)) % 16, t = idx % (NT * 8);
            float v = 0.f;
#pragma unroll
            for (int wv = 0; wv < kWarps; ++wv) v += red[wv][s][r][t];
            dst[rank][s][r][t] = v;
        }
    }
    if (a.cluster > 1) {
        cluster.sync();
        if (rank != 0) return;
    } else {
        __syncthreads();
    }

    if (a.mode == SK_QKV_ROPE) {
        // one thread per (pair or element pair, token): rows r and r + 8 of the tile
        const int hd = a.head_dim, half = hd / 2, per_rot = half / 8, per_v = hd / 16;
        const int rot_tiles = (a.heads + a.kv_heads) * per_rot;
        for (int idx = threadIdx.x; idx < 8 * NT * 8; idx += kThreads) {
            const int r = idx / (NT * 8), t = idx - r * (NT * 8);
            if (t >= a.T) continue;
            float lo = 0.f, hi = 0.f;
            for (int c = 0; c < a.cluster; ++c) { lo += across[c][0][r][t]; hi += across[c][0][r + 8][t]; }
            bool dummy;
            const int n_lo = tile_row(a, tile, r, 0, &dummy), n_hi = tile_row(a, tile, r + 8, 0, &dummy);
            if (a.bias) {
                lo += a.bias_dt == F32 ? ((const float*)a.bias)[n_lo] : __bfloat162float(((const __nv_bfloat16*)a.bias)[n_lo]);
                hi += a.bias_dt == F32 ? ((const float*)a.bias)[n_hi] : __bfloat162float(((const __nv_bfloat16*)a.bias)[n_hi]);
            }
            const int pos = a.positions[t];
            const int head = n_lo / hd, d_lo = n_lo - head * hd, d_hi = n_hi - head * hd;
            if (tile < rot_tiles) {
                const float c = a.cos_table[(size_t)pos * half + d_lo], s = a.sin_table[(size_t)pos * half + d_lo];
                const float r0 = lo * c - hi * s, r1 = lo * s + hi * c;
                lo = r0;
                hi = r1;
            }
            if (head < a.heads) {
                __nv_bfloat16* qo = (__nv_bfloat16*)a.q_out + ((size_t)t * a.heads + head) * hd;
                qo[d_lo] = __float2bfloat16_rn(lo);
                qo[d_hi] = __float2bfloat16_rn(hi);
            } else {
                const bool is_v = head >= a.heads + a.kv_heads;
                const int kvh = is_v ? head - a.heads - a.kv_heads : head - a.heads;
                PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};
                __nv_bfloat16* c = (__nv_bfloat16*)(is_v ? a.v_pool : a.k_pool) + paged.row_offset(a.token_slot[t], pos, kvh);
                c[d_lo] = __float2bfloat16_rn(lo);
                c[d_hi] = __float2bfloat16_rn(hi);
            }
        }
        return;
    }
    for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += kThreads) {
        const int r = idx / (NT * 8), t = idx - r * (NT * 8);
        const int n = tile * 16 + r;
        if (t >= a.T || n >= a.N) continue;
        float v = 0.f, u = 0.f;
        for (int c = 0; c < a.cluster; ++c) {
            v += across[c][0][r][t];
            if (DUAL) u += across[c][DUAL ? 1 : 0][r][t];
        }
        const size_t o = (size_t)t * a.N + n;
        if (a.mode == SK_SWIGLU) v = u * (v / (1.0f + expf(-v)));
        else if (a.bias) v += a.bias_dt == F32 ? ((const float*)a.bias)[n] : __bfloat162float(((const __nv_bfloat16*)a.bias)[n]);
        if (a.mode == SK_RESIDUAL) ((float*)a.out)[o] += v;
        else if (a.out_dt == F32) ((float*)a.out)[o] = v;
        else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(v);
    }
}

template <int NT, bool NORM, bool DUAL>
void launch_one(const SkinnyArgs& a, int tiles, cudaStream_t stream) {
    constexpr int SETS = DUAL ? 2 : 1, COLS = NT * 8 + 1;
    constexpr int kXStride = kWarps * Round<DUAL>::kPre * 32 + 32;
    const size_t smem = (size_t)(kWarps + a.cluster) * SETS * 16 * COLS * sizeof(float) +
                        (size_t)NT * 8 * kXStride * sizeof(__nv_bfloat16);
    auto kernel = gemm_skinny_kernel<NT, NORM, DUAL>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) throw std::runtime_error(std::string("gemm_skinny: ") + cudaGetErrorString(e));
    }
    launch_kernel("gemm_skinny", kernel, dim3((unsigned)(tiles * a.cluster)), dim3(kThreads), smem, stream, a.cluster,
                  dependent_launch_enabled(), a);
}

template <int NT>
void launch_nt(const SkinnyArgs& a, int tiles, cudaStream_t stream) {
    const bool norm = a.norm_w != nullptr, dual = a.mode == SK_SWIGLU;
    if (norm && dual) launch_one<NT, true, true>(a, tiles, stream);
    else if (norm) launch_one<NT, true, false>(a, tiles, stream);
    else if (dual) launch_one<NT, false, true>(a, tiles, stream);
    else launch_one<NT, false, false>(a, tiles, stream);
}

// CTAs per tile. Measured on a B200 (decode shapes of a 0.5B model, 8 tokens): a CTA should get
// through its share of K in one round of prefetched weights, but clusters are not free (their
// CTAs must be co-scheduled and meet at a cluster barrier) and more CTAs than fit the machine at
// once cost a second wave; so: the smallest cluster of at most 4 that reaches one round, as
// long as all CTAs are resident together (2 per SM).
int pick_cluster(int tiles, int K, bool dual) {
    const int kblocks = (K + 31) / 32;
    const int round_blocks = kWarps * (dual ? Round<true>::kPre : Round<false>::kPre);
    const int resident = 148 * 2;
    int c = 1;
    while (c < 4 && (kblocks + c - 1) / c > round_blocks && tiles * c * 2 <= resident) c *= 2;
    return c;
}

}  // namespace

bool gemm_skinny_supports(int T, int N, int K) { return T > 0 && T <= 32 && N > 0 && K > 0 && K % 8 == 0; }

void gemm_skinny(const void* x, const void* norm_w, DType norm_w_dt, float eps, const void* w, int T, int N, int K,
                 int mode, const void* bias, DType bias_dt, void* out, DType out_dt, int up_offset,
                 const SkinnyRope* rope, cudaStream_t stream) {
    if (!gemm_skinny_supports(T, N, K))
        throw std::invalid_argument("gemm_skinny: T = " + std::to_string(T) + " must be at most 32 and K = " +
                                    std::to_string(K) + " a multiple of 8");
    if (((uintptr_t)x | (uintptr_t)w) & 15) throw std::invalid_argument("gemm_skinny: operands must be 16-byte aligned");
    SkinnyArgs a{};
    a.x = x; a.norm_w = norm_w; a.norm_w_dt = norm_w_dt; a.eps = eps;
    a.w = (const __nv_bfloat16*)w; a.T = T; a.N = N; a.K = K; a.mode = mode;
    a.bias = bias; a.bias_dt = bias_dt; a.out = out; a.out_dt = out_dt; a.up_offset = up_offset;
    int tiles = (N + 15) / 16;
    if (mode == SK_QKV_ROPE) {
        if (!rope) throw std::invalid_argument("gemm_skinny: the q/k/v epilogue needs its arguments");
        if (rope->head_dim % 16 || rope->rotary_dim != rope->head_dim)
            throw std::invalid_argument("gemm_skinny: the fused q/k/v epilogue takes head sizes that are multiples of 16 with full rotation");
        if (N != (rope->heads + 2 * rope->kv_heads) * rope->head_dim)
            throw std::invalid_argument("gemm_skinny: q/k/v rows do not match the head counts");
        a.heads = rope->heads; a.kv_heads = rope->kv_heads; a.head_dim = rope->head_dim;
        a.positions = rope->positions; a.cos_table = rope->cos_table; a.sin_table = rope->sin_table;
        a.q_out = rope->q_out; a.k_pool = rope->k_pool; a.v_pool = rope->v_pool; a.page_table = rope->page_table;
        a.table_stride = rope->table_stride; a.ring = rope->ring; a.token_slot = rope->token_slot;
        tiles = N / 16;
    }
    a.cluster = pick_cluster(tiles, K, mode == SK_SWIGLU);
    note_launch();
    if (T <= 8) launch_nt<1>(a, tiles, stream);
    else if (T <= 16) launch_nt<2>(a, tiles, stream);
    else launch_nt<4>(a, tiles, stream);
}

}  // namespace sm
