// out[t, n] = sum_k x[t, k] * w[n, k] for a handful of tokens (decode: T <= 32) and
// bfloat16 weights. The step is bound by reading w once, and every product of a layer is
// small (1.6 to 17 MB), so the kernel is built to have ALL of its weight bytes in flight at
// once and to fold in what surrounds the product, so that a layer is five launches:
//   * prologue: x is either bfloat16 rows, or the float residual normalised on the fly
//     (RMSNorm: x * inv_rms * weight, rounded to bfloat16 as the stand-alone kernel does);
//   * epilogues: store (+bias), add into the float residual, act(gate) * up from two row
//     sets, or q/k/v with bias, rotation and the cache write (src/model.c:506-526).
//
// 16 output rows (two sets of 16 for gate/up) belong to a thread-block cluster of 1, 2 or 4
// CTAs that split K. The first thing a CTA does -- before it waits for the kernel before it
// (programmatic dependent launch) -- is to ask for its whole share of the weights: one thread
// issues a bulk copy (cp.async.bulk, the TMA engine) per weight row into shared memory, all
// on one mbarrier. Shared memory rather than registers holds the bytes in flight, so three
// CTAs fit an SM and even the largest product of a 0.5B model is one wave. While the weights
// travel, the CTA stages x (computing the norm if asked). Then its 8 warps split the CTA's
// share of K, multiply on the tensor cores (mma.sync m16n8k16, operands by ldmatrix) and add
// their partial sums through shared memory in warp order; the other CTAs of the cluster write
// theirs into the first CTA's shared memory (distributed shared memory) and it adds them in
// rank order and runs the epilogue. No workspace, and no result depends on timing.
//
// The wait for the weights is bounded: if it runs out the CTA records a code in the library's
// error word and leaves without writing.
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
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr int kOperandBytes = 73 * 1024;   // shared memory for the operands of a round: three CTAs fit an SM

// k elements of a CTA's share that are in shared memory at once, for a tile of `rows` operand rows
// (16 or 32 of the weights and 8, 16 or 32 tokens): at most 1536, a multiple of 32.
constexpr int max_round_k(int rows) {
    int k = (kOperandBytes / (rows * 2) - 8) / 32 * 32;
    return k < 1536 ? k : 1536;
}

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
    void* k_pool;
    void* v_pool;
    const int32_t* page_table;
    int table_stride, ring;
    const int32_t* token_slot;
    void* k_packed;             // or null: the step's rotated keys and its values, packed [T, kv_heads, head_dim]
    void* v_packed;
    const int32_t* token_end;   // or null: with a ring, positions before token_end - ring are not stored
    int cluster;                // CTAs that share a tile (1, 2 or 4)
    int round_k;                // k elements staged per round (a multiple of 32)
    int* error;
    int act;                    // SK_SWIGLU: the activation (Activation in common.cuh)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}
__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// One contiguous run of bytes (a multiple of 16, both ends on 16 bytes) from global to shared memory.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void load_norm_weight8(const SkinnyArgs& a, int k, float (&nw)[8]) {
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
}

// Which global row of w the tile's row r (0..15) is, for set s (0: gate or the only set, 1: up).
__device__ __forceinline__ int tile_row(const SkinnyArgs& a, int tile, int r, int set) {
    if (a.mode == SK_QKV_ROPE) {
        // tiles: for every q and k head half/8 tiles of 8 pairs (rows 0-7: dims i0.., rows 8-15:
        // dims i0 + half..), then for every v head head_dim/16 tiles of 16 dims
        const int hd = a.head_dim, half = hd / 2, per_rot = half / 8, per_v = hd / 16;
        const int rot_tiles = (a.heads + a.kv_heads) * per_rot;
        if (tile < rot_tiles) {
            int head = tile / per_rot, i0 = (tile - head * per_rot) * 8;
            return head * hd + (r < 8 ? i0 + r : half + i0 + (r - 8));
        }
        int vt = tile - rot_tiles, head = vt / per_v, d0 = (vt - head * per_v) * 16;
        return (a.heads + a.kv_heads + head) * hd + d0 + r;
    }
    int n = tile * 16 + r;
    return (n < a.N ? n : a.N - 1) + (set ? a.up_offset : 0);   // rows past the end repeat the last one and are masked
}

template <int NT, bool NORM, bool DUAL>
__global__ void __launch_bounds__(kThreads, 3) gemm_skinny_kernel(SkinnyArgs a) {
    constexpr int SETS = DUAL ? 2 : 1, TOK = NT * 8, COLS = TOK + 1;
    const int stride = a.round_k + 8;                      // bf16 elements: 16 bytes of padding keep ldmatrix conflict-free
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* ws = reinterpret_cast<__nv_bfloat16*>(smem_raw);                       // [SETS][16][stride]
    __nv_bfloat16* xs = ws + (size_t)SETS * 16 * stride;                                  // [TOK][stride]
    // the warps' partial sums reuse the operands' space once the products are done; the cluster's do
    // not, since another CTA may write them while this one still multiplies
    float (*red)[SETS][16][COLS] = reinterpret_cast<float (*)[SETS][16][COLS]>(smem_raw);                         // [kWarps]
    size_t operand_bytes = (size_t)(SETS * 16 + TOK) * stride * sizeof(__nv_bfloat16);
    if (operand_bytes < sizeof(float) * kWarps * SETS * 16 * COLS) operand_bytes = (sizeof(float) * kWarps * SETS * 16 * COLS + 15) / 16 * 16;
    float (*across)[SETS][16][COLS] = reinterpret_cast<float (*)[SETS][16][COLS]>(smem_raw + operand_bytes);     // [cluster]
    __shared__ float squares[4][TOK];      // per CTA of the cluster and token: sum of x^2 over that CTA's share of K
    __shared__ __align__(8) uint64_t weights_bar;
    __shared__ int failed;
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = a.cluster > 1 ? (int)cluster.block_rank() : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.cluster;
    const int K = a.K;
    // this CTA's contiguous share of K, in multiples of 32
    const int kblocks = (K + 31) / 32, per_cta = (kblocks + a.cluster - 1) / a.cluster;
    const int k_cta0 = min(K, rank * per_cta * 32), k_cta1 = min(K, (rank + 1) * per_cta * 32);
    const int rounds = (k_cta1 - k_cta0 + a.round_k - 1) / a.round_k;

    // the first warp asks for every weight row of a round: a bulk copy per lane, all on one barrier
    auto request_weights = [&](int k_lo, int k_hi) {
        const uint32_t bytes = (uint32_t)(k_hi - k_lo) * 2;      // K and k_lo are multiples of 8: 16-byte runs
        if (lane == 0) mbar_expect_tx(&weights_bar, bytes * 16 * SETS);
        __syncwarp();
        if (lane < 16 * SETS)
            bulk_load(ws + (size_t)lane * stride, a.w + (size_t)tile_row(a, tile, lane & 15, lane >> 4) * K + k_lo, bytes,
                      &weights_bar);
    };
    if (warp == 0) {
        if (lane == 0) {
            mbar_init(&weights_bar, 1);
            failed = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        if (rounds > 0) request_weights(k_cta0, min(k_cta1, k_cta0 + a.round_k));
    }
    // the weights are on their way: let the next kernel in, then wait for the previous one, whose output x is
    pdl_launch_dependents();
    pdl_wait();

    // What the epilogue will need from memory is asked for now, so that it arrives while the product runs.
    // q/k/v: one thread per (rotation pair or pair of v elements, token), rows r and r + 8 of the tile.
    float pre_a = 0.f, pre_b = 0.f, pre_cos = 1.f, pre_sin = 0.f;
    __nv_bfloat16* dst_lo = nullptr;
    __nv_bfloat16* dst_hi = nullptr;
    __nv_bfloat16* packed_lo = nullptr;      // keys and values also go to the step's packed tensors, where it has them
    __nv_bfloat16* packed_hi = nullptr;
    if (a.mode == SK_QKV_ROPE) {
        const int r = threadIdx.x / TOK, t = threadIdx.x - r * TOK;
        if (r < 8 && t < a.T) {
            const int hd = a.head_dim, half = hd / 2, per_rot = half / 8;
            const int rot_tiles = (a.heads + a.kv_heads) * per_rot;
            const int n_lo = tile_row(a, tile, r, 0), n_hi = tile_row(a, tile, r + 8, 0);
            const int pos = a.positions[t];
            const int head = n_lo / hd, d_lo = n_lo - head * hd, d_hi = n_hi - head * hd;
            if (a.bias) {
                pre_a = a.bias_dt == F32 ? ((const float*)a.bias)[n_lo] : __bfloat162float(((const __nv_bfloat16*)a.bias)[n_lo]);
                pre_b = a.bias_dt == F32 ? ((const float*)a.bias)[n_hi] : __bfloat162float(((const __nv_bfloat16*)a.bias)[n_hi]);
            }
            if (tile < rot_tiles) {
                pre_cos = a.cos_table[(size_t)pos * half + d_lo];
                pre_sin = a.sin_table[(size_t)pos * half + d_lo];
            }
            if (head < a.heads) {
                dst_lo = (__nv_bfloat16*)a.q_out + ((size_t)t * a.heads + head) * hd;
            } else {
                const bool is_v = head >= a.heads + a.kv_heads;
                const int kvh = is_v ? head - a.heads - a.kv_heads : head - a.heads;
                if (a.k_pool != nullptr && !(a.ring > 0 && a.token_end != nullptr && pos < a.token_end[t] - a.ring)) {
                    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, hd};
                    dst_lo = (__nv_bfloat16*)(is_v ? a.v_pool : a.k_pool) + paged.row_offset(a.token_slot[t], pos, kvh);
                }
                if (a.k_packed != nullptr) {
                    packed_lo = (__nv_bfloat16*)(is_v ? a.v_packed : a.k_packed) + ((size_t)t * a.kv_heads + kvh) * hd;
                    packed_hi = packed_lo + d_hi;
                    packed_lo += d_lo;
                }
            }
            if (dst_lo != nullptr) {
                dst_hi = dst_lo + d_hi;
                dst_lo += d_lo;
            }
        }
    } else {
        // the others: thread -> (row r, token t) of the tile, twice if there are more than 256 of them
        const int idx = threadIdx.x, r = idx / TOK, t = idx - r * TOK;
        const int n = tile * 16 + r;
        if (a.mode == SK_RESIDUAL) {
            if (r < 16 && t < a.T && n < a.N) pre_a = ((const float*)a.out)[(size_t)t * a.N + n];
            if (TOK * 16 > kThreads) {
                const int r2 = (idx + kThreads) / TOK, n2 = tile * 16 + r2;
                if (r2 < 16 && t < a.T && n2 < a.N) pre_b = ((const float*)a.out)[(size_t)t * a.N + n2];
            }
        } else if (a.mode == SK_STORE && a.bias) {
            if (r < 16 && n < a.N)
                pre_a = a.bias_dt == F32 ? ((const float*)a.bias)[n] : __bfloat162float(((const __nv_bfloat16*)a.bias)[n]);
            if (TOK * 16 > kThreads) {
                const int r2 = (idx + kThreads) / TOK, n2 = tile * 16 + r2;
                if (r2 < 16 && n2 < a.N)
                    pre_b = a.bias_dt == F32 ? ((const float*)a.bias)[n2] : __bfloat162float(((const __nv_bfloat16*)a.bias)[n2]);
            }
        }
    }
    __syncthreads();   // the barrier and `failed` are set up

    float acc[SETS][NT][4];
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.f;
    float sq[NT];          // this lane's share of the sums of squares of tokens warp, warp + 8, ...
#pragma unroll
    for (int j = 0; j < NT; ++j) sq[j] = 0.f;

    int round = 0;
    for (; round < rounds; ++round) {
        const int k_lo = k_cta0 + round * a.round_k, k_hi = min(k_cta1, k_lo + a.round_k);
        const int span = k_hi - k_lo, span16 = (span + 15) / 16 * 16;
        if (round > 0) {
            __syncthreads();   // the previous round's operands have been read
            if (warp == 0) {
                // the copies overwrite what ldmatrix has just read: order the two kinds of access
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                request_weights(k_lo, k_hi);
            }
        }
        // x of this round's k range as bfloat16 rows: warp w stages tokens w, w + 8, ...; a lane takes the
        // chunks of 8 whose number within the CTA's share is its own modulo 32, in rising order, so that a
        // token's sum of squares is added up in the same order however the share is cut into rounds.
        // With a norm, x * weight is staged and the sum's 1 / rms is applied to the product at the end.
        {
            const int chunks = span16 / 8, valid_chunks = span / 8;
            const int first = (lane - ((k_lo - k_cta0) >> 3)) & 31;
            constexpr int U = NORM && NT > 1 ? 2 : 4;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int t = j * 8 + warp;
                __nv_bfloat16* row = xs + (size_t)t * stride;
                const bool live = t < a.T;
                for (int c0 = first; c0 < chunks; c0 += 32 * U) {
                    uint4 xb[U];
                    if (NORM && a.norm_w_dt == BF16) {
                        float4 p[U][2];
                        uint4 nraw[U];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const int c = c0 + 32 * u;
                            if (live && c < valid_chunks) {
                                const float* xp = (const float*)a.x + (size_t)t * K + k_lo + c * 8;
                                p[u][0] = *reinterpret_cast<const float4*>(xp);
                                p[u][1] = *reinterpret_cast<const float4*>(xp + 4);
                                nraw[u] = ldg16((const __nv_bfloat16*)a.norm_w + k_lo + c * 8);
                            } else {
                                p[u][0] = p[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                                nraw[u] = make_uint4(0, 0, 0, 0);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&nraw[u]);
                            const float2 n0 = __bfloat1622float2(h[0]), n1 = __bfloat1622float2(h[1]);
                            const float2 n2 = __bfloat1622float2(h[2]), n3 = __bfloat1622float2(h[3]);
                            const float4 p0 = p[u][0], p1 = p[u][1];
                            float s = sq[j];
                            s = fmaf(p0.x, p0.x, s); s = fmaf(p0.y, p0.y, s); s = fmaf(p0.z, p0.z, s); s = fmaf(p0.w, p0.w, s);
                            s = fmaf(p1.x, p1.x, s); s = fmaf(p1.y, p1.y, s); s = fmaf(p1.z, p1.z, s); s = fmaf(p1.w, p1.w, s);
                            sq[j] = s;
                            xb[u].x = pack2(p0.x * n0.x, p0.y * n0.y);
                            xb[u].y = pack2(p0.z * n1.x, p0.w * n1.y);
                            xb[u].z = pack2(p1.x * n2.x, p1.y * n2.y);
                            xb[u].w = pack2(p1.z * n3.x, p1.w * n3.y);
                        }
                    } else if (NORM) {
                        // norm weights kept in 32 bits: the same, one chunk at a time
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const int c = c0 + 32 * u;
                            xb[u] = make_uint4(0, 0, 0, 0);
                            if (live && c < valid_chunks) {
                                const float* xp = (const float*)a.x + (size_t)t * K + k_lo + c * 8;
                                const float4 p0 = *reinterpret_cast<const float4*>(xp), p1 = *reinterpret_cast<const float4*>(xp + 4);
                                float nw[8];
                                load_norm_weight8(a, k_lo + c * 8, nw);
                                float s = sq[j];
                                s = fmaf(p0.x, p0.x, s); s = fmaf(p0.y, p0.y, s); s = fmaf(p0.z, p0.z, s); s = fmaf(p0.w, p0.w, s);
                                s = fmaf(p1.x, p1.x, s); s = fmaf(p1.y, p1.y, s); s = fmaf(p1.z, p1.z, s); s = fmaf(p1.w, p1.w, s);
                                sq[j] = s;
                                xb[u].x = pack2(p0.x * nw[0], p0.y * nw[1]);
                                xb[u].y = pack2(p0.z * nw[2], p0.w * nw[3]);
                                xb[u].z = pack2(p1.x * nw[4], p1.y * nw[5]);
                                xb[u].w = pack2(p1.z * nw[6], p1.w * nw[7]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const int c = c0 + 32 * u;
                            xb[u] = live && c < valid_chunks ? ldg16((const __nv_bfloat16*)a.x + (size_t)t * K + k_lo + c * 8)
                                                             : make_uint4(0, 0, 0, 0);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int c = c0 + 32 * u;
                        if (c < chunks) *reinterpret_cast<uint4*>(row + c * 8) = xb[u];
                    }
                }
            }
        }
        // the weights of this round have landed (bounded wait)
        {
            bool ok = false;
            for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
                if (mbar_try_wait(&weights_bar, (uint32_t)round & 1u)) { ok = true; break; }
            if (!ok) failed = 1;
        }
        // the tail of a last block of 16 that the copies did not cover reads as zero
        if (span16 > span)
            for (int idx = threadIdx.x; idx < SETS * 16; idx += kThreads)
                *reinterpret_cast<uint4*>(ws + (size_t)idx * stride + span) = make_uint4(0, 0, 0, 0);
        __syncthreads();
        if (failed) break;
        // the warps take the blocks of 16 in turn, counted from the start of the CTA's share (so that a
        // warp's sum does not depend on how the share is cut into rounds)
        const int blocks16 = span16 / 16;
        for (int blk = (warp - ((k_lo - k_cta0) >> 4)) & (kWarps - 1); blk < blocks16; blk += kWarps) {
            const int k = blk * 16;
            uint32_t af[SETS][4];
#pragma unroll
            for (int s = 0; s < SETS; ++s)
                ldmatrix_x4(af[s], ws + ((size_t)s * 16 + (lane & 15)) * stride + k + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint32_t bx0, bx1;
                ldmatrix_x2(bx0, bx1, xs + (size_t)(j * 8 + (lane & 7)) * stride + k + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int s = 0; s < SETS; ++s) mma16816(acc[s][j], af[s], bx0, bx1);
            }
        }
    }
    if (failed && threadIdx.x == 0) {
        if (a.error) atomicExch(a.error, 5);
        // the copies of the round that did not arrive in time may still land in this CTA's shared memory: one more
        // bounded wait for them before anything of it is given up
        bool landed = false;
        for (uint32_t spin = 0; spin < kSpinLimit && !landed; ++spin) landed = mbar_try_wait(&weights_bar, (uint32_t)round & 1u);
    }
    // (on a failure the flow goes on with what there is: the cluster's barrier below must be reached by everyone)
    if (NORM) {
        float (*sq_dst)[TOK] = a.cluster > 1 ? cluster.map_shared_rank(squares, 0) : squares;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const float s = warp_sum(sq[j]);
            if (lane == 0) sq_dst[rank][j * 8 + warp] = s;
        }
    }
    __syncthreads();   // every warp has read its operands: their space now takes the partial sums
    // partial sums of this warp: rows g and g + 8, tokens 2q and 2q + 1 of each group of 8
    {
        const int g = lane >> 2, q = lane & 3;
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                red[warp][s][g][j * 8 + 2 * q] = acc[s][j][0];
                red[warp][s][g][j * 8 + 2 * q + 1] = acc[s][j][1];
                red[warp][s][g + 8][j * 8 + 2 * q] = acc[s][j][2];
                red[warp][s][g + 8][j * 8 + 2 * q + 1] = acc[s][j][3];
            }
    }
    __syncthreads();
    // this CTA's sums over its warps, in warp order, into `across[rank]` of the first CTA
    {
        float (*dst)[SETS][16][COLS] = a.cluster > 1 ? cluster.map_shared_rank(across, 0) : across;
        for (int idx = threadIdx.x; idx < SETS * 16 * TOK; idx += kThreads) {
            const int s = idx / (16 * TOK), r = (idx / TOK) % 16, t = idx % TOK;
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
    if (failed) return;

    // 1 / rms of a token's row from the CTAs' sums of squares, in rank order
    auto inv_rms = [&](int t) {
        float s = 0.f;
        for (int c = 0; c < a.cluster; ++c) s += squares[c][t];
        return 1.0f / sqrtf(s / (float)K + a.eps);
    };

    if (a.mode == SK_QKV_ROPE) {
        const int r = threadIdx.x / TOK, t = threadIdx.x - r * TOK;
        if (r >= 8 || t >= a.T) return;
        float lo = 0.f, hi = 0.f;
        for (int c = 0; c < a.cluster; ++c) { lo += across[c][0][r][t]; hi += across[c][0][r + 8][t]; }
        if (NORM) { const float inv = inv_rms(t); lo *= inv; hi *= inv; }
        lo += pre_a;
        hi += pre_b;
        const float r0 = lo * pre_cos - hi * pre_sin, r1 = lo * pre_sin + hi * pre_cos;   // cos 1, sin 0 for v
        if (dst_lo != nullptr) {
            *dst_lo = __float2bfloat16_rn(r0);
            *dst_hi = __float2bfloat16_rn(r1);
        }
        if (packed_lo != nullptr) {
            *packed_lo = __float2bfloat16_rn(r0);
            *packed_hi = __float2bfloat16_rn(r1);
        }
        return;
    }
#pragma unroll
    for (int pass = 0; pass < (TOK * 16 + kThreads - 1) / kThreads; ++pass) {
        const int idx = threadIdx.x + pass * kThreads;
        const int r = idx / TOK, t = idx - r * TOK;
        const int n = tile * 16 + r;
        if (r >= 16 || t >= a.T || n >= a.N) continue;
        const float pre = pass == 0 ? pre_a : pre_b;
        float v = 0.f, u = 0.f;
        for (int c = 0; c < a.cluster; ++c) {
            v += across[c][0][r][t];
            if (DUAL) u += across[c][DUAL ? 1 : 0][r][t];
        }
        if (NORM) { const float inv = inv_rms(t); v *= inv; u *= inv; }
        const size_t o = (size_t)t * a.N + n;
        if (a.mode == SK_SWIGLU) v = u * activate(a.act, v);
        else v += pre;                     // the bias, or what the residual held
        if (a.mode == SK_RESIDUAL || a.out_dt == F32) ((float*)a.out)[o] = v;
        else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(v);
    }
}

template <int NT, bool NORM, bool DUAL>
void launch_one(const SkinnyArgs& a, int tiles, cudaStream_t stream) {
    constexpr int SETS = DUAL ? 2 : 1, COLS = NT * 8 + 1;
    size_t operands = (size_t)(SETS * 16 + NT * 8) * (a.round_k + 8) * sizeof(__nv_bfloat16);
    const size_t sums = (size_t)kWarps * SETS * 16 * COLS * sizeof(float);
    if (operands < sums) operands = (sums + 15) / 16 * 16;
    const size_t smem = operands + (size_t)a.cluster * SETS * 16 * COLS * sizeof(float);
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

// CTAs per tile. Clusters are not free (their CTAs must be co-scheduled and meet at a cluster
// barrier; measured on a B200, clusters of 8 cost more than they gain), and more CTAs than are
// resident at once cost a second wave; so: the smallest cluster of at most 4 whose CTAs hold
// their share of K in one round, as long as all CTAs are resident together (3 per SM).
int pick_cluster(int tiles, int K, int round_limit) {
    const int resident = 148 * 3;
    int c = 1;
    while (c < 4 && (K + c - 1) / c > round_limit && tiles * c * 2 <= resident) c *= 2;
    return c;
}

}  // namespace

bool gemm_skinny_supports(int T, int N, int K) { return T > 0 && T <= 32 && N > 0 && K > 0 && K % 8 == 0; }

int gemm_skinny_rounds(int T, int N, int K, bool gated) {
    const int nt = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
    const int weight_rows = gated ? 32 : 16;
    const int cluster = pick_cluster((N + 15) / 16, K, max_round_k(weight_rows + 8));
    const int kblocks = (K + 31) / 32, per_cta = (kblocks + cluster - 1) / cluster;
    const int limit = max_round_k(weight_rows + nt * 8);
    return (per_cta * 32 + limit - 1) / limit;
}

void gemm_skinny(const void* x, const void* norm_w, DType norm_w_dt, float eps, const void* w, int T, int N, int K,
                 int mode, const void* bias, DType bias_dt, void* out, DType out_dt, int up_offset,
                 const SkinnyRope* rope, cudaStream_t stream) {
    if (!gemm_skinny_supports(T, N, K))
        throw std::invalid_argument("gemm_skinny: T = " + std::to_string(T) + " must be at most 32 and K = " +
                                    std::to_string(K) + " a multiple of 8");
    if (((uintptr_t)x | (uintptr_t)w) & 15) throw std::invalid_argument("gemm_skinny: operands must be 16-byte aligned");
    SkinnyArgs a{};
    a.x = x; a.norm_w = norm_w; a.norm_w_dt = norm_w_dt; a.eps = eps;
    a.act = mode >> 8;          // mode: the epilogue in its low byte, the gated product's activation above it
    mode &= 0xff;
    if (a.act < 0 || a.act >= ACT_COUNT) throw std::invalid_argument("gemm_skinny: unknown activation " + std::to_string(a.act));
    a.w = (const __nv_bfloat16*)w; a.T = T; a.N = N; a.K = K; a.mode = mode;
    a.bias = bias; a.bias_dt = bias_dt; a.out = out; a.out_dt = out_dt; a.up_offset = up_offset;
    a.error = error_word();
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
        a.k_packed = rope->k_packed; a.v_packed = rope->v_packed; a.token_end = rope->token_end;
        tiles = N / 16;
    }
    {
        const int nt = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
        const int round_limit = max_round_k((mode == SK_SWIGLU ? 32 : 16) + nt * 8);
        // the cluster is chosen as for 8 tokens, so that the split of K over CTAs does not depend on T
        a.cluster = pick_cluster(tiles, K, max_round_k((mode == SK_SWIGLU ? 32 : 16) + 8));
        const int kblocks = (K + 31) / 32, per_cta = (kblocks + a.cluster - 1) / a.cluster;
        const int share = per_cta * 32;
        a.round_k = share < round_limit ? share : round_limit;
    }
    note_launch();
    if (T <= 8) launch_nt<1>(a, tiles, stream);
    else if (T <= 16) launch_nt<2>(a, tiles, stream);
    else launch_nt<4>(a, tiles, stream);
}

}  // namespace sm
