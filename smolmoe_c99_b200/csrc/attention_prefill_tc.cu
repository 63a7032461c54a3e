// Causal attention of whole prompts over their own keys for bfloat16 (prefill) on the
// 5th-generation tensor cores: the same result as attention_prefill.cu (packed sequences of
// unequal lengths, grouped heads, optional window, running softmax in float; the reference
// scans [start, pos] per query and head: src/model.c:459-491, src/kernels.c:1156-1176), for
// head sizes 64 and 128.
//
// One CTA of 128 threads per (tile of 128 queries of one sequence, head). Q, and tiles of 128
// keys and values, come into shared memory by TMA (128-byte swizzle). For every key tile:
//   S = Q K^T   tcgen05.mma 128 x 128 x head_dim, both operands K-major, S (float) in tensor memory;
//   each thread owns one query row (its lane of tensor memory): it reads the row with
//   tcgen05.ld, masks, takes the running maximum, writes P = exp2(S - max) as bfloat16 into
//   shared memory in the swizzled K-major layout an MMA operand needs;
//   PV = P V    tcgen05.mma 128 x head_dim x 128 with V as it lies in memory ([key][dim], the
//   "MN-major" operand form), into a second accumulator; the thread adds its row of PV to the
//   output it keeps in registers, rescaled when the maximum moved.
// One thread issues the copies and the MMAs. The MMAs of S for the next tile are issued right
// behind those of PV, so they run while the threads finish this tile; two CTAs share an SM
// (head size 64), so one's MMAs also run under the other's softmax.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in *error and the
// CTA leaves without writing.
#include <math_constants.h>

#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"

namespace sm {

namespace {

using namespace tc5;

constexpr int kBM = 128, kBN = 128, kThreads = 128;
constexpr int kBlockBytes = 128 * 128;      // 128 rows of 128 bytes: one swizzled block of 64 bfloat16 columns

struct PrefillTcArgs {
    __nv_bfloat16* out;       // [T, heads, HD]
    const int32_t* tiles;     // [n_tiles, 3]: packed index of the sequence's first token, its length, first query (tiles of 64)
    int heads, kv_heads, window;
    float scale_log2;         // scale * log2(e)
    int* error;
};

// Descriptor of an "MN-major" operand tile with 128-byte swizzle: rows of the reduction dimension are 128
// bytes (64 elements of the other dimension), groups of 8 rows lie `sbo` bytes apart, blocks of 64 elements
// of the other dimension `lbo` bytes apart.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;              // descriptor version
    d |= (uint64_t)2 << 61;              // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD>
__global__ void __launch_bounds__(kThreads) prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                        const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v,
                                                                        PrefillTcArgs a) {
    constexpr int DB = HD / 64;                       // blocks of 64 columns of the head dimension
    constexpr int kQBytes = DB * kBlockBytes;         // Q tile, and one K or V tile
    constexpr uint32_t kTmemCols = 256;               // S: 128 columns, PV: HD columns
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;   // late tiles (most keys) first
    const int seq_start = a.tiles[3 * tile], seq_len = a.tiles[3 * tile + 1], q0 = a.tiles[3 * tile + 2];
    if (q0 % kBM) return;                             // the second half of a tile of 128 queries
    const int kvh = h / (a.heads / a.kv_heads);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;                              // [DB][128 queries][128 B]
    uint8_t* k_s = q_s + kQBytes;                     // 2 x [DB][128 keys][128 B]
    uint8_t* v_s = k_s + 2 * kQBytes;                 // [DB][128 keys][128 B]
    uint8_t* p_s = v_s + kQBytes;                     // [2][128 queries][128 B]: keys 0-63 and 64-127 of the tile
    uint64_t* bars = (uint64_t*)(p_s + 2 * kBlockBytes);
    uint64_t* q_bar = bars;
    uint64_t* k_bar = bars + 1;                       // [2]
    uint64_t* v_bar = bars + 3;
    uint64_t* s_bar = bars + 4;
    uint64_t* pv_bar = bars + 5;
    uint32_t* tmem_slot = (uint32_t*)(bars + 6);
    volatile int* failed = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int row = threadIdx.x;                      // this thread's query row of the tile, and its lane of tensor memory
    const int qpos = q0 + row;

    if (threadIdx.x == 0) {
        mbar_init(q_bar, 1);
        mbar_init(&k_bar[0], 1);
        mbar_init(&k_bar[1], 1);
        mbar_init(v_bar, 1);
        mbar_init(s_bar, 1);
        mbar_init(pv_bar, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);   // (not the warp whose first thread has just branched off)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + 128;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;

    // key tiles this query tile sees
    const int q_last = min(q0 + kBM, seq_len) - 1;
    const int first_key = a.window > 0 ? max(0, q0 - a.window + 1) : 0;
    const int kt0 = first_key / kBN;
    const int n_kt = q_last / kBN - kt0 + 1;

    const uint32_t idesc_s = instr_desc(kBM, kBN);
    const uint32_t idesc_pv = instr_desc(kBM, HD) | (1u << 16);   // B (= V) is MN-major

    auto load_k = [&](int t) {      // key tile t (counted from kt0) into buffer t & 1
        uint8_t* dst = k_s + (size_t)(t & 1) * kQBytes;
        mbar_expect_tx(&k_bar[t & 1], (uint32_t)kQBytes);
#pragma unroll
        for (int b = 0; b < DB; ++b)
            tma_load_2d(dst + b * kBlockBytes, &map_k, kvh * HD + b * 64, seq_start + (kt0 + t) * kBN, &k_bar[t & 1]);
    };
    auto load_v = [&](int t) {
        mbar_expect_tx(v_bar, (uint32_t)kQBytes);
#pragma unroll
        for (int b = 0; b < DB; ++b)
            tma_load_2d(v_s + b * kBlockBytes, &map_v, kvh * HD + b * 64, seq_start + (kt0 + t) * kBN, v_bar);
    };
    auto issue_s = [&](int t) {     // S = Q K^T for key tile t
        const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s + (size_t)(t & 1) * kQBytes);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t off = (uint32_t)(ks / 4) * kBlockBytes + (uint32_t)(ks % 4) * 32;
            umma_bf16(tmem_s, smem_desc(qa + off), smem_desc(ka + off), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(s_bar);
    };
    auto issue_pv = [&]() {         // PV = P V for the tile whose P lies in shared memory
        const uint32_t pa = smem_u32(p_s), va = smem_u32(v_s);
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
            const uint32_t p_off = (uint32_t)(ks / 4) * kBlockBytes + (uint32_t)(ks % 4) * 32;
            const uint32_t v_off = (uint32_t)ks * 16 * 128;          // 16 keys of 128 bytes
            umma_bf16(tmem_pv, smem_desc(pa + p_off), smem_desc_mn(va + v_off, kBlockBytes, 1024), idesc_pv, ks > 0 ? 1u : 0u);
        }
        umma_commit(pv_bar);
    };
    auto fail = [&](int code) {
        *failed = 1;
        if (a.error) atomicExch(a.error, code);
    };

    if (threadIdx.x == 0) {
        mbar_expect_tx(q_bar, (uint32_t)kQBytes);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_2d(q_s + b * kBlockBytes, &map_q, h * HD + b * 64, seq_start + q0, q_bar);
        load_k(0);
        load_v(0);
        if (n_kt > 1) load_k(1);
        if (mbar_wait(q_bar, 0) && mbar_wait(&k_bar[0], 0)) {
            tc_fence_after();
            issue_s(0);
        } else {
            fail(11);
        }
    }

    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    float m = -CUDART_INF_F, l = 0.f;

    for (int it = 0; it < n_kt; ++it) {
        const int n0 = (kt0 + it) * kBN;
        if (!mbar_wait(s_bar, (uint32_t)it & 1u)) fail(12);
        tc_fence_after();
        // every key of the tile visible to every query of the tile: no mask needed
        const bool full = n0 + kBN - 1 <= q0 && n0 + kBN - 1 < seq_len && (a.window <= 0 || n0 > q0 + kBM - 1 - a.window);
        // otherwise this row sees the keys n0 + j with vis_lo <= j <= vis_hi
        const int vis_hi = min(qpos, seq_len - 1) - n0;
        const int vis_lo = a.window > 0 ? qpos - a.window + 1 - n0 : -(1 << 30);
        // The row's scores are read from tensor memory SW columns at a time: all 128 at once when the registers
        // allow it (head size 64), else twice 64, in two passes (maximum first, then the exponentials).
        constexpr int SW = HD == 64 ? 128 : 64, NS = kBN / SW;
        float sv[SW];
        auto read_scores = [&](int part) {
            if constexpr (SW == 128) tmem_ld128(tmem_s + lane_base, sv);
            else tmem_ld64(tmem_s + lane_base + (uint32_t)(part * SW), sv);
            if (!full) {
#pragma unroll
                for (int j = 0; j < SW; ++j)
                    if (part * SW + j > vis_hi || part * SW + j < vis_lo) sv[j] = -CUDART_INF_F;
            }
        };
        // maximum of the raw scores; the scale is positive, so it can be applied to the maximum
        float raw = -CUDART_INF_F;
#pragma unroll 1
        for (int part = 0; part < NS; ++part) {
            read_scores(part);
#pragma unroll
            for (int j = 0; j < SW; ++j) raw = fmaxf(raw, sv[j]);
        }
        const float mx = fmaxf(m, raw * a.scale_log2);
        // a row that has seen no key yet keeps m = -inf; 0 as its reference avoids inf - inf
        const float ref = mx == -CUDART_INF_F ? 0.f : mx;
        const float corr = ex2_approx(m - ref);
        m = mx;
        // P = 2^(S * scale - max) as bfloat16 into shared memory, and its sum
        float sum = 0.f;
#pragma unroll 1
        for (int part = 0; part < NS; ++part) {
            if (NS > 1) read_scores(part);
#pragma unroll
            for (int c = 0; c < SW / 8; ++c) {       // pieces of 8 keys (16 bytes)
                uint32_t pk[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p0 = ex2_approx(fmaf(sv[c * 8 + 2 * e], a.scale_log2, -ref));
                    const float p1 = ex2_approx(fmaf(sv[c * 8 + 2 * e + 1], a.scale_log2, -ref));
                    sum += p0 + p1;
                    pk[e] = pack_bf16(p0, p1);
                }
                // the piece's place within its block of 64 keys is swizzled with the row
                const int piece = part * (SW / 8) + c;
                uint8_t* prow = p_s + (size_t)(piece / 8) * kBlockBytes + (size_t)row * 128;
                *reinterpret_cast<uint4*>(prow + (((piece % 8) ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        }
        l = l * corr + sum;
        // P is written: make it visible to the tensor core's reads, then everyone meets
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_before();
        if (__syncthreads_or(*failed)) break;   // (evaluated by every thread as it arrives: the same answer for all)
        if (threadIdx.x == 0) {
            tc_fence_after();
            if (mbar_wait(v_bar, (uint32_t)it & 1u)) {
                tc_fence_after();
                issue_pv();
                if (it + 1 < n_kt) {
                    if (mbar_wait(&k_bar[(it + 1) & 1], (uint32_t)((it + 1) >> 1) & 1u)) {
                        tc_fence_after();
                        issue_s(it + 1);
                    } else {
                        fail(13);
                    }
                }
                if (it + 2 < n_kt) load_k(it + 2);   // S of this tile is done: its key buffer is free
            } else {
                fail(14);
            }
        }
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] *= corr;
        if (!mbar_wait(pv_bar, (uint32_t)it & 1u)) fail(15);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            float pv[32];
            tmem_ld32(tmem_pv + lane_base + (uint32_t)(c * 32), pv);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[c * 32 + j] += pv[j];
        }
        if (threadIdx.x == 0 && it + 1 < n_kt && !*failed) load_v(it + 1);   // PV is done: the value buffer is free
    }

    if (!*failed && qpos < seq_len) {
        const float inv = 1.0f / l;
        __nv_bfloat16* orow = a.out + ((size_t)(seq_start + qpos) * a.heads + h) * HD;
#pragma unroll
        for (int i = 0; i < HD; i += 8)
            *reinterpret_cast<uint4*>(orow + i) =
                make_uint4(pack_bf16(o[i] * inv, o[i + 1] * inv), pack_bf16(o[i + 2] * inv, o[i + 3] * inv),
                           pack_bf16(o[i + 4] * inv, o[i + 5] * inv), pack_bf16(o[i + 6] * inv, o[i + 7] * inv));
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    if (!fn) throw std::runtime_error("attention_prefill_tc: the driver does not provide cuTensorMapEncodeTiled");
    return fn;
}

// A [T, width] row-major bfloat16 matrix, boxes of 128 rows x 64 elements, 128-byte swizzle; rows and columns
// outside the matrix read as zero.
CUtensorMap make_map(const void* base, int T, int width) {
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)T};
    cuuint64_t strides[1] = {(cuuint64_t)width * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        throw std::runtime_error("attention_prefill_tc: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r) +
                                 " for a " + std::to_string(T) + " x " + std::to_string(width) + " matrix");
    return map;
}

template <int HD>
void launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillTcArgs& a, int n_tiles,
            cudaStream_t stream) {
    constexpr int DB = HD / 64;
    const size_t smem = 1024 + (size_t)(4 * DB + 2) * kBlockBytes + 64;   // alignment, Q + 2 K + V, P, barriers
    auto kernel = prefill_attention_tc_kernel<HD>;
    static bool prepared = false;
    if (!prepared) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) throw std::runtime_error(std::string("attention_prefill_tc: ") + cudaGetErrorString(e));
        prepared = true;
    }
    kernel<<<dim3(n_tiles, a.heads), kThreads, smem, stream>>>(mq, mk, mv, a);
}

}  // namespace

bool attention_prefill_tc_supports(int heads, int kv_heads, int head_dim) {
    return (head_dim == 64 || head_dim == 128) && kv_heads > 0 && heads % kv_heads == 0 && heads <= 65535;
}

void attention_prefill_tc(const void* q, const void* k, const void* v, void* out, const int32_t* tiles, int n_tiles, int T,
                          int heads, int kv_heads, int head_dim, float scale, int window, int* error,
                          cudaStream_t stream) {
    if (n_tiles <= 0) return;
    if (!attention_prefill_tc_supports(heads, kv_heads, head_dim))
        throw std::invalid_argument("attention_prefill_tc: head_dim " + std::to_string(head_dim) +
                                    " is not 64 or 128 (the mma.sync kernel takes multiples of 16 up to 128)");
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
        throw std::invalid_argument("attention_prefill_tc: operands must be 16-byte aligned");
    const CUtensorMap mq = make_map(q, T, heads * head_dim);
    const CUtensorMap mk = make_map(k, T, kv_heads * head_dim);
    const CUtensorMap mv = make_map(v, T, kv_heads * head_dim);
    PrefillTcArgs a{(__nv_bfloat16*)out, tiles, heads, kv_heads, window, scale * 1.4426950408889634f, error};
    note_launch();
    if (head_dim == 64) launch<64>(mq, mk, mv, a, n_tiles, stream);
    else launch<128>(mq, mk, mv, a, n_tiles, stream);
}

}  // namespace sm
