// out[t, n] = sum_k x[t, k] * w[n, k] for bfloat16 operands on the 5th-generation tensor
// cores: tcgen05.mma with both operands staged in shared memory by TMA (128-byte swizzle)
// and the float accumulator in tensor memory.
//
// The weight rows are the M side of the instruction (128 output features a tile, one per
// TMEM lane) and the tokens are the N side (16..256 a tile), so the same kernel serves
// prefill (many tokens) and decode (a handful): with few tokens the instruction shrinks
// instead of wasting a 128-row tile on them. One CTA computes one 128 x TN tile over a range
// of K; when K is split over several CTAs the partial sums go to a workspace and a second
// kernel adds them in split order and applies the epilogue.
//
// Roles (192 threads): warp 0 issues the TMA loads, warp 1 allocates tensor memory and
// issues the MMAs, warps 2-5 read the accumulator back (each its own quarter of the lanes)
// and write the result. Epilogues: store (+bias), add into a float residual, or
// act(gate) * up from two accumulators.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in *error and
// the CTA drains and leaves without writing.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"

namespace sm {

namespace {

constexpr int kTileM = 128;          // output features per CTA
constexpr int kBlockK = 64;          // bf16 elements per 128-byte swizzled row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 24;

enum Epilogue : int { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3 };

struct GemmParams {
    int T, N, K;              // tokens, output features, reduction
    int tile_n;               // tokens per CTA (multiple of 16, <= 256)
    int stages;
    int splits;               // CTAs along K
    int kblocks_per_split;
    int epilogue;
    int dual;                 // two weight tiles (gate rows n, up rows up_offset + n) per stage
    int up_offset;
    const void* bias;         // [N] or null
    int bias_dt;
    void* out;                // [T, N]
    int out_dt;
    float* workspace;         // [splits, T, N] for EPI_PARTIAL
    int* error;
};

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

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
// Bounded wait: false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_in_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_in_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled in
// groups of 8 rows (1024 bytes): start address, stride between row groups, descriptor
// version 1, layout 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;              // leading byte offset (not used by swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;    // stride byte offset
    d |= (uint64_t)1 << 46;              // descriptor version
    d |= (uint64_t)2 << 61;              // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D float, A and B bfloat16, both K-major, M x N.
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of the tiles is what the swizzle pattern assumes
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int a_bytes = kTileM * kBlockK * 2 * (p.dual ? 2 : 1);
    const int b_bytes = p.tile_n * kBlockK * 2;
    const int stage_bytes = a_bytes + b_bytes;
    uint64_t* full_bar = (uint64_t*)(smem + (size_t)p.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + p.stages;
    uint64_t* tmem_full_bar = empty_bar + p.stages;
    uint32_t* tmem_slot = (uint32_t*)(tmem_full_bar + 1);
    int* failed = (int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kTileM, t0 = blockIdx.y * p.tile_n, split = blockIdx.z;
    const int kb_total = (p.K + kBlockK - 1) / kBlockK;
    const int kb_begin = split * p.kblocks_per_split;
    const int kb_end = min(kb_total, kb_begin + p.kblocks_per_split);
    const int n_kb = kb_end - kb_begin;   // >= 1 by construction of the grid
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < p.tile_n * (p.dual ? 2 : 1)) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(tmem_full_bar, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < n_kb; ++i) {
                int s = i % p.stages;
                uint32_t phase = (uint32_t)(i / p.stages) & 1u;
                if (!mbar_wait(&empty_bar[s], phase ^ 1u)) { *failed = 1; atomicExch(p.error, 1); break; }
                uint8_t* a = smem + (size_t)s * stage_bytes;
                mbar_expect_tx(&full_bar[s], (uint32_t)stage_bytes);
                int k = (kb_begin + i) * kBlockK;
                tma_load_2d(a, &map_w, k, n0, &full_bar[s]);
                if (p.dual) tma_load_2d(a + kTileM * kBlockK * 2, &map_w, k, p.up_offset + n0, &full_bar[s]);
                tma_load_2d(a + a_bytes, &map_x, k, t0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(kTileM, p.tile_n);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                int s = i % p.stages;
                uint32_t phase = (uint32_t)(i / p.stages) & 1u;
                if (!mbar_wait(&full_bar[s], phase)) { *failed = 1; atomicExch(p.error, 2); ok = false; break; }
                tc_fence_after();
                uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes);
                uint32_t b_addr = a_addr + a_bytes;
                uint64_t da = smem_desc(a_addr), db = smem_desc(b_addr);
                uint64_t du = smem_desc(a_addr + kTileM * kBlockK * 2);
#pragma unroll
                for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                    uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    uint64_t step = (uint64_t)((k * kUmmaK * 2) >> 4);   // 32 bytes a step inside the swizzled row
                    umma_bf16(tmem_base, da + step, db + step, idesc, acc);
                    if (p.dual) umma_bf16(tmem_base + (uint32_t)p.tile_n, du + step, db + step, idesc, acc);
                }
                umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
            }
            umma_commit(tmem_full_bar);        // the accumulator is complete once all MMAs are done
        }
    } else {
        // epilogue warps 2..5: TMEM lanes of quarter (warp % 4)
        const int quarter = warp & 3;
        const int n = n0 + quarter * 32 + lane;
        bool ok = mbar_wait(tmem_full_bar, 0);
        if (!ok && lane == 0) { *failed = 1; atomicExch(p.error, 3); }
        ok = ok && (*(volatile int*)failed == 0);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (ok) {
            const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
            float bias_v = 0.f;
            if (p.bias && n < p.N)
                bias_v = p.bias_dt == F32 ? ((const float*)p.bias)[n] : __bfloat162float(((const __nv_bfloat16*)p.bias)[n]);
            for (int c0 = 0; c0 < p.tile_n; c0 += 16) {
                if (t0 + c0 >= p.T) break;   // the same for the whole warp
                float g[16], u[16];
                tmem_ld16(lane_base + (uint32_t)c0, g);
                if (p.dual) tmem_ld16(lane_base + (uint32_t)(p.tile_n + c0), u);
                if (n >= p.N) continue;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    int t = t0 + c0 + j;
                    if (t >= p.T) break;
                    size_t o = (size_t)t * p.N + n;
                    float v = g[j];
                    if (p.epilogue == EPI_PARTIAL) {
                        p.workspace[((size_t)split * p.T + t) * p.N + n] = v;
                        if (p.dual) p.workspace[(((size_t)p.splits + split) * p.T + t) * p.N + n] = u[j];
                        continue;
                    }
                    if (p.epilogue == EPI_SWIGLU) v = u[j] * (v / (1.0f + expf(-v)));
                    else v += bias_v;
                    if (p.epilogue == EPI_ACCUM) {
                        ((float*)p.out)[o] += v;
                    } else if (p.out_dt == F32) {
                        ((float*)p.out)[o] = v;
                    } else {
                        ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// Adds the splits in order and applies the epilogue. One thread per output element.
__global__ void splitk_reduce_kernel(GemmParams p) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)p.T * p.N;
    if (i >= total) return;
    int n = (int)(i % p.N);
    float g = 0.f, u = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        g += p.workspace[(size_t)s * total + i];
        if (p.dual) u += p.workspace[((size_t)p.splits + s) * total + i];
    }
    float v = g;
    if (p.epilogue == EPI_SWIGLU) v = u * (g / (1.0f + expf(-g)));
    else if (p.bias) v += p.bias_dt == F32 ? ((const float*)p.bias)[n] : __bfloat162float(((const __nv_bfloat16*)p.bias)[n]);
    if (p.epilogue == EPI_ACCUM) ((float*)p.out)[i] += v;
    else if (p.out_dt == F32) ((float*)p.out)[i] = v;
    else ((__nv_bfloat16*)p.out)[i] = __float2bfloat16_rn(v);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    });
    if (!fn) throw std::runtime_error("gemm_tc: the driver does not provide cuTensorMapEncodeTiled");
    return fn;
}

// A [rows, K] row-major bfloat16 matrix, boxes of box_rows x 64 elements, 128-byte swizzle.
// Rows and columns outside the matrix read as zero.
CUtensorMap make_map(const void* base, int rows, int K, int box_rows) {
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        throw std::runtime_error("gemm_tc: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r) +
                                 " for a " + std::to_string(rows) + " x " + std::to_string(K) + " matrix");
    return map;
}

int device_sm_count() {
    static int count = 0;
    if (!count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
        if (count <= 0) count = 148;
    }
    return count;
}

}  // namespace

bool gemm_tc_supports(int T, int N, int K) { return T > 0 && N > 0 && K > 0 && K % 8 == 0; }

void gemm_tc_plan(int T, int N, int K, bool dual, int* tile_n, int* splits) {
    int sms = device_sm_count();
    int tiles_m = (N + kTileM - 1) / kTileM;
    int t16 = ((T + 15) / 16) * 16;
    int max_tile = dual ? 128 : 256;
    int tn = 16;
    // the largest token tile that still fills the machine, else the smallest that covers T
    for (int cand = max_tile; cand >= 16; cand >>= 1) {
        if (cand > t16 && cand > 16) continue;
        int ctas = tiles_m * ((T + cand - 1) / cand);
        tn = cand;
        if (ctas >= sms) break;
    }
    int ctas = tiles_m * ((T + tn - 1) / tn);
    int kb = (K + kBlockK - 1) / kBlockK;
    int sp = 1;
    if (ctas < sms && kb >= 4) {
        sp = (2 * sms + ctas - 1) / ctas;
        if (sp > kb / 2) sp = kb / 2;
        if (sp > 16) sp = 16;
        if (sp < 1) sp = 1;
    }
    // no empty split: every CTA along K gets at least one block
    int per = (kb + sp - 1) / sp;
    sp = (kb + per - 1) / per;
    *tile_n = tn;
    *splits = sp;
}

size_t gemm_tc_workspace_bytes(int T, int N, int K, bool dual) {
    int tn, sp;
    gemm_tc_plan(T, N, K, dual, &tn, &sp);
    return sp > 1 ? (size_t)sp * (dual ? 2 : 1) * T * N * sizeof(float) : 0;
}

void gemm_tc(const void* x, const void* w, const void* bias, DType bias_dt, void* out, DType out_dt, int T, int N,
             int K, int mode, int up_offset, float* workspace, int* error, cudaStream_t stream) {
    if (!gemm_tc_supports(T, N, K))
        throw std::invalid_argument("gemm_tc: K = " + std::to_string(K) + " must be a positive multiple of 8 (TMA rows start on 16 bytes)");
    if (((uintptr_t)x | (uintptr_t)w) & 15) throw std::invalid_argument("gemm_tc: operands must be 16-byte aligned");
    const bool dual = mode == EPI_SWIGLU;
    GemmParams p{};
    p.T = T; p.N = N; p.K = K;
    gemm_tc_plan(T, N, K, dual, &p.tile_n, &p.splits);
    int kb = (K + kBlockK - 1) / kBlockK;
    p.kblocks_per_split = (kb + p.splits - 1) / p.splits;
    p.dual = dual ? 1 : 0;
    p.up_offset = up_offset;
    p.bias = bias; p.bias_dt = bias_dt;
    p.out = out; p.out_dt = out_dt;
    p.workspace = workspace;
    p.error = error;
    const int final_mode = mode;
    p.epilogue = p.splits > 1 ? EPI_PARTIAL : final_mode;
    if (p.splits > 1 && !workspace) throw std::invalid_argument("gemm_tc: this shape splits K and needs a workspace");
    int stage_bytes = kTileM * kBlockK * 2 * (dual ? 2 : 1) + p.tile_n * kBlockK * 2;
    int budget = p.tile_n <= 64 ? 100 * 1024 : 200 * 1024;   // small tiles: two CTAs share an SM
    p.stages = budget / stage_bytes;
    if (p.stages > 8) p.stages = 8;
    if (p.stages < 2) p.stages = 2;
    size_t smem = (size_t)p.stages * stage_bytes + 1024 /*alignment*/ + (2 * p.stages + 1) * 8 + 16;
    CUtensorMap map_w = make_map(w, dual ? up_offset + N : N, K, kTileM);
    CUtensorMap map_x = make_map(x, T, K, p.tile_n);
    static std::once_flag attr_once;
    std::call_once(attr_once, [] {
        cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    });
    dim3 grid((N + kTileM - 1) / kTileM, (T + p.tile_n - 1) / p.tile_n, p.splits);
    gemm_tc_kernel<<<grid, kThreads, smem, stream>>>(map_w, map_x, p);
    note_launch(p.splits > 1 ? 2 : 1);
    if (p.splits > 1) {
        p.epilogue = final_mode;
        size_t total = (size_t)T * N;
        splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(p);
    }
}

}  // namespace sm
