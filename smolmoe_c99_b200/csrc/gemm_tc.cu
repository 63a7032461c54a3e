// out[t, n] = sum_k x[t, k] * w[n, k] for bfloat16 operands on the 5th-generation tensor
// cores: tcgen05.mma with both operands staged in shared memory by TMA (128-byte swizzle)
// and the float accumulator in tensor memory.
//
// The weight rows are the M side of the instruction (128 output features a tile, one per
// TMEM lane) and the tokens are the N side (16..256 a tile), so the same kernel serves
// prefill (many tokens) and decode batches too large for the weight-streaming kernel: with
// few tokens the instruction shrinks instead of wasting a 128-row tile on them.
//
// The kernel is persistent: one CTA per SM takes work units (a 128 x TN tile over a range of
// K) round-robin. Roles (192 threads): warp 0 issues the TMA loads into a ring of stages,
// warp 1 allocates tensor memory and issues the MMAs, warps 2-5 are the epilogue (each its
// own quarter of the TMEM lanes). Tensor memory holds TWO accumulators, so the MMAs of the
// next unit run while the epilogue drains the previous one. The epilogue reads 32 tokens at a
// time with tcgen05.ld, applies bias / SwiGLU, transposes through shared memory and hands the
// chunk to TMA: a bulk tensor store, or a bulk tensor float add for "+= into the residual"
// (TMA drops what lies outside the matrix, so ragged edges need no code). Outputs whose rows
// TMA cannot address, and the partial sums of a split K, are written by the threads directly;
// split partial sums go to a workspace and a second kernel adds them in split order.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in *error and
// the CTA leaves without writing, after it has waited (bounded again) for the copies it has asked
// for and the MMAs it has issued (drain.cuh).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "common.cuh"
#include "drain.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "tcgen05.cuh"

namespace sm {

namespace {

constexpr int kTileM = 128;          // output features per CTA
constexpr int kBlockK = 64;          // bf16 elements per 128-byte swizzled row
constexpr int kAtoms = 2;            // swizzled blocks of K per pipeline stage: a stage holds kStageK = 128 elements of K,
constexpr int kStageK = kAtoms * kBlockK;   // so that the issuing thread's wait and commit are paid once per 8 MMAs
constexpr int kUmmaK = 16;
constexpr int kBoxRows = 64;         // rows of one TMA box (a token tile below 64 rows is one box of its own size)
constexpr int kThreads = 192;

enum Epilogue : int { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3, EPI_QKV_ROPE = 4 };

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
    int tiles_m, tiles_t;     // tile grid: 128 features x tile_n tokens
    int units;                // tiles_m * tiles_t * splits work units, shared out round-robin
    int tma_out;              // the epilogue leaves through shared memory and TMA (store or add)
    int final_epilogue;       // what the epilogue is once the splits are added up
    int cluster_reduce;       // small kernel: the CTAs along K are one cluster and add their sums up among themselves
    SkinnyRope rope;          // EPI_QKV_ROPE: where q goes and where the cache is (out is unused)
    int act;                  // the gated product's activation (Activation in common.cuh)
    int halves;               // small kernel, gated product: a tile is 64 gate rows and their 64 up rows in ONE accumulator
                              // (dual = 0); gate and up meet where the splits are added up
};

using namespace tc5;   // the PTX wrappers (tcgen05.cuh)

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

constexpr int kChunk = 32;                                  // tokens per epilogue chunk
constexpr int kStagingBytes = kChunk * kTileM * 4;          // one staged chunk (float)

// Which tile and K range a work unit is: units that run side by side share the token tile.
// What lane `lane` of the loading warp brings of every stage: the weight tile (and the second one of a gated
// product) goes as 128 / kBoxRows boxes, the token tile as ceil(tile_n / kBoxRows) boxes, one box a lane. A box is
// kBoxRows rows of 128 bytes: a multiple of the 1,024-byte swizzle atom, so boxes side by side are the same bytes as
// one large box.
// up * gate / (1 + e^-gate) with the hardware's exponential and reciprocal (a few ulp of float; the result is
// stored as bfloat16). The epilogue's four warps have a scheduler each, so every instruction saved is time.
__device__ __forceinline__ float gated(int act, float gate, float up) { return up * activate_fast(act, gate); }

// A stage lies in shared memory as [weight tile][block of K][128 rows], [second weight tile ...], then
// [block of K][tile_n token rows], every row 128 bytes.
struct StageBox {
    bool active, from_x;    // this lane loads something; from the token matrix (else from the weights)
    int offset;             // bytes from the stage's start
    int row;                // first row, relative to the tile's first row (for the second weight tile: + up_offset)
    int k;                  // first element of K, relative to the stage's
};
__device__ __forceinline__ StageBox stage_box(int lane, int a_bytes, const GemmParams& p) {
    constexpr int kPerTile = kTileM / kBoxRows;
    constexpr int kBoxBytes = kBoxRows * kBlockK * 2;
    const int w_boxes = kPerTile * kAtoms * (p.dual ? 2 : 1);
    const int x_parts = (p.tile_n + kBoxRows - 1) / kBoxRows;
    StageBox b{false, false, 0, 0, 0};
    if (lane < w_boxes) {
        const int part = lane % kPerTile, atom = (lane / kPerTile) % kAtoms, tile = lane / (kPerTile * kAtoms);
        b.active = true;
        b.offset = lane * kBoxBytes;
        b.row = p.halves ? (part ? p.up_offset : 0) : (tile ? p.up_offset : 0) + part * kBoxRows;
        b.k = atom * kBlockK;
    } else if (lane < w_boxes + x_parts * kAtoms) {
        const int idx = lane - w_boxes, atom = idx / x_parts, part = idx - atom * x_parts;
        b.active = b.from_x = true;
        b.offset = a_bytes + (atom * p.tile_n + part * kBoxRows) * kBlockK * 2;
        b.row = part * kBoxRows;
        b.k = atom * kBlockK;
    }
    return b;
}

struct Unit {
    int n0, t0, kb_begin, kb_end, split;
};
__device__ __forceinline__ Unit unit_of(const GemmParams& p, int u) {
    const int tm = u % p.tiles_m, rest = u / p.tiles_m, tt = rest % p.tiles_t, split = rest / p.tiles_t;
    const int kb_total = (p.K + kStageK - 1) / kStageK;
    Unit r;
    r.n0 = tm * kTileM;
    r.t0 = tt * p.tile_n;
    r.split = split;
    r.kb_begin = split * p.kblocks_per_split;
    r.kb_end = min(kb_total, r.kb_begin + p.kblocks_per_split);
    return r;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_out, GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of the tiles is what the swizzle pattern assumes
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int a_bytes = kTileM * kStageK * 2 * (p.dual ? 2 : 1);
    const int b_bytes = p.tile_n * kStageK * 2;
    const int stage_bytes = a_bytes + b_bytes;
    uint8_t* staging = smem + (size_t)p.stages * stage_bytes;                 // 2 x kStagingBytes
    uint64_t* full_bar = (uint64_t*)(staging + 2 * kStagingBytes);
    uint64_t* empty_bar = full_bar + p.stages;
    uint64_t* tfull_bar = empty_bar + p.stages;       // [2] accumulator complete
    uint64_t* tempty_bar = tfull_bar + 2;             // [2] accumulator drained
    uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
    volatile int* failed = (volatile int*)(tmem_slot + 1);
    // for the way out after a failure (drain.cuh): a barrier for a commit behind the last MMA, the stage fills asked for and
    // waited for, whether any MMA was issued (in the dynamic allocation: a static one would lower its limit)
    uint64_t& drain_bar = *(uint64_t*)(tmem_slot + 2);
    long long& fills_issued = *(long long*)(tmem_slot + 4);
    long long& fills_consumed = *(long long*)(tmem_slot + 6);
    int& mmas_issued = *(int*)(tmem_slot + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    const int buf_cols = p.tile_n * (p.dual ? 2 : 1);
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * buf_cols) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4); }
        mbar_init(&drain_bar, 1);
        *failed = 0;
        fills_issued = fills_consumed = 0;
        mmas_issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // The whole warp runs the loop; a stage's tiles are loaded as boxes of kBoxRows rows, one box a lane.
        // (One thread's TMA copies are taken one after another, ~0.35 us each whatever their size: measured on a
        // B200 with bulk copies from L2, a thread moves 16 KB copies at 6.5 TB/s over 148 SMs, two lanes at 12,
        // four at 18. With one issuing thread this kernel sat at 5.4 TB/s of operand traffic.)
        // (The loops of this warp and of the issuing thread below are kept free of divisions and of anything else
        // that can be counted up: a thread alone on its scheduler waits out the latency of every instruction, and at
        // ~1,000 cycles a block of K these two loops, not memory or the tensor core, bounded the kernel.)
        const StageBox box = stage_box(lane, a_bytes, p);
        // The weights do not depend on the kernel before this one: the weight tiles of the first unit's first
        // stages are asked for before the wait for it, their token tiles after.
        int early = 0;
        {
            const Unit w = unit_of(p, blockIdx.x);   // the grid is never larger than the number of units
            early = min(p.stages, w.kb_end - w.kb_begin);
            for (int i = 0; i < early; ++i) {
                if (lane == 0) mbar_expect_tx(&full_bar[i], (uint32_t)stage_bytes);
                __syncwarp();
                if (box.active && !box.from_x)
                    tma_load_2d(smem + (size_t)i * stage_bytes + box.offset, &map_w, (w.kb_begin + i) * kStageK + box.k, w.n0 + box.row, &full_bar[i]);
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                if (box.active && box.from_x)
                    tma_load_2d(smem + (size_t)i * stage_bytes + box.offset, &map_x, (w.kb_begin + i) * kStageK + box.k, w.t0 + box.row, &full_bar[i]);
        }
        int s = early == p.stages ? 0 : early;
        uint32_t phase = early == p.stages ? 1u : 0u;
        long long issued = early;
        bool ok = true;
        for (int u = blockIdx.x; u < p.units && ok && !*failed; u += gridDim.x) {
            const Unit w = unit_of(p, u);
            const int row = box.from_x ? w.t0 + box.row : w.n0 + box.row;
            for (int kb = w.kb_begin + (u == (int)blockIdx.x ? early : 0); kb < w.kb_end; ++kb) {
                ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[s], phase ^ 1u));
                if (!ok) {
                    if (lane == 0) { *failed = 1; atomicExch(p.error, 1); }
                    break;
                }
                if (lane == 0) mbar_expect_tx(&full_bar[s], (uint32_t)stage_bytes);
                __syncwarp();
                if (box.active)
                    tma_load_2d(smem + (size_t)s * stage_bytes + box.offset, box.from_x ? &map_x : &map_w, kb * kStageK + box.k, row, &full_bar[s]);
                ++issued;
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
        }
        if (lane == 0) fills_issued = issued;
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(kTileM, p.tile_n);
            // descriptors differ in the start address only (bits 0-13, in units of 16 bytes): one per stage's first
            // tile is kept running, the others are a constant away
            const uint64_t desc_first = smem_desc(smem_u32(smem));
            const uint64_t stage_step = (uint64_t)(stage_bytes >> 4), b_off = (uint64_t)(a_bytes >> 4);
            const uint64_t up_off = (uint64_t)((kTileM * kStageK * 2) >> 4);
            // a step of 16 elements of K: 32 bytes on inside its swizzled block, the blocks a tile's rows apart
            const uint64_t a_atom = (uint64_t)((kTileM * kBlockK * 2) >> 4), b_atom = (uint64_t)((p.tile_n * kBlockK * 2) >> 4);
            uint64_t da = desc_first;
            int s = 0;
            uint32_t phase = 0;
            int i = 0;
            long long consumed = 0;
            for (int u = blockIdx.x; u < p.units && !*failed; u += gridDim.x, ++i) {
                const Unit w = unit_of(p, u);
                const int b = i & 1;
                // the epilogue has drained this accumulator (its first use is free)
                if (!mbar_wait(&tempty_bar[b], (((uint32_t)i >> 1) & 1u) ^ 1u)) { *failed = 1; atomicExch(p.error, 4); break; }
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(b * buf_cols);
                const uint32_t d_up = d + (uint32_t)p.tile_n;
                uint32_t acc = 0;
                for (int kb = w.kb_begin; kb < w.kb_end; ++kb) {
                    if (!mbar_wait(&full_bar[s], phase)) { *failed = 1; atomicExch(p.error, 2); break; }
                    ++consumed;
                    tc_fence_after();
                    const uint64_t db = da + b_off, du = da + up_off;
#pragma unroll
                    for (int k = 0; k < kStageK / kUmmaK; ++k) {
                        const uint64_t sub = (uint64_t)(((k % (kBlockK / kUmmaK)) * kUmmaK * 2) >> 4);
                        const uint64_t a_step = (k / (kBlockK / kUmmaK)) * a_atom + sub, b_step = (k / (kBlockK / kUmmaK)) * b_atom + sub;
                        umma_bf16(d, da + a_step, db + b_step, idesc, acc);
                        if (p.dual) umma_bf16(d_up, du + a_step, db + b_step, idesc, acc);
                        acc = 1;
                    }
                    umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
                    da += stage_step;
                    if (++s == p.stages) { s = 0; phase ^= 1u; da = desc_first; }
                }
                umma_commit(&tfull_bar[b]);        // the accumulator is complete once all MMAs are done
            }
            fills_consumed = consumed;
            mmas_issued = consumed > 0;
        }
    } else {
        // epilogue warps 2..5: TMEM lanes of quarter (warp % 4); one output feature per thread
        const int quarter = warp & 3;
        const bool issuer = warp == 2 && lane == 0;
        int i = 0;
        uint32_t chunk_count = 0;
        pdl_wait();   // the output (read for "+=") and everything written below come after the kernel before
        for (int u = blockIdx.x; u < p.units; u += gridDim.x, ++i) {
            const Unit w = unit_of(p, u);
            const int b = i & 1;
            bool ok = mbar_wait(&tfull_bar[b], ((uint32_t)i >> 1) & 1u);
            if (!ok && lane == 0) { *failed = 1; atomicExch(p.error, 3); }
            ok = __all_sync(0xffffffffu, ok && *failed == 0);
            if (!ok) break;
            tc_fence_after();
            const int n = w.n0 + quarter * 32 + lane;
            const uint32_t acc_addr = tmem_base + (uint32_t)(b * buf_cols) + ((uint32_t)(quarter * 32) << 16);
            float bias_v = 0.f;
            if (p.bias && n < p.N)
                bias_v = p.bias_dt == F32 ? ((const float*)p.bias)[n] : __bfloat162float(((const __nv_bfloat16*)p.bias)[n]);
            if (p.tma_out) {
                for (int c0 = 0; c0 < p.tile_n; c0 += kChunk, ++chunk_count) {
                    if (w.t0 + c0 >= p.T) break;   // the same for all epilogue threads
                    uint8_t* stage = staging + (chunk_count & 1u) * kStagingBytes;
                    // the store that used this buffer two chunks ago has read it
                    if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    epilogue_barrier();
                    float g[32], up[32];
                    tmem_ld32(acc_addr + (uint32_t)c0, g);
                    if (p.dual) tmem_ld32(acc_addr + (uint32_t)(p.tile_n + c0), up);
                    const int f = quarter * 32 + lane;
                    // (the choice of the activation stays outside the loop over the chunk's 32 values: this epilogue's
                    // instruction count is what a gated unit's time is made of)
                    if (p.epilogue == EPI_SWIGLU) {
                        if (p.act == ACT_SILU) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) g[j] = up[j] * __fdividef(g[j], 1.0f + __expf(-g[j]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) g[j] = gated(p.act, g[j], up[j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) g[j] += bias_v;
                    }
                    if (p.out_dt == F32) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) ((float*)stage)[j * kTileM + f] = g[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) ((__nv_bfloat16*)stage)[j * kTileM + f] = __float2bfloat16_rn(g[j]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    epilogue_barrier();
                    if (issuer) {
                        if (p.epilogue == EPI_ACCUM) tma_add_2d(&map_out, stage, w.n0, w.t0 + c0);
                        else tma_store_2d(&map_out, stage, w.n0, w.t0 + c0);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            } else {
                for (int c0 = 0; c0 < p.tile_n; c0 += 16) {
                    if (w.t0 + c0 >= p.T) break;   // the same for the whole warp
                    float g[16], up[16], old[16];
                    tmem_ld16(acc_addr + (uint32_t)c0, g);
                    if (p.dual) tmem_ld16(acc_addr + (uint32_t)(p.tile_n + c0), up);
                    if (n >= p.N) continue;
                    if (p.epilogue == EPI_ACCUM) {   // all the old values first: the loads overlap
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = w.t0 + c0 + j;
                            old[j] = t < p.T ? ((const float*)p.out)[(size_t)t * p.N + n] : 0.f;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = w.t0 + c0 + j;
                        if (t >= p.T) break;
                        const size_t o = (size_t)t * p.N + n;
                        float v = g[j];
                        if (p.epilogue == EPI_PARTIAL) {
                            p.workspace[((size_t)w.split * p.T + t) * p.N + n] = v;
                            if (p.dual) p.workspace[(((size_t)p.splits + w.split) * p.T + t) * p.N + n] = up[j];
                            continue;
                        }
                        if (p.epilogue == EPI_SWIGLU) v = gated(p.act, v, up[j]);
                        else v += bias_v;
                        if (p.epilogue == EPI_ACCUM) ((float*)p.out)[o] = old[j] + v;
                        else if (p.out_dt == F32) ((float*)p.out)[o] = v;
                        else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v);
                    }
                }
            }
            // this accumulator may be overwritten by the MMAs of the unit after next
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[b]);
        }
        if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // shared memory stays valid until read
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*failed) {
        // the way out after a wait that ran out (drain.cuh): the copies asked for land, the MMAs issued finish, and only
        // then are tensor memory and this CTA's shared memory given up
        if (threadIdx.x == 0) {
            OutstandingFill left[8];
            const int n = outstanding_fills(fills_issued, fills_consumed, p.stages, left);
            for (int i = 0; i < n; ++i) mbar_wait(&full_bar[left[i].stage], left[i].parity);
        }
        if (warp == 1 && lane == 0 && mmas_issued) {
            umma_commit(&drain_bar);
            mbar_wait(&drain_bar, 0);
        }
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// The kernel for at most 160 tokens (decode batches beyond the weight-streaming kernel, short prompts, and the
// output head): one CTA per work unit, few registers, two CTAs to an SM. With so few tokens a
// unit is nothing but a stream of weight tiles, and two small CTAs keep more of them in flight
// than one persistent CTA does (measured on the 151,936 x 896 head at 8 tokens: 54 against 75 us).
//
// Where K is split, the CTAs of a tile are one thread-block cluster (grid x = the split): each leaves
// its partial sums in its own shared memory, and after a cluster barrier CTA r adds up the r-th part
// of the tile from all of them, in split order, through distributed shared memory, applies the
// epilogue and writes it. No partial sum goes to global memory and no second kernel runs (that
// kernel and the workspace's round trip cost 6 to 16 us a product at 64 tokens).
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr, uint32_t cta) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(cta));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
    return v;
}

__global__ void __launch_bounds__(kThreads, 2)
gemm_tc_small_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of the tiles is what the swizzle pattern assumes
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int a_bytes = kTileM * kStageK * 2 * (p.dual ? 2 : 1);
    const int b_bytes = p.tile_n * kStageK * 2;
    const int stage_bytes = a_bytes + b_bytes;
    uint64_t* full_bar = (uint64_t*)(smem + (size_t)p.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + p.stages;
    uint64_t* tmem_full_bar = empty_bar + p.stages;
    uint32_t* tmem_slot = (uint32_t*)(tmem_full_bar + 1);
    int* failed = (int*)(tmem_slot + 1);
    // for the way out after a failure (drain.cuh), in the dynamic allocation (a static one would lower its limit)
    uint64_t& drain_bar = *(uint64_t*)(tmem_slot + 2);
    int& fills_issued = *(int*)(tmem_slot + 4);
    int& fills_consumed = *(int*)(tmem_slot + 5);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, n0 = blockIdx.y * (p.halves ? kTileM / 2 : kTileM), t0 = blockIdx.z * p.tile_n;
    pdl_launch_dependents();
    const int kb_total = (p.K + kStageK - 1) / kStageK;
    const int kb_begin = split * p.kblocks_per_split;
    const int kb_end = min(kb_total, kb_begin + p.kblocks_per_split);
    const int n_kb = kb_end - kb_begin;   // >= 1 by construction of the grid
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < p.tile_n * (p.dual ? 2 : 1)) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(tmem_full_bar, 1);
        mbar_init(&drain_bar, 1);
        *failed = 0;
        fills_issued = fills_consumed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // the whole warp: one box of a stage's tiles a lane (see the persistent kernel)
        const StageBox box = stage_box(lane, a_bytes, p);
        const int row = box.from_x ? t0 + box.row : n0 + box.row;
        // The weights do not depend on the kernel before this one: the first stages' weight tiles are asked for
        // before the wait for it, their token tiles after.
        const int early = min(p.stages, n_kb);
        for (int i = 0; i < early; ++i) {
            if (lane == 0) mbar_expect_tx(&full_bar[i], (uint32_t)stage_bytes);
            __syncwarp();
            if (box.active && !box.from_x)
                tma_load_2d(smem + (size_t)i * stage_bytes + box.offset, &map_w, (kb_begin + i) * kStageK + box.k, row, &full_bar[i]);
        }
        pdl_wait();
        for (int i = 0; i < early; ++i)
            if (box.active && box.from_x)
                tma_load_2d(smem + (size_t)i * stage_bytes + box.offset, &map_x, (kb_begin + i) * kStageK + box.k, row, &full_bar[i]);
        int s = early == p.stages ? 0 : early;
        uint32_t phase = early == p.stages ? 1u : 0u;
        int issued = early;
        for (int i = early; i < n_kb; ++i) {
            if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], phase ^ 1u))) {
                if (lane == 0) { *failed = 1; atomicExch(p.error, 1); }
                break;
            }
            if (lane == 0) mbar_expect_tx(&full_bar[s], (uint32_t)stage_bytes);
            __syncwarp();
            if (box.active)
                tma_load_2d(smem + (size_t)s * stage_bytes + box.offset, box.from_x ? &map_x : &map_w, (kb_begin + i) * kStageK + box.k, row, &full_bar[s]);
            ++issued;
            if (++s == p.stages) { s = 0; phase ^= 1u; }
        }
        if (lane == 0) fills_issued = issued;
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(kTileM, p.tile_n);
            const uint64_t desc_first = smem_desc(smem_u32(smem));
            const uint64_t stage_step = (uint64_t)(stage_bytes >> 4), b_off = (uint64_t)(a_bytes >> 4);
            const uint64_t up_off = (uint64_t)((kTileM * kStageK * 2) >> 4);
            const uint64_t a_atom = (uint64_t)((kTileM * kBlockK * 2) >> 4), b_atom = (uint64_t)((p.tile_n * kBlockK * 2) >> 4);
            const uint32_t d_up = tmem_base + (uint32_t)p.tile_n;
            uint64_t da = desc_first;
            int s = 0;
            uint32_t phase = 0, acc = 0;
            bool ok = true;
            int consumed = 0;
            for (int i = 0; i < n_kb && ok; ++i) {
                if (!mbar_wait(&full_bar[s], phase)) { *failed = 1; atomicExch(p.error, 2); ok = false; break; }
                ++consumed;
                tc_fence_after();
                const uint64_t db = da + b_off, du = da + up_off;
#pragma unroll
                for (int k = 0; k < kStageK / kUmmaK; ++k) {
                    const uint64_t sub = (uint64_t)(((k % (kBlockK / kUmmaK)) * kUmmaK * 2) >> 4);
                    const uint64_t a_step = (k / (kBlockK / kUmmaK)) * a_atom + sub, b_step = (k / (kBlockK / kUmmaK)) * b_atom + sub;
                    umma_bf16(tmem_base, da + a_step, db + b_step, idesc, acc);
                    if (p.dual) umma_bf16(d_up, du + a_step, db + b_step, idesc, acc);
                    acc = 1;
                }
                umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
                da += stage_step;
                if (++s == p.stages) { s = 0; phase ^= 1u; da = desc_first; }
            }
            umma_commit(tmem_full_bar);        // the accumulator is complete once all MMAs are done
            fills_consumed = consumed;
        }
    } else {
        // epilogue warps 2..5: TMEM lanes of quarter (warp % 4)
        const int quarter = warp & 3;
        const int n = n0 + quarter * 32 + lane;
        pdl_wait();   // the output (read for "+=") and everything written below come after the kernel before
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
                float g[16], u[16], old[16];
                tmem_ld16(lane_base + (uint32_t)c0, g);
                if (p.dual) tmem_ld16(lane_base + (uint32_t)(p.tile_n + c0), u);
                if (p.cluster_reduce) {
                    // [gate | up][token][128 features] floats over the pipeline's stages, which are free: the
                    // accumulator is complete, so every MMA has read its operands
                    float* mine = reinterpret_cast<float*>(smem);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        mine[(c0 + j) * kTileM + quarter * 32 + lane] = g[j];
                        if (p.dual) mine[(p.tile_n + c0 + j) * kTileM + quarter * 32 + lane] = u[j];
                    }
                    continue;
                }
                if (n >= p.N) continue;
                if (p.epilogue == EPI_ACCUM) {   // all the old values first: the loads overlap
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = t0 + c0 + j;
                        old[j] = t < p.T ? ((const float*)p.out)[(size_t)t * p.N + n] : 0.f;
                    }
                }
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
                    if (p.epilogue == EPI_SWIGLU) v = gated(p.act, v, u[j]);
                    else v += bias_v;
                    if (p.epilogue == EPI_ACCUM) {
                        ((float*)p.out)[o] = old[j] + v;
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
    if (p.cluster_reduce) {
        // every thread of every CTA of the cluster comes here, whatever happened above
        cluster_barrier();
        if (warp >= 2) {
            const int pieces = p.tile_n * (kTileM / 4);                 // float4s of one accumulator
            const int per = (pieces + p.splits - 1) / p.splits;
            const int hi = min(pieces, (split + 1) * per);
            const uint32_t base = smem_u32(smem);
            if (p.final_epilogue == EPI_QKV_ROPE) {
                // q/k/v rows: bias, rotation of (d, d + head_dim / 2) with the position's angles, q to its matrix,
                // keys and values into the paged cache (src/model.c:501-526 of the reference: bias before the
                // rotation, the rotated key into the cache). The head size divides the tile's 128 rows, so both
                // halves of a head are in this tile; a thread takes four neighbouring dimensions and their partners.
                const SkinnyRope& r = p.rope;
                const int hd = r.head_dim, half = hd / 2, hp = hd / 8;       // hp: float4s of half a head
                const int pairs = p.tile_n * (kTileM / 8);
                const int per_pairs = (pairs + p.splits - 1) / p.splits;
                const int hi_pair = min(pairs, (split + 1) * per_pairs);
                PagedKV paged{r.page_table, r.table_stride, r.ring, r.kv_heads, hd};
                for (int pp = split * per_pairs + (int)threadIdx.x - 64; pp < hi_pair; pp += 128) {
                    const int tcol = pp / (kTileM / 8), q = pp - tcol * (kTileM / 8);
                    const int lo_piece = (q / hp) * (2 * hp) + q % hp, hi_piece = lo_piece + hp;
                    const int t = t0 + tcol, n_lo = n0 + lo_piece * 4;
                    if (t >= p.T || n_lo >= p.N) continue;
                    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi4 = lo;
#pragma unroll 4
                    for (int sp = 0; sp < p.splits; ++sp) {
                        const float4 a = ld_cluster_f4(base + (uint32_t)(tcol * (kTileM / 4) + lo_piece) * 16u, (uint32_t)sp);
                        const float4 b = ld_cluster_f4(base + (uint32_t)(tcol * (kTileM / 4) + hi_piece) * 16u, (uint32_t)sp);
                        lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
                        hi4.x += b.x; hi4.y += b.y; hi4.z += b.z; hi4.w += b.w;
                    }
                    float vl[4] = {lo.x, lo.y, lo.z, lo.w}, vh[4] = {hi4.x, hi4.y, hi4.z, hi4.w};
                    const int head = n_lo / hd, d = n_lo - head * hd;
                    if (p.bias) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            vl[e] += p.bias_dt == F32 ? ((const float*)p.bias)[n_lo + e] : __bfloat162float(((const __nv_bfloat16*)p.bias)[n_lo + e]);
                            vh[e] += p.bias_dt == F32 ? ((const float*)p.bias)[n_lo + half + e] : __bfloat162float(((const __nv_bfloat16*)p.bias)[n_lo + half + e]);
                        }
                    }
                    const int pos = r.positions[t];
                    const bool is_v = head >= r.heads + r.kv_heads;
                    if (!is_v) {
                        const float4 c4 = *reinterpret_cast<const float4*>(r.cos_table + (size_t)pos * half + d);
                        const float4 s4 = *reinterpret_cast<const float4*>(r.sin_table + (size_t)pos * half + d);
                        const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float r0 = vl[e] * cs[e] - vh[e] * sn[e], r1 = vl[e] * sn[e] + vh[e] * cs[e];
                            vl[e] = r0;
                            vh[e] = r1;
                        }
                    }
                    __nv_bfloat162 a0 = __floats2bfloat162_rn(vl[0], vl[1]), a1 = __floats2bfloat162_rn(vl[2], vl[3]);
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(vh[0], vh[1]), b1 = __floats2bfloat162_rn(vh[2], vh[3]);
                    uint2 pl, ph;
                    pl.x = *reinterpret_cast<uint32_t*>(&a0); pl.y = *reinterpret_cast<uint32_t*>(&a1);
                    ph.x = *reinterpret_cast<uint32_t*>(&b0); ph.y = *reinterpret_cast<uint32_t*>(&b1);
                    auto store = [&](__nv_bfloat16* dst) {
                        *reinterpret_cast<uint2*>(dst) = pl;
                        *reinterpret_cast<uint2*>(dst + half) = ph;
                    };
                    if (head < r.heads) {
                        store((__nv_bfloat16*)r.q_out + ((size_t)t * r.heads + head) * hd + d);
                    } else {
                        // keys and values: into the paged cache (with a ring, not the positions it has no place for any
                        // more) and, where the step attends over its own packed keys, into those
                        const int kvh = is_v ? head - r.heads - r.kv_heads : head - r.heads;
                        if (r.k_pool != nullptr && !(r.ring > 0 && r.token_end != nullptr && pos < r.token_end[t] - r.ring))
                            store((__nv_bfloat16*)(is_v ? r.v_pool : r.k_pool) + paged.row_offset(r.token_slot[t], pos, kvh) + d);
                        if (r.k_packed != nullptr)
                            store((__nv_bfloat16*)(is_v ? r.v_packed : r.k_packed) + ((size_t)t * r.kv_heads + kvh) * hd + d);
                    }
                }
            } else if (p.halves) {
                // the tile's rows 0-63 are gate rows n0.., rows 64-127 the up rows of the same features
                const int pieces_h = p.tile_n * (kTileM / 8);
                const int per_h = (pieces_h + p.splits - 1) / p.splits;
                const int hi_h = min(pieces_h, (split + 1) * per_h);
                const bool vec = (p.N & 3) == 0 && ((uintptr_t)p.out & 15) == 0;
                for (int c = split * per_h + (int)threadIdx.x - 64; c < hi_h; c += 128) {
                    const int tcol = c / (kTileM / 8), f4 = c - tcol * (kTileM / 8);
                    const int t = t0 + tcol, n = n0 + f4 * 4;
                    if (t >= p.T || n >= p.N) continue;
                    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
#pragma unroll 4
                    for (int sp = 0; sp < p.splits; ++sp) {
                        const float4 a = ld_cluster_f4(base + (uint32_t)(tcol * (kTileM / 4) + f4) * 16u, (uint32_t)sp);
                        const float4 b = ld_cluster_f4(base + (uint32_t)(tcol * (kTileM / 4) + kTileM / 8 + f4) * 16u, (uint32_t)sp);
                        g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
                        u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
                    }
                    const float v[4] = {gated(p.act, g.x, u.x), gated(p.act, g.y, u.y), gated(p.act, g.z, u.z), gated(p.act, g.w, u.w)};
                    const size_t o = (size_t)t * p.N + n;
                    if (vec && p.out_dt != F32) {
                        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi2 = __floats2bfloat162_rn(v[2], v[3]);
                        uint2 packed;
                        packed.x = *reinterpret_cast<uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<uint32_t*>(&hi2);
                        *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + o) = packed;
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (n + e >= p.N) break;
                            if (p.out_dt == F32) ((float*)p.out)[o + e] = v[e];
                            else ((__nv_bfloat16*)p.out)[o + e] = __float2bfloat16_rn(v[e]);
                        }
                    }
                }
            } else {
                // four features at a time where the output's rows allow it (then n + 3 < N whenever n < N)
                const bool vec = (p.N & 3) == 0 && ((uintptr_t)p.out & 15) == 0;
                for (int c = split * per + (int)threadIdx.x - 64; c < hi; c += 128) {
                    const int t = t0 + c / (kTileM / 4), n = n0 + (c % (kTileM / 4)) * 4;
                    if (t >= p.T || n >= p.N) continue;
                    const size_t o = (size_t)t * p.N + n;
                    float old[4] = {0.f, 0.f, 0.f, 0.f};
                    if (p.final_epilogue == EPI_ACCUM) {   // asked for before the sums: the trips overlap
                        if (vec) {
                            const float4 r = *reinterpret_cast<const float4*>((const float*)p.out + o);
                            old[0] = r.x; old[1] = r.y; old[2] = r.z; old[3] = r.w;
                        } else {
    #pragma unroll
                            for (int e = 0; e < 4; ++e) old[e] = n + e < p.N ? ((const float*)p.out)[o + e] : 0.f;
                        }
                    }
                    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
    #pragma unroll 4
                    for (int sp = 0; sp < p.splits; ++sp) {
                        const float4 a = ld_cluster_f4(base + (uint32_t)c * 16u, (uint32_t)sp);
                        g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
                        if (p.dual) {
                            const float4 b = ld_cluster_f4(base + (uint32_t)(pieces + c) * 16u, (uint32_t)sp);
                            u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
                        }
                    }
                    float v[4] = {g.x, g.y, g.z, g.w};
                    const float ups[4] = {u.x, u.y, u.z, u.w};
    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (p.final_epilogue == EPI_SWIGLU) v[e] = gated(p.act, v[e], ups[e]);
                        else if (p.bias && n + e < p.N)
                            v[e] += p.bias_dt == F32 ? ((const float*)p.bias)[n + e] : __bfloat162float(((const __nv_bfloat16*)p.bias)[n + e]);
                        v[e] += old[e];
                    }
                    if (vec) {
                        if (p.out_dt == F32) {
                            *reinterpret_cast<float4*>((float*)p.out + o) = make_float4(v[0], v[1], v[2], v[3]);
                        } else {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi2 = __floats2bfloat162_rn(v[2], v[3]);
                            uint2 packed;
                            packed.x = *reinterpret_cast<uint32_t*>(&lo);
                            packed.y = *reinterpret_cast<uint32_t*>(&hi2);
                            *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + o) = packed;
                        }
                    } else {
    #pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (n + e >= p.N) break;
                            if (p.out_dt == F32) ((float*)p.out)[o + e] = v[e];
                            else ((__nv_bfloat16*)p.out)[o + e] = __float2bfloat16_rn(v[e]);
                        }
                    }
                }
            }
        }
        cluster_barrier();   // no CTA leaves while another reads its shared memory
    }
    tc_fence_before();
    __syncthreads();
    if (*(volatile int*)failed) {
        // the way out after a wait that ran out (drain.cuh)
        if (threadIdx.x == 0) {
            OutstandingFill left[8];
            const int n = outstanding_fills(fills_issued, fills_consumed, p.stages, left);
            for (int i = 0; i < n; ++i) mbar_wait(&full_bar[left[i].stage], left[i].parity);
        }
        if (warp == 1 && lane == 0 && fills_consumed > 0) {
            umma_commit(&drain_bar);
            mbar_wait(&drain_bar, 0);
        }
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// Adds the splits in order and applies the epilogue. One thread per output element.
__global__ void splitk_reduce_kernel(GemmParams p) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)p.T * p.N;
    if (i >= total) return;
    int n = (int)(i % p.N);
    // all the partial sums first (at most 16 splits: the loads are in flight together), then added in split order
    float part[16], part_up[16];
#pragma unroll
    for (int s = 0; s < 16; ++s) {
        part[s] = s < p.splits ? p.workspace[(size_t)s * total + i] : 0.f;
        part_up[s] = p.dual && s < p.splits ? p.workspace[((size_t)p.splits + s) * total + i] : 0.f;
    }
    float g = 0.f, u = 0.f;
#pragma unroll
    for (int s = 0; s < 16; ++s) {
        if (s < p.splits) {
            g += part[s];
            u += part_up[s];
        }
    }
    float v = g;
    if (p.epilogue == EPI_SWIGLU) v = gated(p.act, g, u);
    else if (p.bias) v += p.bias_dt == F32 ? ((const float*)p.bias)[n] : __bfloat162float(((const __nv_bfloat16*)p.bias)[n]);
    if (p.epilogue == EPI_ACCUM) ((float*)p.out)[i] += v;
    else if (p.out_dt == F32) ((float*)p.out)[i] = v;
    else ((__nv_bfloat16*)p.out)[i] = __float2bfloat16_rn(v);
}

// A [rows, K] row-major bfloat16 matrix, boxes of box_rows x 64 elements, 128-byte swizzle.
// Rows and columns outside the matrix read as zero.
CUtensorMap make_map(const void* base, int rows, int K, int box_rows) {
    return tiled_map_2d("gemm_tc", CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, (uint64_t)K, (uint64_t)rows, (uint64_t)K * 2, kBlockK,
                        (uint32_t)box_rows, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

// The [T, N] row-major output, boxes of kChunk tokens x 128 features, no swizzle. Stores and
// adds outside the matrix are dropped.
CUtensorMap make_out_map(void* base, int T, int N, DType dt) {
    const size_t elem_bytes = dt == F32 ? 4 : 2;
    return tiled_map_2d("gemm_tc", dt == F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, (uint64_t)N,
                        (uint64_t)T, (uint64_t)N * elem_bytes, kTileM, kChunk, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
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

namespace {

// The small kernel's launch for a plan: pipeline stages, shared memory, and whether the CTAs along K can be one
// cluster (at most 8 CTAs, and the GPU can hold such a cluster).
struct SmallLaunch {
    int stages;
    size_t smem;
    bool cluster;
};
SmallLaunch small_launch(int tile_n, int splits, bool dual) {
    const int stage_bytes = kTileM * kStageK * 2 * (dual ? 2 : 1) + tile_n * kStageK * 2;
    SmallLaunch l{};
    l.stages = 100 * 1024 / stage_bytes;
    if (l.stages > 8) l.stages = 8;
    if (l.stages < 2) l.stages = 2;
    l.smem = (size_t)l.stages * stage_bytes + 1024 /*alignment*/ + (2 * l.stages + 1) * 8 + 32;
    static std::once_flag once;
    std::call_once(once, [] {
        cudaFuncSetAttribute(gemm_tc_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    });
    l.cluster = false;
    // the partial sums (tile_n x 128 floats, twice for a gated product) lie over the stages
    if (splits >= 2 && splits <= 8 && (size_t)tile_n * kTileM * 4 * (dual ? 2 : 1) <= (size_t)l.stages * stage_bytes) {
        struct Known { int splits; size_t smem; bool ok; };
        static std::mutex lock;
        static std::vector<Known> known;
        std::lock_guard<std::mutex> hold(lock);
        for (const Known& k : known)
            if (k.splits == splits && k.smem == l.smem) { l.cluster = k.ok; return l; }
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(splits, 1, 1);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = l.smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)splits;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_small_kernel, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        l.cluster = n >= 1;
        known.push_back({splits, l.smem, l.cluster});
    }
    return l;
}

}  // namespace


namespace {
// Up to this many tokens a product goes to the small kernel (one CTA per unit, K split inside a cluster), above it to the
// two-CTA kernel of gemm_pair.cu. Measured on the 0.5B sizes, whole prompt steps with the small kernel against the
// persistent one: 65 tokens 1.34 against 1.44 ms, 128 tokens 1.33 against 1.77, 160 tokens 1.53 against 1.77; beyond that
// the small kernel falls behind the two-CTA one (176 tokens 2.08 against 1.86).
constexpr int small_tokens() { return 160; }
}  // namespace

bool gemm_tc_supports(int T, int N, int K) { return T > 0 && N > 0 && K > 0 && K % 8 == 0; }

namespace {

// A gated product of the small kernel as tiles of 64 gate rows + their 64 up rows in one accumulator: half the
// shared memory of two accumulators, so two CTAs to an SM and twice the tiles. Gate and up meet where the
// cluster adds its sums up, so the plan needs that path (one split included). Returns the CTAs along K.
bool gated_halves_plan(int T, int N, int K, int* splits) {
    if (T > small_tokens()) return false;
    const int sms = device_sm_count();
    const int tiles = (N + kTileM / 2 - 1) / (kTileM / 2);
    const int t16 = T <= 64 ? ((T + 15) / 16) * 16 : ((T + 63) / 64) * 64;    // (above 64 rows: boxes of 64 rows)
    const int kb = (K + kStageK - 1) / kStageK;
    const SmallLaunch l = small_launch(t16, 2, false);
    int per_sm = (int)((size_t)227 * 1024 / l.smem);
    per_sm = per_sm > 2 ? 2 : (per_sm < 1 ? 1 : per_sm);
    int sp = sms * per_sm / tiles;
    if (sp > (kb + 1) / 2) sp = (kb + 1) / 2;
    if (sp > 8) sp = 8;
    if (sp < 1) sp = 1;
    const int per = (kb + sp - 1) / sp;
    sp = (kb + per - 1) / per;
    if (tiles * sp * 2 < sms) return false;
    if (sp > 1 && !small_launch(t16, sp, false).cluster) return false;
    *splits = sp;
    return true;
}

}  // namespace

void gemm_tc_plan(int T, int N, int K, bool dual, int* tile_n, int* splits) {
    if (dual && gated_halves_plan(T, N, K, splits)) {
        *tile_n = T <= 64 ? ((T + 15) / 16) * 16 : ((T + 63) / 64) * 64;
        return;
    }
    const int sms = device_sm_count();
    const int tiles_m = (N + kTileM - 1) / kTileM;
    const int t16 = ((T + 15) / 16) * 16;
    const int kb = (K + kStageK - 1) / kStageK;   // stages of K
    if (T <= small_tokens()) {
        // (a token tile of more than 64 rows is loaded as boxes of 64 rows: a multiple of 64)
        const int t16 = T <= 64 ? ((T + 15) / 16) * 16 : ((T + 63) / 64) * 64;
        // A handful of tokens: the product is bound by reading the weights once. One token tile (so that no
        // weight row is read twice) and, where the row tiles are too few to fill the machine, K split among the
        // CTAs of a cluster: as many as still run in ONE wave (measured at 64 tokens: 38 row tiles of a gated
        // product x 3 splits 12.7 us, x 4 splits = 152 CTAs on 148 SMs 19.0 us), at most 8 (clusters of 10 to 16
        // cost 1.3 to 4 times as much as clusters of 8) and about two stages of 128 of K each or more.
        const SmallLaunch l = small_launch(t16, 2, dual);
        int per_sm = (int)((size_t)227 * 1024 / l.smem);
        if (per_sm > 2) per_sm = 2;
        if (per_sm < 1) per_sm = 1;
        int sp = sms * per_sm / tiles_m;
        if (sp > (kb + 1) / 2) sp = (kb + 1) / 2;
        if (sp > 8) sp = 8;
        if (sp < 1) sp = 1;
        const int per = (kb + sp - 1) / sp;
        sp = (kb + per - 1) / per;
        if (tiles_m * sp * 2 >= sms) {
            *tile_n = t16;
            *splits = sp;
            return;
        }
        // (a matrix this small stays in L2: token tiles that read it again, as below, give more CTAs)
    }
    const int max_tile = dual ? 128 : 256;
    int tn = 16;
    // the largest token tile that keeps most of the machine busy, else the smallest that covers T
    for (int cand = max_tile; cand >= 16; cand >>= 1) {
        if (cand > t16 && cand > 16) continue;
        const int tiles = tiles_m * ((T + cand - 1) / cand);
        tn = cand;
        if (tiles * 10 >= sms * 7) break;
    }
    const int tiles = tiles_m * ((T + tn - 1) / tn);
    int sp = 1;
    if (tiles * 2 < sms && kb >= 2) {
        sp = (2 * sms + tiles - 1) / tiles;
        if (sp > kb) sp = kb;
        if (sp > 16) sp = 16;
        if (sp < 1) sp = 1;
    }
    // In the small kernel the CTAs along K can be one cluster that adds its sums up in shared memory: at most 8 of them. More
    // splits would go through a workspace and a second kernel (896 x 4864 at 64 tokens took 10 splits and the reduce
    // kernel; with 8 in a cluster the decode step of the 0.5B sizes at batch 64 went from 1.36 to 1.31 ms).
    // Up to 16 tokens the many splits and the reduce kernel are the faster way (the step at batch 16: 0.93 against 1.00 ms).
    if (T > 16 && T <= small_tokens() && sp > 8 && small_launch(tn, 8, dual).cluster) sp = 8;
    // no empty split: every unit along K gets at least one block
    const int per = (kb + sp - 1) / sp;
    sp = (kb + per - 1) / per;
    *tile_n = tn;
    *splits = sp;
}

size_t gemm_tc_workspace_bytes(int T, int N, int K, bool dual) {
    int tn, sp;
    gemm_tc_plan(T, N, K, dual, &tn, &sp);
    if (dual && gated_halves_plan(T, N, K, &sp)) return 0;
    if (sp > 1 && T <= small_tokens() && small_launch(tn, sp, dual).cluster) return 0;   // the splits are added up inside a cluster
    return sp > 1 ? (size_t)sp * (dual ? 2 : 1) * T * N * sizeof(float) : 0;
}

namespace {

// Whether the fused q/k/v epilogue can take this product: the small kernel (at most 160 tokens) with its sums added up
// inside the CTA or the cluster, and heads that do not straddle the tiles of 128 rows.
bool qkv_rope_possible(int T, int N, int K, const SkinnyRope& r) {
    if (T > small_tokens() || !gemm_tc_supports(T, N, K) || r.head_dim < 16 || kTileM % r.head_dim || r.rotary_dim != r.head_dim) return false;
    int tn, sp;
    gemm_tc_plan(T, N, K, false, &tn, &sp);
    return sp == 1 || small_launch(tn, sp, false).cluster;
}

void gemm_tc_impl(const void* x, const void* w, const void* bias, DType bias_dt, void* out, DType out_dt, int T, int N,
                  int K, int mode, int up_offset, float* workspace, int* error, const SkinnyRope* rope, cudaStream_t stream) {
    const int act = mode >> 8;      // mode: the epilogue in its low byte, the gated product's activation above it
    mode &= 0xff;
    if (act < 0 || act >= ACT_COUNT) throw std::invalid_argument("gemm_tc: unknown activation " + std::to_string(act));
    if (!gemm_tc_supports(T, N, K))
        throw std::invalid_argument("gemm_tc: K = " + std::to_string(K) + " must be a positive multiple of 8 (TMA rows start on 16 bytes)");
    if (((uintptr_t)x | (uintptr_t)w) & 15) throw std::invalid_argument("gemm_tc: operands must be 16-byte aligned");
    // many tokens: the two-CTA kernel
    if (!rope && gemm_pair_takes(x, w, out, out_dt, T, N, K, mode)) {
        gemm_pair(x, w, bias, bias_dt, out, out_dt, T, N, K, mode | act << 8, up_offset, error, stream);
        return;
    }
    const bool gated_mode = mode == EPI_SWIGLU;
    GemmParams p{};
    p.T = T; p.N = N; p.K = K;
    p.act = act;
    gemm_tc_plan(T, N, K, gated_mode, &p.tile_n, &p.splits);
    int halves_splits = 0;
    const bool halves = gated_mode && gated_halves_plan(T, N, K, &halves_splits);
    p.halves = halves ? 1 : 0;
    const bool dual = gated_mode && !halves;   // two accumulators
    const int kb = (K + kStageK - 1) / kStageK;
    p.kblocks_per_split = (kb + p.splits - 1) / p.splits;
    p.dual = dual ? 1 : 0;
    p.up_offset = up_offset;
    p.bias = bias; p.bias_dt = bias_dt;
    p.out = out; p.out_dt = out_dt;
    p.workspace = workspace;
    p.error = error;
    p.tiles_m = halves ? (N + kTileM / 2 - 1) / (kTileM / 2) : (N + kTileM - 1) / kTileM;
    p.tiles_t = (T + p.tile_n - 1) / p.tile_n;
    p.units = p.tiles_m * p.tiles_t * p.splits;
    const int final_mode = rope ? (int)EPI_QKV_ROPE : mode;
    if (rope) p.rope = *rope;
    p.epilogue = p.splits > 1 ? EPI_PARTIAL : final_mode;
    if (p.splits > 1 && !workspace && !(T <= small_tokens() && small_launch(p.tile_n, p.splits, dual).cluster))
        throw std::invalid_argument("gemm_tc: this shape splits K and needs a workspace");
    if (rope && !qkv_rope_possible(T, N, K, *rope))
        throw std::invalid_argument("gemm_tc: the fused q/k/v epilogue does not take this shape");
    // the output leaves through shared memory and TMA where TMA can address it: rows that start
    // on 16 bytes (TMA stores outside the matrix are dropped, so ragged edges need no care)
    const size_t out_elem = out_dt == F32 ? 4 : 2;
    // (a chunk is 32 tokens, so the token tile must hold at least one)
    p.tma_out = p.splits == 1 && p.tile_n >= kChunk && ((size_t)N * out_elem) % 16 == 0 && ((uintptr_t)out & 15) == 0 ? 1 : 0;
    const int stage_bytes = kTileM * kStageK * 2 * (dual ? 2 : 1) + p.tile_n * kStageK * 2;
    if (T <= small_tokens()) {
        // few tokens: one CTA per unit, two CTAs to an SM
        const SmallLaunch l = small_launch(p.tile_n, p.splits, dual);
        p.tma_out = 0;
        p.stages = l.stages;
        p.final_epilogue = final_mode;
        // (the fused q/k/v epilogue lives in the code that adds the splits up: a single split goes the same way)
        p.cluster_reduce = l.cluster || rope || halves ? 1 : 0;
        if (p.tiles_m > 65535 || p.tiles_t > 65535) throw std::invalid_argument("gemm_tc: more than 65535 tiles along a side");
        const CUtensorMap mw = make_map(w, gated_mode ? up_offset + N : N, K, kBoxRows);
        const CUtensorMap mx = make_map(x, T, K, p.tile_n < kBoxRows ? p.tile_n : kBoxRows);
        dim3 grid3(p.splits, p.tiles_m, p.tiles_t);
        launch_kernel("gemm_tc", gemm_tc_small_kernel, grid3, dim3(kThreads), l.smem, stream, l.cluster ? p.splits : 1,
                      dependent_launch_enabled(), mw, mx, p);
        note_launch(p.splits > 1 && !l.cluster ? 2 : 1);
        if (p.splits > 1 && !l.cluster) {
            p.epilogue = final_mode;
            size_t total = (size_t)T * N;
            splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(p);
        }
        return;
    }
    const int budget = 227 * 1024 - 1024 - 2 * kStagingBytes - 512;
    p.stages = budget / stage_bytes;
    if (p.stages > 8) p.stages = 8;
    if (p.stages < 2) throw std::runtime_error("gemm_tc: a pipeline stage does not fit shared memory twice");
    const size_t smem = (size_t)p.stages * stage_bytes + 1024 /*alignment*/ + 2 * kStagingBytes + (2 * p.stages + 4) * 8 + 48;
    const CUtensorMap map_w = make_map(w, dual ? up_offset + N : N, K, kBoxRows);
    const CUtensorMap map_x = make_map(x, T, K, p.tile_n < kBoxRows ? p.tile_n : kBoxRows);
    const CUtensorMap map_out = p.tma_out ? make_out_map(out, T, N, out_dt) : map_x;
    static std::once_flag attr_once;
    std::call_once(attr_once, [] {
        cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    });
    const int sms = device_sm_count();
    const int grid = p.units < sms ? p.units : sms;
    launch_kernel("gemm_tc", gemm_tc_kernel, dim3(grid), dim3(kThreads), smem, stream, 1, dependent_launch_enabled(), map_w, map_x, map_out, p);
    note_launch(p.splits > 1 ? 2 : 1);
    if (p.splits > 1) {
        p.epilogue = final_mode;
        size_t total = (size_t)T * N;
        splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(p);
    }
}

}  // namespace

void gemm_tc(const void* x, const void* w, const void* bias, DType bias_dt, void* out, DType out_dt, int T, int N,
             int K, int mode, int up_offset, float* workspace, int* error, cudaStream_t stream) {
    gemm_tc_impl(x, w, bias, bias_dt, out, out_dt, T, N, K, mode, up_offset, workspace, error, nullptr, stream);
}

bool gemm_tc_qkv_rope(const void* x, const void* w, const void* bias, DType bias_dt, int T, int K, const SkinnyRope& rope,
                      int* error, cudaStream_t stream) {
    const int N = (rope.heads + 2 * rope.kv_heads) * rope.head_dim;
    if (!qkv_rope_possible(T, N, K, rope)) return false;
    gemm_tc_impl(x, w, bias, bias_dt, nullptr, BF16, T, N, K, EPI_STORE, 0, nullptr, error, &rope, stream);
    return true;
}

}  // namespace sm
