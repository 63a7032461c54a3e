// out[t, n] = sum_k x[t, k] * w[n, k] for more than 160 tokens (prefill, prompt portions, large decode batches): two CTAs on two SMs work as a pair on one tile of
// 256 tokens x 128 or 256 output features with the two-CTA form of tcgen05.mma (cta_group::2).
//
// Why a pair. A tcgen05.mma reads both operands from shared memory. With one CTA and a 128 x 128 tile every 16 elements
// of K are 8 KB read for 64 cycles of arithmetic, which is all of an SM's 128 bytes a cycle before TMA has written a
// byte: the one-CTA kernel (gemm_tc.cu) ran the prefill's products at a third of the tensor pipe for that reason. In a
// pair each CTA holds 128 of the 256 token rows (the M side) and HALF of the tile's weight rows (the N side); the
// instruction takes the other half from the partner's shared memory. Per 64 elements of K a CTA then writes 32 KB by
// TMA and reads 32 KB for 512 cycles of arithmetic (256 features), so shared memory and the tensor pipe are level.
//
// Tokens are the M side here (one token per TMEM lane) and output features are the columns, the other way round from
// gemm_tc.cu. A gated product is ONE instruction 256 features wide: the leader CTA loads 128 gate rows, its partner
// the 128 up rows of the same features, and every thread of the epilogue finds gate and up of a feature 128 columns
// apart in its own lane.
//
// Roles in each CTA (192 threads): warp 0 loads its CTA's tiles by TMA into a ring of stages; warp 1 allocates tensor
// memory (both CTAs together) and, in the leader only, one thread issues the MMAs for the pair; warps 2-5 are the
// epilogue of the CTA's own 128 tokens. Tensor memory holds two accumulators, so the next unit's MMAs run while the
// epilogue drains the last. The kernel is persistent: pair i takes units i, i + pairs, ...
//
// Few tiles and a long K (the down product of a prompt of a few hundred tokens has 7 to 35 tiles for 74 pairs, and a pair
// streams K at what its two SMs take from L2): the launch then puts two pairs into one cluster of four CTAs, each pair
// with half of the tile's K. Every CTA leaves its share of the sums in its own shared memory (over the stages, idle by
// then), the cluster meets at a barrier, and each pair finishes half of the tile's columns: a thread reads its token's row
// of them from both pairs through distributed shared memory, adds them in the order of the pairs and hands the sum to
// TMA's float add. The order is fixed, so the result does not depend on which pair was first.
//
// The barriers. All "stage is full" barriers are the leader's: both CTAs' TMA copies count their bytes on them (the
// cta_group::2 form of the copy may signal the partner's barrier), and the leader expects the bytes of both. "Stage
// is empty" and "accumulator complete" are signalled by tcgen05.commit to the barrier of the same name in both CTAs at
// once. "Accumulator drained" is the leader's and counts the epilogue warps of both CTAs. No load here uses
// multicast. Every wait is bounded; a wait that runs out records a code in *error and the CTA writes nothing more.
// On the way out the leader waits (bounded) for the copies asked for and the MMAs issued, and both CTAs meet at a
// cluster barrier before tensor memory and shared memory are given up (drain.cuh), so neither leaves while its
// partner's instructions can still read its shared memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "drain.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "tcgen05.cuh"

namespace sm {

namespace {

constexpr int kRows = 128;           // token rows per CTA: the pair's tile is 2 * kRows tokens
constexpr int kBlockK = 64;          // bf16 elements per 128-byte swizzled row
constexpr int kAtoms = 2;            // swizzled blocks of K per pipeline stage
constexpr int kStageK = kAtoms * kBlockK;
constexpr int kUmmaK = 16;
constexpr int kBoxRows = 64;         // rows of one TMA box
constexpr int kThreads = 192;
constexpr int kStagingBytes = kRows * 128;   // one chunk on its way out: 128 token rows of 128 bytes, swizzled
constexpr int kBiasBytes = 256 * 4;          // the biases of a unit's columns
constexpr int kPairMinTokens = 161;  // (a pair's tile is 256 tokens. Measured on the 0.5B sizes, whole prompt steps: 160 tokens 1.84 ms
                                      // against 1.77 with the one-CTA kernel, 176 tokens 1.86 against 1.93, 700 tokens 2.17 against 3.13)
// A gated product is ahead here earlier: launch by launch from 65 tokens, where the one-CTA kernel's token tile leaves 64
// (0.5B sizes, 65 / 160 tokens: 12.0 / 15.9 -> 10.1 / 10.0 us; 7B sizes: 68 / 90 -> 50 / 53), but inside a whole step only
// from about 112 (its CTAs fill the SMs, so its neighbours in the chain overlap it less: prompt steps of 65 / 100 / 128 / 160
// tokens 1.19 / 1.28 / 1.32 / 1.52 -> 1.21 / 1.29 / 1.30 / 1.43 ms). A q/k/v product with its rotation and the += products
// stay with the one-CTA kernel up to 160 tokens (down at 160 tokens: 11.5 us there against 21.4 here, one pair a feature tile).
constexpr int kPairMinTokensGated = 112;
// Pairs that may share a unit's K. The kernel takes 2 or 4; with 4 (clusters of 8 CTAs) whole prompt steps of the 0.5B sizes were
// no faster than with 2 (176 / 512 / 1,024 tokens: 1.57 / 1.76 / 2.05 ms against 1.54 / 1.74 / 2.06; 1.68 / 1.86 / 2.16 without).
constexpr int kPairMaxSplits = 2;

enum PairEpilogue : int { P_STORE = 0, P_ACCUM = 1, P_GATED = 2, P_QKV = 3 };

struct PairParams {
    int T, N, K;
    int tile_f;               // the instruction's N: weight rows per tile, 128 or 256 (gated: 128 gate + 128 up rows)
    int half;                 // tile_f / 2: the weight rows each CTA loads
    int stages;
    int epilogue;
    int up_offset;            // gated: the up rows lie this many rows below the gate rows
    int act;
    const void* bias;         // [N] or null
    int bias_dt;
    int out_dt;
    int* error;
    int tiles_f, units;       // feature tiles; units = feature tiles x token tiles
    int splits;               // pairs that share a unit's K (1, 2 or 4): a cluster of 2 * splits CTAs, each pair with
    int kb_per;               // kb_per stages of K, their sums added up through distributed shared memory
    PairRope rope;            // P_QKV: the heads, the rotation's tables and where q, keys and values go
};


using namespace tc5;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of this CTA's shared address `addr` in CTA `rank`.
__device__ __forceinline__ uint32_t in_cta(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ void pair_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile into this CTA's shared memory, its bytes counted on a barrier that may be the partner's.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_in_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_in_cluster) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the MMAs issued so far are done, on the barrier at this address in BOTH CTAs of the pair.
__device__ __forceinline__ void umma_commit_both(uint64_t* bar, uint16_t both) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void umma_commit_pair_local(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_in_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_in_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mbar_arrive_in_cluster(uint32_t bar_in_cluster) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_in_cluster) : "memory");
}
// Bounded wait on a barrier of this CTA on which the partner arrives too.
__device__ __forceinline__ bool mbar_wait_pair(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Sixteen bytes of row `row` of a staged chunk: rows are 128 bytes, and the 16-byte pieces of a row are exchanged
// among themselves by the row's number (the 128-byte swizzle that the output's tensor map undoes), so that the 32
// threads of a warp, each writing its own row, spread over all banks.
__device__ __forceinline__ void stage_piece(uint8_t* stage, int row, int piece, uint4 v) {
    *(uint4*)(stage + row * 128 + ((piece ^ (row & 7)) << 4)) = v;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(const uint32_t*)&v;
}
__device__ __forceinline__ float bias_at(const PairParams& p, int n) {
    if (!p.bias || n >= p.N) return 0.f;
    return p.bias_dt == F32 ? ((const float*)p.bias)[n] : __bfloat162float(((const __nv_bfloat16*)p.bias)[n]);
}

// What lane `lane` of the loading warp brings of every stage. A stage lies in shared memory as
// [block of K][128 token rows], then [block of K][half weight rows], every row 128 bytes; the tiles go as boxes of
// kBoxRows rows, one box a lane.
struct PairBox {
    bool active, from_x;
    int offset;               // bytes from the stage's start
    int row;                  // first row, relative to the CTA's first token row / first weight row
    int k;                    // first element of K, relative to the stage's
};
__device__ __forceinline__ PairBox pair_box(int lane, const PairParams& p) {
    constexpr int kTokenBoxes = kAtoms * (kRows / kBoxRows);
    const int parts = p.half / kBoxRows;
    PairBox b{false, false, 0, 0, 0};
    if (lane < kTokenBoxes) {
        const int atom = lane / (kRows / kBoxRows), part = lane % (kRows / kBoxRows);
        b.active = b.from_x = true;
        b.offset = (atom * kRows + part * kBoxRows) * 128;
        b.row = part * kBoxRows;
        b.k = atom * kBlockK;
    } else if (lane < kTokenBoxes + kAtoms * parts) {
        const int idx = lane - kTokenBoxes, atom = idx / parts, part = idx % parts;
        b.active = true;
        b.offset = kRows * kStageK * 2 + (atom * p.half + part * kBoxRows) * 128;
        b.row = part * kBoxRows;
        b.k = atom * kBlockK;
    }
    return b;
}

struct PairUnit {
    int t0;        // this CTA's first token
    int w0;        // this CTA's first weight row
    int n0;        // the tile's first output feature
};
__device__ __forceinline__ PairUnit pair_unit(const PairParams& p, int u, int rank) {
    const int tf = u % p.tiles_f, tt = u / p.tiles_f;
    PairUnit r;
    r.t0 = tt * 2 * kRows + rank * kRows;
    if (p.epilogue == P_GATED) {
        r.n0 = tf * p.half;
        r.w0 = r.n0 + (rank ? p.up_offset : 0);
    } else {
        r.n0 = tf * p.tile_f;
        r.w0 = r.n0 + rank * p.half;
    }
    return r;
}

// One group of 32 columns of this thread's token on its way out: the values (for a gated product act(gate) * up, else
// the sum plus the bias) as 16-byte pieces of the staged row.
template <bool WIDE, bool GATED>
__device__ __forceinline__ void group_out(const PairParams& p, uint32_t (&gr)[32], uint32_t (&ur)[32], const float* bias32, uint8_t* stage,
                                          int row, int first_piece) {
    float g[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) g[j] = __uint_as_float(gr[j]);
    if (GATED) {
        // (the choice of the activation stays outside the loop over the 32 values: this epilogue's instruction count
        // is what a gated unit's time is made of)
        if (p.act == ACT_SILU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = __uint_as_float(ur[j]) * __fdividef(g[j], 1.0f + __expf(-g[j]));
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = __uint_as_float(ur[j]) * activate_fast(p.act, g[j]);
        }
    } else if (bias32) {
        // (the unit's biases lie in shared memory: every thread reads the same word, once a group)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 b = ((const float4*)bias32)[j];
            g[4 * j] += b.x; g[4 * j + 1] += b.y; g[4 * j + 2] += b.z; g[4 * j + 3] += b.w;
        }
    }
    if (WIDE) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            stage_piece(stage, row, first_piece + j, make_uint4(__float_as_uint(g[4 * j]), __float_as_uint(g[4 * j + 1]),
                                                                __float_as_uint(g[4 * j + 2]), __float_as_uint(g[4 * j + 3])));
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            stage_piece(stage, row, first_piece + j, make_uint4(pack_bf16(g[8 * j], g[8 * j + 1]), pack_bf16(g[8 * j + 2], g[8 * j + 3]),
                                                                pack_bf16(g[8 * j + 4], g[8 * j + 5]), pack_bf16(g[8 * j + 6], g[8 * j + 7])));
    }
}

// The epilogue of one unit for this thread's token: 64 columns a turn, as two groups of 32 whose loads from tensor
// memory run one group ahead of the arithmetic. A turn of float output fills both staging buffers (a row of 32 floats
// is the 128 bytes a staged row holds), a turn of bfloat16 output one buffer, the other still being read by the store
// of the turn before.
template <bool WIDE, bool GATED>
__device__ __forceinline__ void unit_out(const PairParams& p, const PairUnit& w, uint32_t acc, int row, uint8_t* staging,
                                         uint32_t& turn_count, bool issuer, const CUtensorMap& map_out, const float* bias_s) {
    const int out_cols = GATED ? p.half : p.tile_f;
    uint32_t ga[32], ua[32], gb[32], ub[32];
    tmem_ld32_issue(acc, ga);
    if (GATED) tmem_ld32_issue(acc + (uint32_t)p.half, ua);
    for (int c0 = 0; c0 < out_cols; c0 += 64, ++turn_count) {
        if (w.n0 + c0 >= p.N) break;                 // the same for all epilogue threads
        uint8_t* first = WIDE ? staging : staging + (turn_count & 1u) * kStagingBytes;
        uint8_t* second = WIDE ? staging + kStagingBytes : first;
        // the stores that used these buffers have read them
        if (issuer) {
            if (WIDE) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        }
        epilogue_barrier();
        tmem_ld_wait(ga);
        if (GATED) tmem_ld_wait(ua);
        tmem_ld32_issue(acc + (uint32_t)(c0 + 32), gb);
        if (GATED) tmem_ld32_issue(acc + (uint32_t)(p.half + c0 + 32), ub);
        group_out<WIDE, GATED>(p, ga, ua, bias_s ? bias_s + c0 : nullptr, first, row, 0);
        tmem_ld_wait(gb);
        if (GATED) tmem_ld_wait(ub);
        if (c0 + 64 < out_cols && w.n0 + c0 + 64 < p.N) {
            tmem_ld32_issue(acc + (uint32_t)(c0 + 64), ga);
            if (GATED) tmem_ld32_issue(acc + (uint32_t)(p.half + c0 + 64), ua);
        }
        group_out<WIDE, GATED>(p, gb, ub, bias_s ? bias_s + c0 + 32 : nullptr, second, row, WIDE ? 0 : 4);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        epilogue_barrier();
        if (issuer) {
            if (p.epilogue == P_ACCUM) {
                tma_add_2d(&map_out, first, w.n0 + c0, w.t0);
                tma_add_2d(&map_out, second, w.n0 + c0 + 32, w.t0);
            } else {
                tma_store_2d(&map_out, first, w.n0 + c0, w.t0);
                if (WIDE) tma_store_2d(&map_out, second, w.n0 + c0 + 32, w.t0);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
}

// The epilogue of a q/k/v product: the tile's columns are whole heads (64 or 128 wide). Each thread adds the bias to its
// token's row of a head, rotates it by the token's position if it is a query or key head (pairs (i, i + head_dim / 2),
// the angle's cosine and sine from the tables, all in float), rounds to bfloat16 once and hands the head to TMA: queries
// to q_out, keys and values to the packed tensors of the step; keys and values also go straight from the registers into
// the paged cache (unless the ring has no place for the position any more).
__device__ __forceinline__ void qkv_heads_out(const PairParams& p, const PairUnit& w, uint32_t acc, int row, uint8_t* staging,
                                              uint32_t& chunk_count, bool issuer, const CUtensorMap& map_q,
                                              const CUtensorMap& map_k, const CUtensorMap& map_v, bool tables_held,
                                              const float4 (&held_cos)[8], const float4 (&held_sin)[8], const float* bias_s) {
    const PairRope& r = p.rope;
    const int hd = r.head_dim, half = hd >> 1, chunks = hd / 64;
    const int t = w.t0 + row;
    const bool live = t < p.T;
    const int pos = live ? r.positions[t] : 0;
    for (int col0 = 0; col0 < p.tile_f; col0 += hd) {
        const int head = (w.n0 + col0) / hd;
        if (head >= r.heads + 2 * r.kv_heads) break;           // the same for all epilogue threads
        const bool is_q = head < r.heads, is_v = head >= r.heads + r.kv_heads;
        const int kvh = is_q ? 0 : head - r.heads - (is_v ? r.kv_heads : 0);
        // a head of 128 takes both staging buffers, a head of 64 the one that the head before did not take
        uint8_t* first = chunks == 2 ? staging : staging + (chunk_count & 1u) * kStagingBytes;
        if (issuer) {
            if (chunks == 2) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        }
        epilogue_barrier();
        __nv_bfloat16* pool_row = nullptr;
        if (!is_q && live && r.k_pool != nullptr && !(r.ring > 0 && pos < r.token_end[t] - r.ring)) {
            const PagedKV paged{r.page_table, r.table_stride, r.ring, r.kv_heads, hd};
            pool_row = (__nv_bfloat16*)(is_v ? r.v_pool : r.k_pool) + paged.row_offset(r.token_slot[t], pos, kvh);
        }
        for (int s = 0; s < half; s += 32) {
            uint32_t lo_r[32], hi_r[32];
            tmem_ld32_issue(acc + (uint32_t)(col0 + s), lo_r);
            tmem_ld32_issue(acc + (uint32_t)(col0 + half + s), hi_r);
            tmem_ld_wait(lo_r);
            tmem_ld_wait(hi_r);
            float lo[32], hi[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) { lo[j] = __uint_as_float(lo_r[j]); hi[j] = __uint_as_float(hi_r[j]); }
            if (bias_s) {
                const float4* bl = (const float4*)(bias_s + col0 + s);
                const float4* bh = (const float4*)(bias_s + col0 + half + s);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 l = bl[j], h = bh[j];
                    lo[4 * j] += l.x; lo[4 * j + 1] += l.y; lo[4 * j + 2] += l.z; lo[4 * j + 3] += l.w;
                    hi[4 * j] += h.x; hi[4 * j + 1] += h.y; hi[4 * j + 2] += h.z; hi[4 * j + 3] += h.w;
                }
            }
            if (!is_v) {
                const float4* c4 = (const float4*)(r.cos_table + (size_t)pos * half + s);
                const float4* s4 = (const float4*)(r.sin_table + (size_t)pos * half + s);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 c = tables_held ? held_cos[j] : __ldg(c4 + j), sn = tables_held ? held_sin[j] : __ldg(s4 + j);
                    const float cs[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float a = lo[4 * j + e], b = hi[4 * j + e];
                        lo[4 * j + e] = a * cs[e] - b * ss[e];
                        hi[4 * j + e] = a * ss[e] + b * cs[e];
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 l = make_uint4(pack_bf16(lo[8 * j], lo[8 * j + 1]), pack_bf16(lo[8 * j + 2], lo[8 * j + 3]),
                                           pack_bf16(lo[8 * j + 4], lo[8 * j + 5]), pack_bf16(lo[8 * j + 6], lo[8 * j + 7]));
                const uint4 h = make_uint4(pack_bf16(hi[8 * j], hi[8 * j + 1]), pack_bf16(hi[8 * j + 2], hi[8 * j + 3]),
                                           pack_bf16(hi[8 * j + 4], hi[8 * j + 5]), pack_bf16(hi[8 * j + 6], hi[8 * j + 7]));
                const int lo_col = s + 8 * j, hi_col = half + s + 8 * j;      // columns within the head
                stage_piece(first + (lo_col >> 6) * kStagingBytes, row, (lo_col & 63) >> 3, l);
                stage_piece(first + (hi_col >> 6) * kStagingBytes, row, (hi_col & 63) >> 3, h);
            }
        }
        if (!is_q && r.k_pool != nullptr) {
            // Keys and values into the cache, from the staged rows of this warp's own 32 tokens: eight lanes write the
            // 128 bytes of a row's chunk side by side (a thread writing its own row would touch 32 lines an instruction)
            __syncwarp();
            const int lane = row & 31, piece = lane & 7;
            for (int c = 0; c < chunks; ++c) {
                const uint8_t* chunk = first + c * kStagingBytes;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int src = 4 * i + (lane >> 3);                   // the lane whose token this is
                    __nv_bfloat16* dst = (__nv_bfloat16*)__shfl_sync(0xffffffffu, (unsigned long long)pool_row, src);
                    const int rr = (row & ~31) + src;
                    if (dst) *(uint4*)(dst + 64 * c + 8 * piece) = *(const uint4*)(chunk + rr * 128 + ((piece ^ (rr & 7)) << 4));
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        epilogue_barrier();
        if (issuer) {
            const CUtensorMap* map = is_q ? &map_q : (is_v ? &map_v : &map_k);
            const bool wanted = is_q || r.k_packed != nullptr;
            if (wanted)
                for (int c = 0; c < chunks; ++c) tma_store_2d(map, first + c * kStagingBytes, (is_q ? head : kvh) * hd + 64 * c, w.t0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        ++chunk_count;
    }
}

// Split K: this CTA's share of a tile's sums (128 tokens x 128 features, float) out of tensor memory into its shared
// memory, over the stages, which are idle once the pair's MMAs are done: four chunks of 32 columns in the staged layout.
__device__ __forceinline__ void split_stash(uint32_t acc, int row, uint8_t* smem) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        float v[32];
        tmem_ld32(acc + (uint32_t)(c * 32), v);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            stage_piece(smem + c * kStagingBytes, row, j, make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                                                                    __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3])));
    }
}

// Split K, after the cluster's barrier: pair `slice` finishes columns [slice * 128 / splits, +128 / splits) of the tile.
// Each thread adds up its token's row of those columns over the pairs, always in the order of the pairs (the sums do
// not depend on who was first), reading the other pairs' shares from their CTAs of the same rank through distributed
// shared memory, and the sum is added to the output by TMA.
__device__ __forceinline__ void split_finish(const PairParams& p, const PairUnit& w, bool issuer, int row, int rank, int slice,
                                             uint8_t* smem, uint8_t* staging, const CUtensorMap& map_out, bool failed) {
    const int chunks = 4 / p.splits;                // chunks of 32 columns a pair finishes
    for (int cc = 0; cc < chunks; ++cc) {
        const int c = slice * chunks + cc;
        float4 sum[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!failed) {
            // (all the loads first, then the additions: a load from another SM's shared memory takes about a microsecond)
            const uint32_t mine = smem_u32(smem + c * kStagingBytes + row * 128);
            float4 v[4][8];
#pragma unroll
            for (int s2 = 0; s2 < 4; ++s2) {
                if (s2 < p.splits) {
                    const uint32_t theirs = in_cta(mine, (uint32_t)(2 * s2 + rank));
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(v[s2][j].x), "=f"(v[s2][j].y), "=f"(v[s2][j].z), "=f"(v[s2][j].w)
                                     : "r"(theirs + (uint32_t)((j ^ (row & 7)) << 4)));
                }
            }
#pragma unroll
            for (int s2 = 0; s2 < 4; ++s2) {
                if (s2 < p.splits) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        sum[j].x += v[s2][j].x; sum[j].y += v[s2][j].y; sum[j].z += v[s2][j].z; sum[j].w += v[s2][j].w;
                    }
                }
            }
        }
        uint8_t* out_chunk = staging + (cc & 1) * kStagingBytes;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            stage_piece(out_chunk, row, j, make_uint4(__float_as_uint(sum[j].x), __float_as_uint(sum[j].y), __float_as_uint(sum[j].z),
                                                      __float_as_uint(sum[j].w)));
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        epilogue_barrier();
        if (issuer && !failed && w.t0 < p.T) {
            tma_add_2d(&map_out, out_chunk, w.n0 + c * 32, w.t0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory stays valid until read
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, PairParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // (the same offset in both CTAs: the instruction addresses the partner's tiles by this CTA's descriptors)
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int a_bytes = kRows * kStageK * 2;
    const int stage_bytes = a_bytes + p.half * kStageK * 2;
    uint8_t* staging = smem + (size_t)p.stages * stage_bytes;                 // 2 x kStagingBytes
    uint64_t* full_bar = (uint64_t*)(staging + 2 * kStagingBytes);
    uint64_t* empty_bar = full_bar + p.stages;
    uint64_t* tfull_bar = empty_bar + p.stages;       // [2] accumulator complete
    uint64_t* tempty_bar = tfull_bar + 2;             // [2] accumulator drained (the leader's counts)
    uint64_t* drain_bar = tempty_bar + 2;
    uint32_t* tmem_slot = (uint32_t*)(drain_bar + 1);
    volatile int* failed = (volatile int*)(tmem_slot + 1);
    long long& fills_issued = *(long long*)(tmem_slot + 2);
    long long& fills_consumed = *(long long*)(tmem_slot + 4);
    int& mmas_issued = *(int*)(tmem_slot + 6);
    float* bias_s = (float*)((uint8_t*)full_bar + 256);                       // [tile_f] the biases of the unit on its way out

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_rank();
    const int rank = (int)(crank & 1u);              // within the pair
    const int slice = (int)(crank >> 1);             // which share of K this pair has, where a cluster holds several pairs
    const uint32_t lead = crank & ~1u;               // the pair's leader, as a rank of the cluster
    const uint16_t both = (uint16_t)(3u << lead);    // the pair, as a mask of the cluster's CTAs
    const bool leader = rank == 0;
    const int pair = (int)blockIdx.x / (2 * p.splits), pairs = (int)gridDim.x / (2 * p.splits);
    pdl_launch_dependents();
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * p.tile_f) tmem_cols <<= 1;

    if (threadIdx.x == 32) {
        prefetch_tensor_map(&map_w);
        prefetch_tensor_map(&map_x);
        prefetch_tensor_map(&map_out);
        if (p.epilogue == P_QKV && p.rope.k_packed != nullptr) {
            prefetch_tensor_map(&map_k);
            prefetch_tensor_map(&map_v);
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 8); }
        mbar_init(drain_bar, 1);
        *failed = 0;
        fills_issued = fills_consumed = 0;
        mmas_issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    pair_barrier();            // the partner's barriers exist before anything is signalled on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int kb_first = slice * p.kb_per;            // this pair's stages of K
    const int kb_total = min(p.kb_per, (p.K + kStageK - 1) / kStageK - kb_first);

    if (warp == 0) {
        const PairBox box = pair_box(lane, p);
        const uint32_t full0 = in_cta(smem_u32(full_bar), lead);   // the leader's "full" barriers
        // The weights do not depend on the kernel before this one: the weight tiles of the first unit's first stages
        // are asked for before the wait for it, the token tiles after.
        const int early = min(p.stages, kb_total);
        {
            const PairUnit w = pair_unit(p, pair, rank);        // the grid never has more pairs than units
            if (leader && lane == 0)
                for (int i = 0; i < early; ++i) mbar_expect_tx(&full_bar[i], 2u * (uint32_t)stage_bytes);
            __syncwarp();
            if (box.active && !box.from_x)
                for (int i = 0; i < early; ++i)
                    tma_load_2d_pair(smem + (size_t)i * stage_bytes + box.offset, &map_w, (kb_first + i) * kStageK + box.k, w.w0 + box.row, full0 + 8u * i);
            pdl_wait();
            for (int i = 0; i < early; ++i)
                if (box.active && box.from_x)
                    tma_load_2d_pair(smem + (size_t)i * stage_bytes + box.offset, &map_x, (kb_first + i) * kStageK + box.k, w.t0 + box.row, full0 + 8u * i);
        }
        int s = early == p.stages ? 0 : early;
        uint32_t phase = early == p.stages ? 1u : 0u;
        long long issued = early;
        bool ok = true;
        for (int u = pair; u < p.units && ok && !*failed; u += pairs) {
            const PairUnit w = pair_unit(p, u, rank);
            const int row = box.from_x ? w.t0 + box.row : w.w0 + box.row;
            for (int kb = u == pair ? early : 0; kb < kb_total; ++kb) {
                ok = __all_sync(0xffffffffu, mbar_wait_pair(&empty_bar[s], phase ^ 1u));
                if (!ok) {
                    if (lane == 0) { *failed = 1; atomicExch(p.error, 1); }
                    break;
                }
                if (leader && lane == 0) mbar_expect_tx(&full_bar[s], 2u * (uint32_t)stage_bytes);
                __syncwarp();
                if (box.active)
                    tma_load_2d_pair(smem + (size_t)s * stage_bytes + box.offset, box.from_x ? &map_x : &map_w, (kb_first + kb) * kStageK + box.k, row,
                                     full0 + 8u * s);
                ++issued;
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
        }
        if (lane == 0) fills_issued = issued;
        // Not before the MMAs have read what was loaded last: they read this CTA's shared memory on the partner's behalf.
        for (int j = 0; j < p.stages && ok && !*failed; ++j) {
            ok = __all_sync(0xffffffffu, mbar_wait_pair(&empty_bar[s], phase ^ 1u));
            if (!ok && lane == 0) { *failed = 1; atomicExch(p.error, 5); }
            if (++s == p.stages) { s = 0; phase ^= 1u; }
        }
    } else if (warp == 1) {
        if (leader && lane == 0) {
            const uint32_t idesc = instr_desc(2 * kRows, p.tile_f);
            const uint64_t desc_first = smem_desc(smem_u32(smem));
            const uint64_t stage_step = (uint64_t)(stage_bytes >> 4), b_off = (uint64_t)(a_bytes >> 4);
            const uint64_t a_atom = (uint64_t)((kRows * kBlockK * 2) >> 4), b_atom = (uint64_t)((p.half * kBlockK * 2) >> 4);
            uint64_t da = desc_first;
            int s = 0;
            uint32_t phase = 0;
            int i = 0;
            long long consumed = 0;
            for (int u = pair; u < p.units && !*failed; u += pairs, ++i) {
                const int b = i & 1;
                // the epilogues of both CTAs have drained this accumulator (its first use is free)
                if (!mbar_wait_pair(&tempty_bar[b], (((uint32_t)i >> 1) & 1u) ^ 1u)) { *failed = 1; atomicExch(p.error, 4); break; }
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(b * p.tile_f);
                uint32_t acc = 0;
                for (int kb = 0; kb < kb_total; ++kb) {
                    if (!mbar_wait_pair(&full_bar[s], phase)) { *failed = 1; atomicExch(p.error, 2); break; }
                    ++consumed;
                    tc_fence_after();
                    const uint64_t db = da + b_off;
#pragma unroll
                    for (int k = 0; k < kStageK / kUmmaK; ++k) {
                        const uint64_t sub = (uint64_t)(((k % (kBlockK / kUmmaK)) * kUmmaK * 2) >> 4);
                        umma_bf16_pair(d, da + (k / (kBlockK / kUmmaK)) * a_atom + sub, db + (k / (kBlockK / kUmmaK)) * b_atom + sub, idesc, acc);
                        acc = 1;
                    }
                    umma_commit_both(&empty_bar[s], both);   // the stage is free in both CTAs once these MMAs have read it
                    da += stage_step;
                    if (++s == p.stages) { s = 0; phase ^= 1u; da = desc_first; }
                }
                if (*failed) break;
                umma_commit_both(&tfull_bar[b], both); // the accumulator is complete in both CTAs
            }
            fills_consumed = consumed;
            mmas_issued = consumed > 0;
        }
    } else {
        // epilogue warps 2..5: the TMEM lanes of quarter (warp % 4), one token per thread
        const int quarter = warp & 3;
        const bool issuer = warp == 2 && lane == 0;
        const int row = quarter * 32 + lane;
        const uint32_t tempty0 = in_cta(smem_u32(tempty_bar), lead);
        int i = 0;
        uint32_t chunk_count = 0;
        pdl_wait();   // the output (read for "+=") and everything written below come after the kernel before
        for (int u = pair; u < p.units; u += pairs, ++i) {
            const PairUnit w = pair_unit(p, u, rank);
            const int b = i & 1;
            // q/k/v with heads of 64: this token's row of the cosine and sine tables (32 floats each) is asked for while
            // the unit's MMAs still run, and serves every head of the unit (each thread reads a row of its own: 32 lines
            // a warp and instruction, which on the way out cost as much as the rest of the epilogue)
            float4 held_cos[8], held_sin[8];
            const bool tables_held = p.epilogue == P_QKV && p.rope.head_dim == 64;
            if (tables_held) {
                const int t = w.t0 + row;
                const int pos = t < p.T ? p.rope.positions[t] : 0;
                const float4* c4 = (const float4*)(p.rope.cos_table + (size_t)pos * 32);
                const float4* s4 = (const float4*)(p.rope.sin_table + (size_t)pos * 32);
#pragma unroll
                for (int j = 0; j < 8; ++j) { held_cos[j] = __ldg(c4 + j); held_sin[j] = __ldg(s4 + j); }
            }
            if (p.bias) {
                // the unit's biases into shared memory while its MMAs run (the unit before has been read out)
                epilogue_barrier();
                for (int c = row; c < p.tile_f; c += kRows) bias_s[c] = bias_at(p, w.n0 + c);
                epilogue_barrier();
            }
            bool ok = mbar_wait_pair(&tfull_bar[b], ((uint32_t)i >> 1) & 1u);
            if (!ok && lane == 0) { *failed = 1; atomicExch(p.error, 3); }
            ok = __all_sync(0xffffffffu, ok && *failed == 0);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + (uint32_t)(b * p.tile_f) + ((uint32_t)(quarter * 32) << 16);
            if (p.epilogue == P_QKV) {
                if (w.t0 < p.T) qkv_heads_out(p, w, acc, row, staging, chunk_count, issuer, map_out, map_k, map_v, tables_held, held_cos, held_sin,
                                                 p.bias ? bias_s : nullptr);
            } else if (p.splits > 1) {
                split_stash(acc, row, smem);
            } else if (w.t0 < p.T) {
                if (p.epilogue == P_GATED) unit_out<false, true>(p, w, acc, row, staging, chunk_count, issuer, map_out, nullptr);
                else if (p.out_dt == F32) unit_out<true, false>(p, w, acc, row, staging, chunk_count, issuer, map_out, p.bias ? bias_s : nullptr);
                else unit_out<false, false>(p, w, acc, row, staging, chunk_count, issuer, map_out, p.bias ? bias_s : nullptr);
            }
            // this accumulator may be overwritten by the MMAs of the unit after next
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_in_cluster(tempty0 + 8u * b);
        }
        if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory stays valid until read
    }
    if (p.splits > 1) {
        // Every pair of the cluster has its share of the sums in its CTAs' shared memory (or has given up: the barrier is
        // met either way). Each pair then finishes its share of the tile's columns.
        __syncwarp();
        pair_barrier();
        if (warp >= 2) {
            const PairUnit w = pair_unit(p, pair, rank);            // one unit a cluster
            split_finish(p, w, warp == 2 && lane == 0, (warp & 3) * 32 + lane, rank, slice, smem, staging, map_out, *failed != 0);
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*failed && leader) {
        // the way out after a wait that ran out (drain.cuh): the copies asked for by both CTAs land (their bytes are
        // counted on the leader's barriers) and the MMAs issued finish before the pair meets below
        if (threadIdx.x == 0) {
            OutstandingFill left[8];
            const int n = outstanding_fills(fills_issued, fills_consumed, p.stages, left);
            for (int i = 0; i < n; ++i) mbar_wait_pair(&full_bar[left[i].stage], left[i].parity);
        }
        if (warp == 1 && lane == 0 && mmas_issued) {
            umma_commit_pair_local(drain_bar);
            mbar_wait(drain_bar, 0);
        }
        __syncthreads();
    }
    pair_barrier();
    tc_fence_after();
    if (warp == 1) tmem_dealloc_pair(tmem_base, tmem_cols);
}

// A [rows, K] row-major bfloat16 matrix, boxes of 64 rows x 64 elements, 128-byte swizzle; what lies outside reads as zero.
CUtensorMap pair_operand_map(const void* base, int rows, int K) {
    return tiled_map_2d("gemm_pair", CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, (uint64_t)K, (uint64_t)rows, (uint64_t)K * 2, kBlockK, kBoxRows,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}
// The [T, N] row-major output: boxes of 128 token rows x 128 bytes of features, 128-byte swizzle. Stores and adds
// outside the matrix are dropped.
CUtensorMap pair_out_map(void* base, int T, int N, DType dt) {
    const size_t elem_bytes = dt == F32 ? 4 : 2;
    return tiled_map_2d("gemm_pair", dt == F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, (uint64_t)N,
                        (uint64_t)T, (uint64_t)N * elem_bytes, (uint32_t)(128 / elem_bytes), kRows, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE);
}

int pair_sm_count() {
    static int count = 0;
    if (!count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
        if (count <= 0) count = 148;
    }
    return count;
}

// How many clusters of `size` CTAs with this much shared memory the GPU runs at once.
int pair_clusters_at_once(int size, size_t smem) {
    struct Known { int size; size_t smem; int clusters; };
    static std::mutex lock;
    static Known known[8];
    static int n_known = 0;
    std::lock_guard<std::mutex> hold(lock);
    for (int i = 0; i < n_known; ++i)
        if (known[i].size == size && known[i].smem == smem) return known[i].clusters;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(size, 1, 1);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    if (n_known < 8) known[n_known++] = {size, smem, n};
    return n;
}

bool g_pair_enabled = true;

}  // namespace

void gemm_pair_enable(bool on) { g_pair_enabled = on; }

bool gemm_pair_takes(const void* x, const void* w, const void* out, DType out_dt, int T, int N, int K, int mode) {
    const int epilogue = mode & 0xff;
    if (!g_pair_enabled || T < (epilogue == P_GATED ? kPairMinTokensGated : kPairMinTokens) || N <= 0 || K <= 0 || K % 8) return false;
    if (epilogue != P_STORE && epilogue != P_ACCUM && epilogue != P_GATED) return false;
    if (epilogue == P_ACCUM && out_dt != F32) return false;
    if (epilogue == P_GATED && out_dt != BF16) return false;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return false;
    return ((size_t)N * (out_dt == F32 ? 4 : 2)) % 16 == 0;        // TMA addresses the output's rows
}

void gemm_pair(const void* x, const void* w, const void* bias, DType bias_dt, void* out, DType out_dt, int T, int N, int K,
               int mode, int up_offset, int* error, cudaStream_t stream) {
    if (!gemm_pair_takes(x, w, out, out_dt, T, N, K, mode))
        throw std::invalid_argument("gemm_pair: this product is not one the two-CTA kernel takes (" + std::to_string(T) + " tokens, N = " +
                                    std::to_string(N) + ", K = " + std::to_string(K) + ", mode " + std::to_string(mode & 0xff) + ")");
    PairParams p{};
    p.T = T; p.N = N; p.K = K;
    p.epilogue = mode & 0xff;
    p.act = mode >> 8;
    if (p.act < 0 || p.act >= ACT_COUNT) throw std::invalid_argument("gemm_pair: unknown activation " + std::to_string(p.act));
    const int pairs_on_gpu = pair_sm_count() / 2;
    const int tiles_t = (T + 2 * kRows - 1) / (2 * kRows);
    if (p.epilogue == P_GATED) {
        p.tile_f = 256;                  // 128 gate rows and their 128 up rows
        p.tiles_f = (N + 127) / 128;
    } else {
        // 256 features a tile where that still gives every pair a unit, else 128
        p.tile_f = ((N + 255) / 256) * tiles_t >= pairs_on_gpu ? 256 : 128;
        p.tiles_f = (N + p.tile_f - 1) / p.tile_f;
    }
    p.half = p.tile_f / 2;
    p.up_offset = up_offset;
    p.bias = bias; p.bias_dt = bias_dt;
    p.out_dt = out_dt;
    p.error = error;
    p.units = p.tiles_f * tiles_t;
    const int stage_bytes = kRows * kStageK * 2 + p.half * kStageK * 2;
    const int budget = 227 * 1024 - 1024 - 2 * kStagingBytes - 256 - kBiasBytes;
    p.stages = budget / stage_bytes;
    if (p.stages > 8) p.stages = 8;
    const size_t smem = (size_t)p.stages * stage_bytes + 1024 /*alignment*/ + 2 * kStagingBytes + 256 /*barriers*/ + kBiasBytes;
    const CUtensorMap map_w = pair_operand_map(w, p.epilogue == P_GATED ? up_offset + N : N, K);
    const CUtensorMap map_x = pair_operand_map(x, T, K);
    const CUtensorMap map_out = pair_out_map(out, T, N, out_dt);
    static std::once_flag attr_once;
    std::call_once(attr_once, [] {
        cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    });
    // A "+=" product with few tiles and a long K (the down product of a prompt of a few hundred tokens: 7 to 35 tiles for
    // 74 pairs, each streaming all of K at what one SM takes from L2): the pairs of a cluster share a tile's K and add
    // their sums up through distributed shared memory, in a fixed order.
    const int kb_total = (K + kStageK - 1) / kStageK;
    p.splits = 1;
    p.kb_per = kb_total;
    if (p.epilogue == P_ACCUM && p.tile_f == 128) {
        for (int s = kPairMaxSplits; s >= 2; s >>= 1)
            if (p.units * s <= pairs_on_gpu && kb_total >= 4 * s && p.units <= pair_clusters_at_once(2 * s, smem)) {
                p.splits = s;
                p.kb_per = (kb_total + s - 1) / s;
                break;
            }
    }
    const int pairs = p.splits > 1 ? p.units : (p.units < pairs_on_gpu ? p.units : pairs_on_gpu);
    launch_kernel("gemm_pair", gemm_pair_kernel, dim3(2 * p.splits * pairs), dim3(kThreads), smem, stream, 2 * p.splits,
                  dependent_launch_enabled(), map_w, map_x, map_out, map_out, map_out, p);
    note_launch(1);
}

bool gemm_pair_qkv(const void* x, const void* w, const void* bias, DType bias_dt, int T, int K, const PairRope& rope, int* error,
                   cudaStream_t stream) {
    const int N = (rope.heads + 2 * rope.kv_heads) * rope.head_dim;
    if (!g_pair_enabled || T < kPairMinTokens || K <= 0 || K % 8 || rope.heads <= 0 || rope.kv_heads < 0) return false;
    if (rope.head_dim != 64 && rope.head_dim != 128) return false;      // whole heads per 128 columns, 128 bytes a piece of a row
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)rope.q_out | (uintptr_t)rope.k_packed | (uintptr_t)rope.v_packed |
         (uintptr_t)rope.k_pool | (uintptr_t)rope.v_pool | (uintptr_t)rope.cos_table | (uintptr_t)rope.sin_table) & 15)
        return false;
    if ((rope.k_packed == nullptr) != (rope.v_packed == nullptr) || (rope.k_pool == nullptr) != (rope.v_pool == nullptr)) return false;
    PairParams p{};
    p.T = T; p.N = N; p.K = K;
    p.epilogue = P_QKV;
    p.tile_f = 128;
    p.half = 64;
    p.tiles_f = (N + 127) / 128;
    p.bias = bias; p.bias_dt = bias_dt;
    p.out_dt = BF16;
    p.error = error;
    p.rope = rope;
    p.units = p.tiles_f * ((T + 2 * kRows - 1) / (2 * kRows));
    p.splits = 1;
    p.kb_per = (K + kStageK - 1) / kStageK;
    const int stage_bytes = kRows * kStageK * 2 + p.half * kStageK * 2;
    const int budget = 227 * 1024 - 1024 - 2 * kStagingBytes - 256 - kBiasBytes;
    p.stages = budget / stage_bytes;
    if (p.stages > 8) p.stages = 8;
    const size_t smem = (size_t)p.stages * stage_bytes + 1024 /*alignment*/ + 2 * kStagingBytes + 256 /*barriers*/ + kBiasBytes;
    const CUtensorMap map_w = pair_operand_map(w, N, K);
    const CUtensorMap map_x = pair_operand_map(x, T, K);
    const CUtensorMap map_q = pair_out_map(rope.q_out, T, rope.heads * rope.head_dim, BF16);
    const bool packed = rope.k_packed != nullptr && rope.kv_heads > 0;
    const CUtensorMap map_k = packed ? pair_out_map(rope.k_packed, T, rope.kv_heads * rope.head_dim, BF16) : map_q;
    const CUtensorMap map_v = packed ? pair_out_map(rope.v_packed, T, rope.kv_heads * rope.head_dim, BF16) : map_q;
    static std::once_flag attr_once;
    std::call_once(attr_once, [] {
        cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    });
    const int pairs_on_gpu = pair_sm_count() / 2;
    const int pairs = p.units < pairs_on_gpu ? p.units : pairs_on_gpu;
    launch_kernel("gemm_pair", gemm_pair_kernel, dim3(2 * pairs), dim3(kThreads), smem, stream, 2, dependent_launch_enabled(), map_w,
                  map_x, map_q, map_k, map_v, p);
    note_launch(1);
    return true;
}

}  // namespace sm
