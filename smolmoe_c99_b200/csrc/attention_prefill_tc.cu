// Causal attention of whole prompts over their own keys for bfloat16 (prefill) on the
// 5th-generation tensor cores: the same result as attention_prefill.cu (packed sequences of
// unequal lengths, grouped heads, optional window, running softmax in float; the reference
// scans [start, pos] per query and head: src/model.c:459-491, src/kernels.c:1156-1176), for
// head sizes 64 and 128.
//
// One CTA per (tile of 128 queries of one sequence, head): 256 threads, two to a query row, and a ninth warp whose
// first thread issues the copies and the MMAs. Q, and tiles of 128 keys and values, come into shared memory by TMA
// (128-byte swizzle). A row's two threads are two streams of their own over the keys: thread `half` takes keys
// 64 * half .. 64 * half + 63 of every tile, with a reference maximum, a sum and an output accumulator of its own, and
// the two are put together once, after the last tile. For every key tile:
//   S = Q K^T   tcgen05.mma 128 x 128 x head_dim, both operands K-major, S (float) in tensor memory;
//   each thread reads its 64 scores (its lane of tensor memory) with tcgen05.ld, masks them and writes
//   P = exp2(S * scale - reference) as bfloat16 into shared memory in the swizzled K-major layout an MMA operand needs;
//   O_half += P_half V_half   tcgen05.mma 128 x head_dim x 64 with V as it lies in memory ([key][dim], the "MN-major"
//   operand form), accumulating over the tiles in tensor memory, one accumulator per stream.
// The reference is lazy: it moves only when a tile's maximum exceeds it by more than 2^8 (P then stays below 256, and the
// float sums have room); only then do the threads of that warp read their accumulators, rescale them and write them
// back (tcgen05.st) before P is handed over. So a tile's chain is: scores, maximum, exponentials, P; nothing is read
// back from the PV product and the row's threads exchange nothing until the end.
// The row threads and the issuing thread meet only at mbarriers: S of the next tile is issued as soon as the rows of
// this one are in registers, and PV runs under the next tile's arithmetic.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in *error and the
// CTA leaves without writing.
#include <math_constants.h>

#include <stdexcept>
#include <string>

#include "common.cuh"
#include "drain.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "tcgen05.cuh"

namespace sm {

namespace {

using namespace tc5;

constexpr int kBM = 128, kBN = 128;
constexpr int kRowThreads = 256;      // two threads per query row (warps w and w + 4 share the rows of lane quarter w)
constexpr int kIssueWarp = 8;         // the warp whose first thread issues copies and MMAs (and which owns tensor memory)
constexpr int kThreads = kRowThreads + 32;
constexpr int kSmCount = 148;            // for the choice between the kernel's two variants only
constexpr int kBlockBytes = 128 * 128;      // 128 rows of 128 bytes: one swizzled block of 64 bfloat16 columns

// Key tiles, and value tiles, in shared memory. One CTA an SM: what fits beside Q and P (four and four at head
// size 64, two and two at 128). Two CTAs an SM (`two`, head size 64 only): one key stage and two value stages,
// 100 KB a CTA.
__host__ __device__ constexpr int key_stages(int head_dim, bool two) { return two ? 1 : (head_dim == 64 ? 4 : 2); }
__host__ __device__ constexpr int value_stages(int head_dim, bool two) { return two ? 2 : (head_dim == 64 ? 4 : 2); }

struct PrefillTcArgs {
    __nv_bfloat16* out;       // [T, heads, HD]
    const int32_t* tiles;     // [n_tiles, 3]: packed index of the sequence's first token, its length, first query (tiles of 64)
                              // over the cache [n_tiles, 5]: ... of the step's tokens, then the position of the step's first
                              // token and the sequence's slot
    int heads, kv_heads, window;
    float scale_log2;         // scale * log2(e)
    int* error;
    const int32_t* page_table;    // over the cache: [slots][table_stride]
    int table_stride;
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

// TWO: the variant of which two CTAs share an SM (fewer registers and stages; scores read 32 at a time, in two
// passes). It wins when every SM has many more key tiles to do than the longest chain of one CTA (long prompts):
// one CTA's waits are then the other's work. With few tiles an SM (2,048 tokens) the launch waits for the
// longest chain, which a second CTA on its SM only slows.
// CACHED: the sequences go on from the cache, which holds the step's own keys and values too (the q/k/v epilogue wrote
// them): keys and values come from the paged pools, a tile of 128 positions as the two pages that hold them (the tensor
// maps are over the pools, boxes of one page of one kv head), and a query sees the positions up to its own.
template <int HD, bool TWO, bool CACHED>
__global__ void __launch_bounds__(kThreads, TWO ? 2 : 1) prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                        const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v,
                                                                        PrefillTcArgs a) {
    constexpr int DB = HD / 64;                       // blocks of 64 columns of the head dimension
    constexpr int kQBytes = DB * kBlockBytes;         // Q tile, and one K or V tile
    constexpr int NSK = key_stages(HD, TWO), NSV = value_stages(HD, TWO);
    constexpr uint32_t kTmemCols = HD == 64 ? 256 : 512;   // S: 128 columns, then one output accumulator of HD columns per stream
    constexpr int PB = (HD == 64 && !TWO) ? 2 : 1;    // buffers of P: with two, P of a tile is written while PV of the tile before reads its own
    // CTAs start in the order of their index, the heads of one tile together: late tiles (most keys) first, so that
    // the longest chains of key tiles begin at once and the short ones fill the SMs that become free
    const int tile = (int)gridDim.y - 1 - (int)blockIdx.y, h = blockIdx.x;
    pdl_launch_dependents();
    constexpr int TW = CACHED ? 5 : 3;
    // seq_len: the sequence's tokens in this step; pos0: the position of the first of them (0 without a cache)
    const int seq_start = a.tiles[TW * tile], seq_len = a.tiles[TW * tile + 1], q0 = a.tiles[TW * tile + 2];
    const int pos0 = CACHED ? a.tiles[TW * tile + 3] : 0, slot = CACHED ? a.tiles[TW * tile + 4] : 0;
    if (q0 % kBM) return;                             // the second half of a tile of 128 queries
    const int kvh = h / (a.heads / a.kv_heads);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;                              // [DB][128 queries][128 B]
    uint8_t* k_s = q_s + kQBytes;                     // NSK x [DB][128 keys][128 B]
    uint8_t* v_s = k_s + NSK * kQBytes;               // NSV x [DB][128 keys][128 B]
    uint8_t* p_s = v_s + NSV * kQBytes;               // [PB][2][128 queries][128 B]: keys 0-63 and 64-127 of the tile
    uint64_t* bars = (uint64_t*)(p_s + PB * 2 * kBlockBytes);
    uint64_t* q_bar = bars;                           // Q has landed
    uint64_t* s_full = bars + 1;                      // the MMAs of S are done
    uint64_t* s_free = bars + 2;                      // all rows of S are in registers
    uint64_t* p_full = bars + 3;                      // all rows of P are in shared memory (and PV of the tile before is read)
    // the MMAs of PV of tile t are done: two barriers, for even and odd tiles, so that a wait for the tile before the
    // last one issued can be told from a wait for the last
    auto pv_bar = [&](int t) { return (t & 1) ? bars + 19 : bars + 4; };
    auto pv_parity = [](int t) { return (uint32_t)(t >> 1) & 1u; };
    uint64_t* pair_bar = bars + 5;                    // [4] the two warps of a lane quarter have both written their streams' figures
    uint64_t* k_bar = bars + 9;                       // [NSK] a key tile has landed
    uint64_t* v_bar = bars + 9 + NSK;                 // [NSV] a value tile has landed
    uint64_t* drain_bar = bars + 17;                  // a commit behind the last MMA, on the way out after a failure (NSK + NSV <= 8)
    uint32_t* tmem_slot = (uint32_t*)(bars + 18);
    volatile int* failed = (volatile int*)(tmem_slot + 1);
    float* half_max = (float*)(bars + 20);            // [2 streams][128 rows]: the streams' references, at the end
    float* half_sum = half_max + 512;                 // [2 streams][128 rows]: their sums

    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        mbar_init(q_bar, 1);
        for (int i = 0; i < NSK; ++i) mbar_init(&k_bar[i], 1);
        for (int i = 0; i < NSV; ++i) mbar_init(&v_bar[i], 1);
        mbar_init(s_full, 1);
        mbar_init(s_free, kRowThreads);
        mbar_init(p_full, kRowThreads);
        mbar_init(pv_bar(0), 1);
        mbar_init(pv_bar(1), 1);
        mbar_init(drain_bar, 1);
        for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 64);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kIssueWarp) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + 128;
    pdl_wait();   // q, k and v come from the kernel before; the tiles' list was written before the step's first kernel

    // key tiles this query tile sees (positions of the sequence, from 0)
    const int q_last = pos0 + min(q0 + kBM, seq_len) - 1;
    const int first_key = a.window > 0 ? max(0, pos0 + q0 - a.window + 1) : 0;
    const int kt0 = first_key / kBN;
    const int n_kt = q_last / kBN - kt0 + 1;
    const int last_page = (pos0 + seq_len - 1) / kPageSize;       // the last page the sequence holds
    auto fail = [&](int code) {
        *failed = 1;
        if (a.error) atomicExch(a.error, code);
    };

    if (warp == kIssueWarp) {
        // ---- one thread issues the copies and the MMAs ----------------------------------------------------
        if ((threadIdx.x & 31) == 0) {
            const uint32_t idesc_s = instr_desc(kBM, kBN);
            const uint32_t idesc_pv = instr_desc(kBM, HD) | (1u << 16);   // B (= V) is MN-major
            // key (value) tile t, counted from kt0, lives in stage t % NSK (NSV); its barrier has parity (t / NSK) & 1
            // key and value tiles asked for / waited for so far, and whether any MMA was issued: what the way out after
            // a wait that ran out has to let finish (drain.cuh)
            int k_issued = 0, k_waited = 0, v_issued = 0, v_waited = 0;
            bool q_waited = false, any_mma = false;
            // Over the cache a tile is the two pages of its 128 positions, each one box (64 rows of one kv head); a page the
            // sequence does not hold yet is replaced by its last one (its rows are masked, but must be numbers).
            auto pool_row = [&](int t, int half) {
                const int page = min(2 * (kt0 + t) + half, last_page);
                return (a.page_table[(size_t)slot * a.table_stride + page] * a.kv_heads + kvh) * kPageSize;
            };
            auto load_k = [&](int t) {
                uint8_t* dst = k_s + (size_t)(t % NSK) * kQBytes;
                ++k_issued;
                mbar_expect_tx(&k_bar[t % NSK], (uint32_t)kQBytes);
#pragma unroll
                for (int b = 0; b < DB; ++b) {
                    if (CACHED) {
                        tma_load_2d(dst + b * kBlockBytes, &map_k, b * 64, pool_row(t, 0), &k_bar[t % NSK]);
                        tma_load_2d(dst + b * kBlockBytes + kBlockBytes / 2, &map_k, b * 64, pool_row(t, 1), &k_bar[t % NSK]);
                    } else {
                        tma_load_2d(dst + b * kBlockBytes, &map_k, kvh * HD + b * 64, seq_start + (kt0 + t) * kBN, &k_bar[t % NSK]);
                    }
                }
            };
            auto load_v = [&](int t) {
                uint8_t* dst = v_s + (size_t)(t % NSV) * kQBytes;
                ++v_issued;
                mbar_expect_tx(&v_bar[t % NSV], (uint32_t)kQBytes);
#pragma unroll
                for (int b = 0; b < DB; ++b) {
                    if (CACHED) {
                        tma_load_2d(dst + b * kBlockBytes, &map_v, b * 64, pool_row(t, 0), &v_bar[t % NSV]);
                        tma_load_2d(dst + b * kBlockBytes + kBlockBytes / 2, &map_v, b * 64, pool_row(t, 1), &v_bar[t % NSV]);
                    } else {
                        tma_load_2d(dst + b * kBlockBytes, &map_v, kvh * HD + b * 64, seq_start + (kt0 + t) * kBN, &v_bar[t % NSV]);
                    }
                }
            };
            // The descriptors of a tile's k-steps differ in the start address only (bits 0-13, in units of 16 bytes):
            // built once, then advanced by an addition; this thread has nobody to hide its arithmetic behind.
            const uint64_t desc_q = smem_desc(smem_u32(q_s)), desc_k0 = smem_desc(smem_u32(k_s));
            const uint64_t desc_p = smem_desc(smem_u32(p_s)), desc_v0 = smem_desc_mn(smem_u32(v_s), kBlockBytes, 1024);
            auto issue_s = [&](int t) {     // S = Q K^T for key tile t
                const uint64_t desc_k = desc_k0 + (uint64_t)(((uint32_t)(t % NSK) * kQBytes) >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint64_t off = (uint64_t)(((uint32_t)(ks / 4) * kBlockBytes + (uint32_t)(ks % 4) * 32) >> 4);
                    umma_bf16(tmem_s, desc_q + off, desc_k + off, idesc_s, ks > 0 ? 1u : 0u);
                }
                umma_commit(s_full);
            };
            auto issue_pv = [&](int t) {    // O_half += P_half V_half for tile t, whose P lies in shared memory
                const uint64_t desc_v = desc_v0 + (uint64_t)(((uint32_t)(t % NSV) * kQBytes) >> 4);
                const uint64_t desc_pt = desc_p + (uint64_t)(((uint32_t)(t % PB) * 2 * kBlockBytes) >> 4);
#pragma unroll
                for (int ks = 0; ks < kBN / 16; ++ks) {
                    const uint64_t p_off = (uint64_t)(((uint32_t)(ks / 4) * kBlockBytes + (uint32_t)(ks % 4) * 32) >> 4);
                    const uint64_t v_off = (uint64_t)(((uint32_t)ks * 16 * 128) >> 4);   // 16 keys of 128 bytes
                    umma_bf16(tmem_pv + (uint32_t)((ks / 4) * HD), desc_pt + p_off, desc_v + v_off, idesc_pv, (t > 0 || (ks % 4) > 0) ? 1u : 0u);
                }
                umma_commit(pv_bar(t));
            };
            mbar_expect_tx(q_bar, (uint32_t)kQBytes);
#pragma unroll
            for (int b = 0; b < DB; ++b) tma_load_2d(q_s + b * kBlockBytes, &map_q, h * HD + b * 64, seq_start + q0, q_bar);
            for (int t = 0; t < NSK && t < n_kt; ++t) load_k(t);
            for (int t = 0; t < NSV && t < n_kt; ++t) load_v(t);
            bool ok = (q_waited = mbar_wait(q_bar, 0)) && mbar_wait(&k_bar[0], 0);
            if (ok) {
                k_waited = 1;
                tc_fence_after();
                issue_s(0);
                any_mma = true;
            } else {
                fail(11);
            }
            for (int it = 0; it < n_kt && ok; ++it) {
                const uint32_t ph = (uint32_t)it & 1u;
                // S of tile it done: its key stage may take tile it + NSK (with one stage that is the next tile, so
                // it is asked for as early as this)
                if (!(ok = mbar_wait(s_full, ph))) { fail(21); break; }
                if (it + NSK < n_kt) load_k(it + NSK);
                // S of tile it is in the threads' registers: S of the next tile may overwrite it
                if (!(ok = mbar_wait(s_free, ph))) { fail(12); break; }
                tc_fence_after();
                if (it + 1 < n_kt) {
                    if (!(ok = mbar_wait(&k_bar[(it + 1) % NSK], (uint32_t)((it + 1) / NSK) & 1u))) { fail(13); break; }
                    k_waited = it + 2;
                    tc_fence_after();
                    issue_s(it + 1);
                }
                // P of tile it is in shared memory. Once PV of the tile before is done, that one's value stage may take
                // tile it - 1 + NSV.
                if (!(ok = mbar_wait(p_full, ph))) { fail(14); break; }
                if (it >= 1 && it - 1 + NSV < n_kt) {
                    if (!(ok = mbar_wait(pv_bar(it - 1), pv_parity(it - 1)))) { fail(22); break; }
                    load_v(it - 1 + NSV);
                }
                if (!(ok = mbar_wait(&v_bar[it % NSV], (uint32_t)(it / NSV) & 1u))) { fail(15); break; }
                v_waited = it + 1;
                tc_fence_after();
                issue_pv(it);
            }
            if (!ok || *failed) {
                // the way out: every tile asked for lands, every MMA issued finishes, before the CTA gives up its
                // shared and tensor memory
                OutstandingFill left[8];
                if (!q_waited) mbar_wait(q_bar, 0);
                int n = outstanding_fills(k_issued, k_waited, NSK, left);
                for (int i = 0; i < n; ++i) mbar_wait(&k_bar[left[i].stage], left[i].parity);
                n = outstanding_fills(v_issued, v_waited, NSV, left);
                for (int i = 0; i < n; ++i) mbar_wait(&v_bar[left[i].stage], left[i].parity);
                if (any_mma) {
                    umma_commit(drain_bar);
                    mbar_wait(drain_bar, 0);
                }
            }
        }
    } else {
        // ---- 256 threads, two per query row: its lane of tensor memory, and 64 of the tile's 128 keys ----------
        const int quarter = warp & 3, half = warp >> 2;
        const int row = quarter * 32 + (threadIdx.x & 31);
        const int qpos = pos0 + q0 + row;           // the query's position in its sequence
        const int seq_end = pos0 + seq_len;         // positions the sequence holds after this step
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        constexpr int OW = HD / 2;          // columns of the output this thread writes at the end
        constexpr float kLazy = 8.0f;       // the reference moves when a tile's maximum exceeds it by more than this (log2)
        const uint32_t tmem_o = tmem_pv + lane_base + (uint32_t)(half * HD);    // this stream's output accumulator
        float m = -CUDART_INF_F, l = 0.f;   // the stream's reference maximum, and the sum of its P against it
        bool ok = true;
        // After a tile's maximum is known: where any thread of the warp has to move its reference, every thread of the
        // warp does (tensor memory is read and written by whole warps), rescaling its sum and, from the second tile on,
        // its accumulator, which PV of the tile before has to have left alone by then.
        auto settle_reference = [&](int it, float mloc) {
            if (!__any_sync(0xffffffffu, mloc > m + kLazy)) return;
            const float mx = fmaxf(m, mloc);
            const float corr = mx == -CUDART_INF_F ? 1.0f : ex2_approx(m - mx);    // 0 for a stream that has seen no key yet
            if (it > 0) {
                if (!mbar_wait(pv_bar(it - 1), pv_parity(it - 1))) { fail(17); ok = false; return; }
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    float acc[32];
                    tmem_ld32(tmem_o + (uint32_t)(c * 32), acc);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] *= corr;
                    tmem_st32(tmem_o + (uint32_t)(c * 32), acc);
                }
            }
            l *= corr;
            m = mx;
        };

        for (int it = 0; it < n_kt && ok; ++it) {
            const int n0 = (kt0 + it) * kBN + half * 64;     // this thread's first key of the tile
            // every key of the tile visible to every query of the tile: no mask needed
            const int t0 = (kt0 + it) * kBN;
            const bool full = t0 + kBN - 1 <= pos0 + q0 && t0 + kBN - 1 < seq_end && (a.window <= 0 || t0 > pos0 + q0 + kBM - 1 - a.window);
            // otherwise this row sees the keys n0 + j with vis_lo <= j <= vis_hi
            const int vis_hi = min(qpos, seq_end - 1) - n0;
            const int vis_lo = a.window > 0 ? qpos - a.window + 1 - n0 : -(1 << 30);
            uint8_t* prow = p_s + (size_t)((it % PB) * 2 + half) * kBlockBytes + (size_t)row * 128;
            if (!mbar_wait(s_full, (uint32_t)it & 1u)) { fail(18); ok = false; break; }
            tc_fence_after();
            if constexpr (!TWO) {
                // this thread's 64 scores into registers; then S may be overwritten
                float sv[64];
                tmem_ld64(tmem_s + lane_base + (uint32_t)(half * 64), sv);
                tc_fence_before();
                mbar_arrive(s_free);
                if (!full) {
    #pragma unroll
                    for (int j = 0; j < 64; ++j)
                        if (j > vis_hi || j < vis_lo) sv[j] = -CUDART_INF_F;
                }
                // maximum of the raw scores (the scale is positive, so it can be applied afterwards); eight running
                // maxima and four running sums, not one chain of dependent instructions
                float raw8[8];
    #pragma unroll
                for (int e = 0; e < 8; ++e) raw8[e] = sv[e];
    #pragma unroll
                for (int j = 8; j + 8 < 64; j += 16)
    #pragma unroll
                    for (int e = 0; e < 8; ++e) raw8[e] = fmax3(raw8[e], sv[j + e], sv[j + 8 + e]);
    #pragma unroll
                for (int e = 0; e < 8; ++e) raw8[e] = fmaxf(raw8[e], sv[56 + e]);
                const float raw = fmaxf(fmaxf(fmaxf(raw8[0], raw8[1]), fmaxf(raw8[2], raw8[3])),
                                        fmaxf(fmaxf(raw8[4], raw8[5]), fmaxf(raw8[6], raw8[7])));
                settle_reference(it, raw * a.scale_log2);
                if (!ok) break;
                // a stream that has seen no key yet keeps m = -inf; 0 as its reference avoids inf - inf
                const float ref = m == -CUDART_INF_F ? 0.f : m;
                // P = 2^(S * scale - reference) as bfloat16, and its sum
                // (the scaling and the sums two at a time, with the packed float instructions)
                uint32_t pk[32];
                const uint64_t scale2 = pack_f32x2(a.scale_log2, a.scale_log2), ref2 = pack_f32x2(-ref, -ref);
                uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};      // (the bits of two float zeros)
    #pragma unroll
                for (int j = 0; j < 64; j += 2) {
                    float x0, x1;
                    unpack_f32x2(fma_f32x2(pack_f32x2(sv[j], sv[j + 1]), scale2, ref2), x0, x1);
                    const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                    sum2[(j / 2) & 3] = add_f32x2(sum2[(j / 2) & 3], pack_f32x2(p0, p1));
                    pk[j / 2] = pack_bf16(p0, p1);
                }
                {
                    float lo, hi;
                    unpack_f32x2(add_f32x2(add_f32x2(sum2[0], sum2[1]), add_f32x2(sum2[2], sum2[3])), lo, hi);
                    l += lo + hi;
                }
                // this buffer of P was read by PV of tile it - PB
                if (it >= PB && !mbar_wait(pv_bar(it - PB), pv_parity(it - PB))) { fail(23); ok = false; break; }
                // this thread's 64 keys are block `half` of P: pieces of 8 keys (16 bytes), swizzled with the row
    #pragma unroll
                for (int piece = 0; piece < 8; ++piece)
                    *reinterpret_cast<uint4*>(prow + ((piece ^ (row & 7)) << 4)) =
                        make_uint4(pk[4 * piece], pk[4 * piece + 1], pk[4 * piece + 2], pk[4 * piece + 3]);
            } else {
                // This thread's 64 scores are read 32 at a time, in two passes (the maximum, then the exponentials):
                // holding all of them would leave too few registers for two CTAs on an SM.
                float sv[32];
                auto read_scores = [&](int part) {
                    tmem_ld32(tmem_s + lane_base + (uint32_t)(half * 64 + part * 32), sv);
                    if (!full) {
    #pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (part * 32 + j > vis_hi || part * 32 + j < vis_lo) sv[j] = -CUDART_INF_F;
                    }
                };
                float raw8[8];
    #pragma unroll
                for (int e = 0; e < 8; ++e) raw8[e] = -CUDART_INF_F;
    #pragma unroll
                for (int part = 0; part < 2; ++part) {
                    read_scores(part);
    #pragma unroll
                    for (int j = 0; j < 32; j += 16)
    #pragma unroll
                        for (int e = 0; e < 8; ++e) raw8[e] = fmax3(raw8[e], sv[j + e], sv[j + 8 + e]);
                }
                const float raw = fmaxf(fmaxf(fmaxf(raw8[0], raw8[1]), fmaxf(raw8[2], raw8[3])),
                                        fmaxf(fmaxf(raw8[4], raw8[5]), fmaxf(raw8[6], raw8[7])));
                settle_reference(it, raw * a.scale_log2);
                if (!ok) break;
                const float ref = m == -CUDART_INF_F ? 0.f : m;
                // the one buffer of P was read by PV of the tile before
                if (it >= PB && !mbar_wait(pv_bar(it - PB), pv_parity(it - PB))) { fail(23); ok = false; break; }
                const uint64_t scale2 = pack_f32x2(a.scale_log2, a.scale_log2), ref2 = pack_f32x2(-ref, -ref);
                uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};      // (the bits of two float zeros)
    #pragma unroll
                for (int part = 0; part < 2; ++part) {
                    read_scores(part);
                    if (part == 1) {   // S is in registers for the last time: it may be overwritten
                        tc_fence_before();
                        mbar_arrive(s_free);
                    }
    #pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t pk[4];
    #pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float x0, x1;
                            unpack_f32x2(fma_f32x2(pack_f32x2(sv[c * 8 + 2 * e], sv[c * 8 + 2 * e + 1]), scale2, ref2), x0, x1);
                            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                            sum2[e] = add_f32x2(sum2[e], pack_f32x2(p0, p1));
                            pk[e] = pack_bf16(p0, p1);
                        }
                        const int piece = part * 4 + c;
                        *reinterpret_cast<uint4*>(prow + ((piece ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                {
                    float lo, hi;
                    unpack_f32x2(add_f32x2(add_f32x2(sum2[0], sum2[1]), add_f32x2(sum2[2], sum2[3])), lo, hi);
                    l += lo + hi;
                }
            }
            // P is written (and a moved reference's accumulator is back in tensor memory): make it visible to the tensor
            // core's reads, then tell the issuing thread
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            mbar_arrive(p_full);
        }
        // The two streams of a row put together: their references and sums through shared memory, their accumulators read
        // from tensor memory by both threads, each for its half of the output's columns.
        half_max[half * 128 + row] = m;
        half_sum[half * 128 + row] = l;
        mbar_arrive(&pair_bar[quarter]);
        if (!mbar_wait(&pair_bar[quarter], 0)) { fail(20); ok = false; }
        if (ok && n_kt > 0 && !mbar_wait(pv_bar(n_kt - 1), pv_parity(n_kt - 1))) { fail(17); ok = false; }
        tc_fence_after();
        if (__all_sync(0xffffffffu, ok && !*failed)) {
            const float m_other = half_max[(half ^ 1) * 128 + row], l_other = half_sum[(half ^ 1) * 128 + row];
            const float top = fmaxf(m, m_other);
            const float w_mine = m == -CUDART_INF_F ? 0.f : ex2_approx(m - top);
            const float w_other = m_other == -CUDART_INF_F ? 0.f : ex2_approx(m_other - top);
            const float sum = l * w_mine + l_other * w_other;
            const float inv = sum > 0.f ? 1.0f / sum : 0.f;
            const float w0 = (half == 0 ? w_mine : w_other) * inv, w1 = (half == 0 ? w_other : w_mine) * inv;   // streams 0 and 1
            const bool live = q0 + row < seq_len;
            __nv_bfloat16* orow = a.out + ((size_t)(seq_start + q0 + row) * a.heads + h) * HD + half * OW;
#pragma unroll
            for (int c = 0; c < OW / 32; ++c) {
                float o0[32], o1[32];
                tmem_ld32(tmem_pv + lane_base + (uint32_t)(half * OW + c * 32), o0);
                tmem_ld32(tmem_pv + lane_base + (uint32_t)(HD + half * OW + c * 32), o1);
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float r[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) r[e] = o0[i + e] * w0 + o1[i + e] * w1;
                        *reinterpret_cast<uint4*>(orow + c * 32 + i) =
                            make_uint4(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]), pack_bf16(r[4], r[5]), pack_bf16(r[6], r[7]));
                    }
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == kIssueWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// A [T, width] row-major bfloat16 matrix, boxes of 128 rows x 64 elements, 128-byte swizzle; rows and columns
// outside the matrix read as zero.
CUtensorMap make_map(const void* base, int T, int width) {
    return tiled_map_2d("attention_prefill_tc", CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, (uint64_t)width, (uint64_t)T, (uint64_t)width * 2,
                        64, 128, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

template <int HD, bool TWO, bool CACHED = false>
void launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillTcArgs& a, int n_tiles,
            cudaStream_t stream) {
    constexpr int DB = HD / 64;
    // alignment; Q, the stages of K and V, P; barriers; maxima and sums
    const int p_buffers = (HD == 64 && !TWO) ? 2 : 1;
    const size_t smem = 1024 + (size_t)((1 + key_stages(HD, TWO) + value_stages(HD, TWO)) * DB + 2 * p_buffers) * kBlockBytes + 160 +
                        3 * 256 * sizeof(float);
    auto kernel = prefill_attention_tc_kernel<HD, TWO, CACHED>;
    static bool prepared = false;
    if (!prepared) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) throw std::runtime_error(std::string("attention_prefill_tc: ") + cudaGetErrorString(e));
        prepared = true;
    }
    launch_kernel("attention_prefill_tc", kernel, dim3(a.heads, n_tiles), dim3(kThreads), smem, stream, 1, dependent_launch_enabled(), mq, mk, mv, a);
}

}  // namespace

bool attention_prefill_tc_supports(int heads, int kv_heads, int head_dim) {
    return (head_dim == 64 || head_dim == 128) && kv_heads > 0 && heads % kv_heads == 0;
}

void attention_prefill_tc(const void* q, const void* k, const void* v, void* out, const int32_t* tiles, int n_tiles, int T,
                          int heads, int kv_heads, int head_dim, float scale, int window, int longest, int variant,
                          int* error, cudaStream_t stream) {
    if (n_tiles <= 0) return;
    if (!attention_prefill_tc_supports(heads, kv_heads, head_dim))
        throw std::invalid_argument("attention_prefill_tc: head_dim " + std::to_string(head_dim) +
                                    " is not 64 or 128 (the mma.sync kernel takes multiples of 16 up to 128)");
    if (n_tiles > 65535) throw std::invalid_argument("attention_prefill_tc: more than 65535 tiles of 64 queries");
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
        throw std::invalid_argument("attention_prefill_tc: operands must be 16-byte aligned");
    const CUtensorMap mq = make_map(q, T, heads * head_dim);
    const CUtensorMap mk = make_map(k, T, kv_heads * head_dim);
    const CUtensorMap mv = make_map(v, T, kv_heads * head_dim);
    PrefillTcArgs a{(__nv_bfloat16*)out, tiles, heads, kv_heads, window, scale * 1.4426950408889634f, error, nullptr, 0};
    note_launch();
    if (head_dim == 128) {
        launch<128, false>(mq, mk, mv, a, n_tiles, stream);
        return;
    }
    bool two = variant == 1;
    if (variant < 0) {
        // Two CTAs an SM when every SM has at least as many key tiles to do as the longest chain of one CTA has
        // (estimated as if every sequence were as long as the longest). Measured on a B200, 14 heads of 64, one
        // CTA against two: one prompt of 2,048 tokens 28.1 / 35.0 us, of 4,096 86 / 66, of 8,192 286 / 206, of
        // 16,384 1,047 / 745 (645 TFLOP/s); eight prompts of 2,048 198 / 146; four of 1,024 37 / 34.
        const long long chain = ((longest > 0 && longest < T ? longest : T) + kBN - 1) / kBN;
        const long long total = (long long)heads * ((T + kBM - 1) / kBM) * (chain + 1) / 2;
        two = total >= chain * kSmCount;
    }
    if (two) launch<64, true>(mq, mk, mv, a, n_tiles, stream);
    else launch<64, false>(mq, mk, mv, a, n_tiles, stream);
}


bool attention_extend_tc_supports(int heads, int kv_heads, int head_dim, long long pool_pages) {
    return attention_prefill_tc_supports(heads, kv_heads, head_dim) && pool_pages > 0 &&
           pool_pages * kv_heads * kPageSize < (1ll << 31);
}

void attention_extend_tc(const void* q, void* out, const int32_t* tiles, int n_tiles, int T, int heads, int kv_heads, int head_dim,
                         float scale, int window, const void* k_pool, const void* v_pool, const int32_t* page_table,
                         int table_stride, long long pool_pages, int longest, int variant, int* error, cudaStream_t stream) {
    if (n_tiles <= 0) return;
    if (!attention_extend_tc_supports(heads, kv_heads, head_dim, pool_pages))
        throw std::invalid_argument("attention_extend_tc: head_dim " + std::to_string(head_dim) + " is not 64 or 128, or the pool has too many rows for a tensor map");
    if (n_tiles > 65535) throw std::invalid_argument("attention_extend_tc: more than 65535 tiles of 64 queries");
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15)
        throw std::invalid_argument("attention_extend_tc: operands must be 16-byte aligned");
    const CUtensorMap mq = make_map(q, T, heads * head_dim);
    // the pools [pages, kv heads, 64 positions, head_dim] as rows of head_dim: a box is one page of one kv head, 64 columns wide
    const uint64_t rows = (uint64_t)pool_pages * kv_heads * kPageSize;
    const CUtensorMap mk = tiled_map_2d("attention_extend_tc", CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, k_pool, (uint64_t)head_dim, rows,
                                        (uint64_t)head_dim * 2, 64, kPageSize, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    const CUtensorMap mv = tiled_map_2d("attention_extend_tc", CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, v_pool, (uint64_t)head_dim, rows,
                                        (uint64_t)head_dim * 2, 64, kPageSize, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    PrefillTcArgs a{(__nv_bfloat16*)out, tiles, heads, kv_heads, window, scale * 1.4426950408889634f, error, page_table, table_stride};
    note_launch();
    if (head_dim == 128) {
        launch<128, false, true>(mq, mk, mv, a, n_tiles, stream);
        return;
    }
    bool two = variant == 1;
    if (variant < 0) {
        // (as in attention_prefill_tc: two CTAs an SM where every SM has at least as many key tiles to do as the longest chain;
        // the query tiles' chains are estimated as those of one sequence that ends at `longest`: chain, chain - 1, ...)
        const long long chain = ((longest > 0 ? longest : T) + kBN - 1) / kBN;
        const long long q_tiles = (T + kBM - 1) / kBM;
        const long long shortest = chain - q_tiles + 1 > 1 ? chain - q_tiles + 1 : 1;
        const long long total = (long long)heads * q_tiles * (chain + shortest) / 2;
        two = total >= chain * kSmCount;
    }
    if (two) launch<64, true, true>(mq, mk, mv, a, n_tiles, stream);
    else launch<64, false, true>(mq, mk, mv, a, n_tiles, stream);
}

}  // namespace sm
