// One decode step of a whole stack of standard decoder layers in ONE persistent kernel, for up to 16
// sequences that each go on by one token (bfloat16 weights and cache).
//
// Launched kernel by kernel, a decode step of a 24-layer model is a chain of ~120 dependent launches
// of a few microseconds each, and every one of them starts asking for its weights only when the one
// before has drained. Here one CTA per SM stays resident for the whole step. The phases of the step
// (per layer: q/k/v with norm, bias, rotation and cache write | attention over the cache | output
// projection into the residual | gate/up with norm and SwiGLU | down projection into the residual; then
// final norm and output head) are separated by a grid-wide barrier, and the weights do not wait for
// those barriers: every warp owns a ring in shared memory and keeps TMA tensor copies
// (cp.async.bulk.tensor) of ITS share of the weights of this and the coming phases in flight, in the
// fixed order in which it will use them. So HBM streams for the whole step while the phases' short
// dependent chains (stage x, multiply, reduce, write, barrier) run on top. A copy brings 8 weight rows
// by a run of 64-element blocks of K (a 3-dimensional tensor map over [rows][K / 64][64], 128-byte
// swizzle, so that the tensor-core loads meet no bank conflicts): few, large copies, since the copy
// engine's time goes by the copy, not by the byte.
//
// Work of a product: units of 8 weight rows (for gate/up 8 gate rows and their 8 up rows; for q and k
// 8 dimensions and their 8 rotation partners) are shared out evenly over the CTAs; inside a CTA the
// units go round-robin over the warps, and where a CTA has fewer units than warps, 2, 4 or 8 warps
// split a unit's K and add their sums up in warp order. Tokens are the 16 rows of the tensor-core
// tile (mma.sync m16n8k16), the 8 weight rows its columns. Every sum is formed in an order that
// depends only on the sizes, never on timing. The math is that of the separate kernels
// (src/model.c:493-542,625-650,654-662 of the reference; softmax and norms in float).
//
// Attention: every (sequence, kv head) is cut along its positions into as many parts as there are
// CTAs to go round; a CTA's 8 warps take tiles of 16 positions (bulk copies, two in flight per
// warp), merge in shared memory, and where a sequence has several parts the CTA that finishes last
// merges them in part order.
//
// Every wait (mbarrier, grid barrier) is bounded; when one runs out the CTA sets the error word and
// an abort flag that makes all others leave at their next barrier.
//
// Where it stands (B200, Qwen2.5-0.5B sizes, 8 sequences at 2,048 positions): correct against the separate
// kernels and the plain model, but a step takes 1.8 ms against their 0.69 ms, so it is off unless asked for
// (Ops.use_fused_decode). The weights do stream ahead (the output head runs at 4.9 TB/s); the time goes
// into the phases' own chains, which are latency-bound at one CTA of 8 warps an SM: staging x from L2 ~3 us a
// phase, the walk to the next piece up to 1-3 us where it crosses into another product, attention with its
// two barriers ~20 us, the epilogues' dependent loads 1-2 us, and a grid barrier ~1.3 us (measured alone). Each
// phase has to come down to ~3 us for the kernel to pass the separate kernels, whose own chain is already ~4.5 us
// a launch; profiles/decode_fused_b8_ctx2048.md has the stamps.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <mutex>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"

namespace sm {

namespace {

using tc5::bulk_load;
using tc5::mbar_expect_tx;
using tc5::mbar_init;
using tc5::mbar_try_wait;
using tc5::smem_u32;

constexpr int kWarps = 8, kThreads = kWarps * 32;
constexpr int kQueue = 8;                          // weight pieces a warp may have in flight (a barrier each)
constexpr int kWarpRing = 16384;                   // bytes of a warp's ring: pieces lie in it one after another
constexpr int kRingBytes = kWarps * kWarpRing;     // 128 KB
constexpr int kXBytes = 33024;                     // x of one chunk of K: 8 rows of 2048 + 8 or 16 rows of 1024 + 8 bfloat16
constexpr int kKvBytes = 63488;                    // attention tiles; partial sums of the products
constexpr int kFlexBytes = kXBytes + kKvBytes;     // attention uses both
constexpr int kBarBytes = kWarps * (kQueue + 2) * 8;   // the warps' barriers: kQueue for weights, 2 for attention tiles
constexpr int kSmemBytes = kRingBytes + kFlexBytes + kBarBytes + 1024;   // (+ 1024: the ring starts on a 1024-byte boundary)
constexpr int kBlockK = 64;                        // elements of K per block: a 128-byte swizzled row
constexpr int kMaxRounds = 2;                      // units a warp may hold sums of while K comes in several chunks
constexpr long long kWaitCycles = 4000000000ll;    // ~2 s: a wait this long is a fault, not a delay

enum Kind : int { K_QKV = 0, K_OUT = 1, K_GATE_UP = 2, K_DOWN = 3, K_HEAD = 4 };

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float bf(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// ---- the schedule: which weight bytes a warp needs, in the order it needs them ---------------------------------
struct Product {
    const CUtensorMap* map;
    int kind, K, units;       // units of 8 output rows (gate/up, and q and k: 8 + 8)
    int bk;                   // blocks of K a copy brings (the map's box)
    int hd, heads, kv_heads, H;
};

__device__ __forceinline__ Product product_of(const FusedArgs& a, int pi) {
    Product p;
    p.hd = a.head_dim; p.heads = a.heads; p.kv_heads = a.kv_heads; p.H = a.H;
    p.map = reinterpret_cast<const CUtensorMap*>(a.maps) + pi;
    if (pi >= 4 * a.n_layers) {
        p.kind = K_HEAD; p.K = a.D; p.units = (a.V + 7) / 8;
    } else {
        p.kind = pi & 3;
        if (p.kind == K_QKV) { p.K = a.D; p.units = (a.heads + a.kv_heads) * a.head_dim / 16 + a.kv_heads * a.head_dim / 8; }
        else if (p.kind == K_OUT) { p.K = a.heads * a.head_dim; p.units = (a.D + 7) / 8; }
        else if (p.kind == K_GATE_UP) { p.K = a.D; p.units = (a.H + 7) / 8; }
        else { p.K = a.H; p.units = (a.D + 7) / 8; }
    }
    p.bk = a.bk[p.kind];
    return p;
}
__device__ __forceinline__ int product_rows_total(const FusedArgs& a, const Product& p) {
    switch (p.kind) {
        case K_QKV: return (a.heads + 2 * a.kv_heads) * a.head_dim;
        case K_GATE_UP: return a.H;
        case K_HEAD: return a.V;
        default: return a.D;
    }
}
// The weight rows of a unit: one or two sets of 8 consecutive rows (gate and up; a q or k head's dimensions j*8..
// and their rotation partners half a head further on). Rows past the matrix read as zero.
struct UnitRows {
    int sets, row_a, row_b;
};
__device__ __forceinline__ UnitRows unit_rows(const Product& p, int unit) {
    UnitRows u{1, unit * 8, 0};
    if (p.kind == K_QKV) {
        const int per_head = p.hd / 16, rot_units = (p.heads + p.kv_heads) * per_head;
        if (unit < rot_units) {
            const int head = unit / per_head, j = unit - head * per_head;
            u.sets = 2; u.row_a = head * p.hd + j * 8; u.row_b = u.row_a + p.hd / 2;
        } else {
            u.row_a = (p.heads + p.kv_heads) * p.hd + (unit - rot_units) * 8;
        }
    } else if (p.kind == K_GATE_UP) {
        u.sets = 2; u.row_b = p.H + unit * 8;
    }
    return u;
}

// How one CTA's warps take a product.
struct Share {
    int u0, n_u;       // this CTA's units
    int wpu;           // warps per unit (1, 2, 4, 8)
    int per_round;     // units the CTA's warps work on at once
    int rounds;
    int chunk;         // k elements of x staged at once
    int n_chunks;
};
__device__ __forceinline__ Share share_of(const Product& p, int cta, int n_ctas, int tokp) {
    Share s;
    s.u0 = (int)(((unsigned)cta * (unsigned)p.units) / (unsigned)n_ctas);
    s.n_u = (int)(((unsigned)(cta + 1) * (unsigned)p.units) / (unsigned)n_ctas) - s.u0;
    s.wpu = s.n_u >= 5 ? 1 : (s.n_u >= 3 ? 2 : (s.n_u == 2 ? 4 : 8));
    s.per_round = kWarps / s.wpu;
    s.rounds = (s.n_u + s.per_round - 1) / s.per_round;
    s.chunk = tokp == 8 ? 2048 : 1024;
    s.n_chunks = (p.K + s.chunk - 1) / s.chunk;
    return s;
}
// The blocks of K (of kBlockK elements) of chunk `chunk` that warp slice `ksub` of `wpu` takes: [lo, hi), counted from the chunk's first.
__device__ __forceinline__ void warp_blocks(const Product& p, const Share& s, int chunk, int ksub, int& lo, int& hi) {
    const int first = chunk * (s.chunk / kBlockK), blocks = min(p.K / kBlockK, first + s.chunk / kBlockK) - first;
    const int per = (blocks + s.wpu - 1) / s.wpu;
    lo = min(blocks, ksub * per);
    hi = min(blocks, lo + per);
}

// A walk over a warp's pieces in the order of use: product, chunk of K, round (unit), piece. What depends only on the
// product or on the chunk is worked out when the walk enters it, so that a step inside a chunk is a few instructions
// (this runs once per copy on every warp: divisions here were a microsecond a piece).
struct Piece {
    bool valid;
    int unit, kb0, nkb;      // blocks of K [kb0, kb0 + nkb) of the matrix (the copy brings bk: the rest is not used)
    const CUtensorMap* map;
    int bk, sets, row_a, row_b;
};
struct Walker {
    int pi, chunk, round, piece;
    // of the product
    Product p;
    int u0, n_u, per_round, rounds, n_chunks, chunk_blocks, slot, ksub, wpu;
    // of the chunk
    int lo, pieces, span;
    bool in_product, in_chunk;

    __device__ void start() { pi = chunk = round = piece = 0; in_product = in_chunk = false; }

    __device__ Piece next(const FusedArgs& a, int cta, int n_ctas, int warp, int tokp) {
        Piece out;
        out.valid = false;
        const int n_products = 4 * a.n_layers + 1;
        while (pi < n_products) {
            if (!in_product) {
                p = product_of(a, pi);
                const Share s = share_of(p, cta, n_ctas, tokp);
                u0 = s.u0; n_u = s.n_u; per_round = s.per_round; rounds = s.rounds; n_chunks = s.n_chunks; wpu = s.wpu;
                chunk_blocks = s.chunk / kBlockK;
                slot = warp / s.wpu; ksub = warp % s.wpu;
                in_product = true;
                in_chunk = false;
            }
            while (chunk < n_chunks) {
                if (!in_chunk) {
                    const int first = chunk * chunk_blocks, blocks = min(p.K / kBlockK, first + chunk_blocks) - first;
                    const int per = (blocks + wpu - 1) / wpu;
                    lo = min(blocks, ksub * per);
                    span = min(blocks, lo + per) - lo;
                    pieces = (span + p.bk - 1) / p.bk;
                    in_chunk = true;
                }
                while (round < rounds) {
                    const int idx = round * per_round + slot;
                    if (idx < n_u && piece < pieces) {
                        const UnitRows ur = unit_rows(p, u0 + idx);
                        out.valid = true;
                        out.unit = u0 + idx;
                        out.kb0 = chunk * chunk_blocks + lo + piece * p.bk;
                        out.nkb = min(p.bk, span - piece * p.bk);
                        out.map = p.map; out.bk = p.bk; out.sets = ur.sets; out.row_a = ur.row_a; out.row_b = ur.row_b;
                        ++piece;
                        return out;
                    }
                    ++round;
                    piece = 0;
                }
                ++chunk;
                round = 0;
                in_chunk = false;
            }
            ++pi;
            chunk = 0;
            in_product = false;
        }
        return out;
    }
};

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}

// ---- the grid barrier -------------------------------------------------------------------------------------------
// words: [0] arrivals of the current barrier, [1] generation, [2] CTAs that have left the kernel, [3] abort
struct GridBarrier {
    unsigned int* words;
    unsigned int gen;     // the generation this CTA waits to see pass
    unsigned int n_ctas;
};
// Returns false when the step is aborted (a wait ran out here or elsewhere).
__device__ bool grid_sync(GridBarrier& b, int* error, int* aborted_smem) {
    __syncthreads();
    if (threadIdx.x == 0) {
        bool ok = true;
        __threadfence();
        const unsigned int old = atomicAdd(&b.words[0], 1u);
        if (old == b.n_ctas - 1) {
            b.words[0] = 0;
            __threadfence();
            atomicAdd(&b.words[1], 1u);
        } else {
            const long long t0 = clock64();
            unsigned int v;
            for (;;) {
                asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(b.words + 1) : "memory");
                if (v != b.gen) break;
                unsigned int ab;
                asm volatile("ld.relaxed.gpu.u32 %0, [%1];" : "=r"(ab) : "l"(b.words + 3) : "memory");
                if (ab) { ok = false; break; }
                if (clock64() - t0 > kWaitCycles) {
                    atomicExch(&b.words[3], 1u);
                    if (error) atomicExch(error, 7);
                    ok = false;
                    break;
                }
            }
        }
        __threadfence();
        if (!ok) *aborted_smem = 1;
    }
    ++b.gen;
    __syncthreads();
    return *aborted_smem == 0;
}

// Bounded wait on an mbarrier (a warp's own): false when it ran out.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > kWaitCycles) return false;
    return true;
}

// ---- the kernel ----------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) decode_fused_kernel(FusedArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // the swizzle's rows
    unsigned char* ring_all = smem;
    unsigned char* flex = smem + kRingBytes;                          // x of the current chunk, then the attention's space
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(flex);
    unsigned char* kv_space = flex + kXBytes;
    float* red = reinterpret_cast<float*>(kv_space);                  // products: [warp][2][4][32] partial sums
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kRingBytes + kFlexBytes);      // [kWarps][kQueue] weights, then [kWarps][2] attention
    __shared__ float inv_rms[16];
    __shared__ __align__(16) __nv_bfloat16 zero_row[8];
    __shared__ int aborted;
    __shared__ int last_flag;
    __shared__ int piece_info[kWarps][4][kQueue];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, n_ctas = gridDim.x;
    const int T = a.T, tokp = T <= 8 ? 8 : 16;
    unsigned char* my_ring = ring_all + (size_t)warp * kWarpRing;
    uint64_t* my_bars = bars + warp * kQueue;
    uint64_t* att_bars = bars + kWarps * kQueue + warp * 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kWarps * (kQueue + 2); ++i) mbar_init(&bars[i], 1);
        aborted = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 8) zero_row[threadIdx.x] = __float2bfloat16(0.f);
    GridBarrier gb;
    gb.words = a.barrier;
    gb.n_ctas = (unsigned)n_ctas;
    {
        unsigned int g;
        asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(g) : "l"(a.barrier + 1) : "memory");
        gb.gen = g;
    }
    __syncthreads();

    // ---- the weight ring: ask for the first pieces at once -----------------------------------------------------
    // The ring is a queue of bytes: a piece takes as many as it needs (rows * (k + 8) * 2), pieces are used and freed in
    // the order they were asked for, and up to kQueue are in flight, each on a barrier of its own. So a warp's copies
    // run most of a layer ahead of its arithmetic, across the grid barriers between the phases.
    Walker ahead;
    ahead.start();
    Piece pending = ahead.next(a, cta, n_ctas, warp, tokp);     // the next piece to ask for
    int q_issued = 0, q_used = 0;            // pieces asked for / used so far (their barrier: count % kQueue)
    int ring_head = 0;                       // where the next piece goes
    int ring_in_flight = 0;                  // bytes from the oldest piece in flight to the head (with the gap at a wrap)
    // per piece in flight, in shared memory by warp: its offset, the bytes it holds of the ring (gap included), its
    // first block of K and how many of its blocks are this warp's
    int* piece_at = &piece_info[warp][0][0];
    int* piece_span = &piece_info[warp][1][0];
    int* piece_kb0 = &piece_info[warp][2][0];
    int* piece_nkb = &piece_info[warp][3][0];
    auto issue_more = [&]() {
        while (pending.valid && q_issued - q_used < kQueue) {
            const int box = pending.bk * 1024;                 // bytes of a copy: bk blocks of 8 rows of 128 bytes
            const int need = pending.sets * box;
            int at = ring_head, span = need;
            if (at + need > kWarpRing) {          // does not fit before the end: it goes to the start, the rest is a gap
                span = need + (kWarpRing - at);
                at = 0;
            }
            if (ring_in_flight + span > kWarpRing) break;     // no room yet
            const int b = q_issued % kQueue;
            if (lane == 0) {
                mbar_expect_tx(&my_bars[b], (uint32_t)need);
                tma_load_3d(my_ring + at, pending.map, 0, pending.row_a, pending.kb0, &my_bars[b]);
                if (pending.sets == 2) tma_load_3d(my_ring + at + box, pending.map, 0, pending.row_b, pending.kb0, &my_bars[b]);
                piece_at[b] = at;
                piece_span[b] = span;
                piece_kb0[b] = pending.kb0;
                piece_nkb[b] = pending.nkb;
            }
            __syncwarp();
            ring_head = at + need;
            ring_in_flight += span;
            ++q_issued;
            pending = ahead.next(a, cta, n_ctas, warp, tokp);
        }
    };
    issue_more();

    // ---- embedding -------------------------------------------------------------------------------------------------
    for (int t = cta; t < T; t += n_ctas) {
        const int tok = a.tokens[t];
        const bool ok = tok >= 0 && tok < a.V;
        if (!ok && threadIdx.x == 0 && a.status) atomicOr(a.status, 1);
        for (int d = threadIdx.x; d < a.D; d += kThreads)
            a.residual[(size_t)t * a.D + d] = ok ? bf(a.embed + (size_t)tok * a.D + d) : 0.f;
    }
    bool alive = grid_sync(gb, a.error, &aborted);

    // ---- one product: x staged chunk by chunk, the warps' pieces multiplied, sums added up, the epilogue ----------
    auto run_product = [&](int pi) {
        const Product p = product_of(a, pi);
        const Share s = share_of(p, cta, n_ctas, tokp);
        const int total_rows = product_rows_total(a, p);
        const FusedLayer* L = p.kind == K_HEAD ? nullptr : &a.layers[pi >> 2];
        const bool norm = p.kind == K_QKV || p.kind == K_GATE_UP || p.kind == K_HEAD;
        const int Tn = p.kind == K_HEAD ? a.n_rows : T;   // rows of x: the step's tokens, or the rows whose logits are wanted
        const int XS = s.chunk + 8;                       // row stride of the staged x
        const int slot = warp / s.wpu, ksub = warp % s.wpu;
        const int g = lane >> 2, q = lane & 3;
        float acc[kMaxRounds][2][4];
#pragma unroll
        for (int r = 0; r < kMaxRounds; ++r)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[r][0][e] = acc[r][1][e] = 0.f;
        float sq[2] = {0.f, 0.f};                         // sums of squares of tokens warp and warp + 8
        bool ok = true;

        // The epilogue of one unit, from the fragment: this thread holds tokens g and g + 8, rows 2q and 2q + 1.
        auto epilogue = [&](int unit, float (&c)[2][4]) {
            if (norm) {
                const float i0 = inv_rms[g], i1 = inv_rms[g + 8];
                c[0][0] *= i0; c[0][1] *= i0; c[0][2] *= i1; c[0][3] *= i1;
                c[1][0] *= i0; c[1][1] *= i0; c[1][2] *= i1; c[1][3] *= i1;
            }
            if (p.kind == K_QKV) {
                // a q or k unit: this thread holds dims d, d + 1 of a head (first sums) and their rotation partners
                // d + half, d + half + 1 (second sums); a v unit: dims d, d + 1 only
                const int hd = p.hd, half = hd / 2;
                const UnitRows ur = unit_rows(p, unit);
                const bool rot = ur.sets == 2;
                const int head = ur.row_a / hd, d = ur.row_a - head * hd + 2 * q;
                float ba0 = 0.f, ba1 = 0.f, bb0 = 0.f, bb1 = 0.f;
                if (L->b_qkv) {
                    ba0 = bf(L->b_qkv + ur.row_a + 2 * q); ba1 = bf(L->b_qkv + ur.row_a + 2 * q + 1);
                    if (rot) { bb0 = bf(L->b_qkv + ur.row_b + 2 * q); bb1 = bf(L->b_qkv + ur.row_b + 2 * q + 1); }
                }
#pragma unroll
                for (int half_t = 0; half_t < 2; ++half_t) {
                    const int t = g + 8 * half_t;
                    if (t >= T) continue;
                    const int pos = a.positions[t];
                    __nv_bfloat16* dst;
                    if (head < p.heads) {
                        dst = a.q + ((size_t)t * p.heads + head) * hd;
                    } else {
                        const bool is_v = head >= p.heads + p.kv_heads;
                        const int kvh = is_v ? head - p.heads - p.kv_heads : head - p.heads;
                        PagedKV paged{L->page_table, L->table_stride, L->ring, p.kv_heads, hd};
                        dst = (is_v ? L->v_pool : L->k_pool) + paged.row_offset(a.token_slot[t], pos, kvh);
                    }
                    const float lo0 = c[0][2 * half_t] + ba0, lo1 = c[0][2 * half_t + 1] + ba1;
                    if (!rot) {
                        *reinterpret_cast<uint32_t*>(dst + d) = pack2(lo0, lo1);
                    } else {
                        const float hi0 = c[1][2 * half_t] + bb0, hi1 = c[1][2 * half_t + 1] + bb1;
                        const float2 cs = *reinterpret_cast<const float2*>(L->cos_table + (size_t)pos * half + d);
                        const float2 sn = *reinterpret_cast<const float2*>(L->sin_table + (size_t)pos * half + d);
                        *reinterpret_cast<uint32_t*>(dst + d) = pack2(lo0 * cs.x - hi0 * sn.x, lo1 * cs.y - hi1 * sn.y);
                        *reinterpret_cast<uint32_t*>(dst + half + d) = pack2(lo0 * sn.x + hi0 * cs.x, lo1 * sn.y + hi1 * cs.y);
                    }
                }
                return;
            }
            const int n = unit * 8 + 2 * q;
#pragma unroll
            for (int half_t = 0; half_t < 2; ++half_t) {
                const int t = g + 8 * half_t;
                if (t >= Tn || n >= total_rows) continue;
                const float v0 = c[0][2 * half_t], v1 = c[0][2 * half_t + 1];
                const bool two = n + 1 < total_rows;
                if (p.kind == K_GATE_UP) {
                    const float u0 = c[1][2 * half_t], u1 = c[1][2 * half_t + 1];
                    __nv_bfloat16* dst = a.h + (size_t)t * a.H + n;
                    const float h0 = u0 * (v0 / (1.0f + expf(-v0))), h1 = u1 * (v1 / (1.0f + expf(-v1)));
                    if (two) *reinterpret_cast<uint32_t*>(dst) = pack2(h0, h1);
                    else *dst = __float2bfloat16_rn(h0);
                } else if (p.kind == K_HEAD) {
                    float* dst = a.logits + (size_t)t * a.V + n;
                    dst[0] = v0;
                    if (two) dst[1] = v1;
                } else {
                    float* dst = a.residual + (size_t)t * a.D + n;
                    if (two) {
                        float2 old = __ldcg(reinterpret_cast<const float2*>(dst));
                        old.x += v0; old.y += v1;
                        *reinterpret_cast<float2*>(dst) = old;
                    } else {
                        dst[0] = __ldcg(dst) + v0;
                    }
                }
            }
        };
        for (int chunk = 0; chunk < s.n_chunks; ++chunk) {
            const int ck0 = chunk * s.chunk, span = min(p.K, ck0 + s.chunk) - ck0;
            if (chunk > 0) __syncthreads();      // the chunk before has been multiplied
            // ---- stage x[:, ck0 : ck0 + span] as bfloat16 rows (with a norm: x * weight; 1 / rms goes onto the sums) ---
            if (s.n_u > 0) {
                for (int tt = warp; tt < tokp; tt += kWarps) {
                    __nv_bfloat16* row = xs + (size_t)tt * XS;
                    const bool live = tt < Tn;
                    if (norm) {
                        const int src_row = p.kind == K_HEAD ? (live ? a.rows[tt] : 0) : tt;
                        const float* xp = a.residual + (size_t)src_row * a.D + ck0;
                        const __nv_bfloat16* nw = (p.kind == K_HEAD ? a.norm_f : (p.kind == K_QKV ? L->norm1 : L->norm2)) + ck0;
                        float sum = sq[tt >> 3];
                        for (int c8 = lane; c8 < span / 8; c8 += 32) {
                            uint4 outv = make_uint4(0, 0, 0, 0);
                            if (live) {
                                const float4 p0 = __ldcg(reinterpret_cast<const float4*>(xp + c8 * 8));
                                const float4 p1 = __ldcg(reinterpret_cast<const float4*>(xp + c8 * 8 + 4));
                                const uint4 nraw = *reinterpret_cast<const uint4*>(nw + c8 * 8);
                                const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&nraw);
                                const float2 n0 = __bfloat1622float2(hh[0]), n1 = __bfloat1622float2(hh[1]);
                                const float2 n2 = __bfloat1622float2(hh[2]), n3 = __bfloat1622float2(hh[3]);
                                sum = fmaf(p0.x, p0.x, sum); sum = fmaf(p0.y, p0.y, sum); sum = fmaf(p0.z, p0.z, sum); sum = fmaf(p0.w, p0.w, sum);
                                sum = fmaf(p1.x, p1.x, sum); sum = fmaf(p1.y, p1.y, sum); sum = fmaf(p1.z, p1.z, sum); sum = fmaf(p1.w, p1.w, sum);
                                outv.x = pack2(p0.x * n0.x, p0.y * n0.y);
                                outv.y = pack2(p0.z * n1.x, p0.w * n1.y);
                                outv.z = pack2(p1.x * n2.x, p1.y * n2.y);
                                outv.w = pack2(p1.z * n3.x, p1.w * n3.y);
                            }
                            *reinterpret_cast<uint4*>(row + c8 * 8) = outv;
                        }
                        sq[tt >> 3] = sum;
                    } else {
                        const __nv_bfloat16* xp = (p.kind == K_OUT ? a.att : a.h) + (size_t)tt * p.K + ck0;
                        for (int c8 = lane; c8 < span / 8; c8 += 32)
                            *reinterpret_cast<uint4*>(row + c8 * 8) =
                                live ? __ldcg(reinterpret_cast<const uint4*>(xp + c8 * 8)) : make_uint4(0, 0, 0, 0);
                    }
                }
                if (norm && chunk == s.n_chunks - 1) {
                    // a token's whole row went through this warp: its 1 / rms (src/model.c:334-342 of the reference)
                    const float eps = p.kind == K_HEAD ? a.eps_f : (p.kind == K_QKV ? L->eps1 : L->eps2);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float total = warp_sum(sq[j]);
                        const int tt = warp + 8 * j;
                        if (lane == 0) inv_rms[tt] = tt < Tn ? 1.0f / sqrtf(total / (float)a.D + eps) : 0.f;
                    }
                }
            }
            __syncthreads();
            // ---- the warps' pieces of this chunk ------------------------------------------------------------------
            int lo, hi;
            warp_blocks(p, s, chunk, ksub, lo, hi);
            const int pieces = (hi - lo + p.bk - 1) / p.bk;
            const bool last_chunk = chunk == s.n_chunks - 1;
            // one round of the CTA's units, with the sums `c` (products that come in one chunk may have any number of
            // rounds and use acc[0] for each in turn; in several chunks a warp keeps one set of sums per round)
            auto run_round = [&](int round, float (&c)[2][4]) {
                {
                    const int idx = round * s.per_round + slot;
                    const bool mine = idx < s.n_u;
                    if (mine) {
                        const bool two_sets = unit_rows(p, s.u0 + idx).sets == 2;
                        for (int pc = 0; pc < pieces && ok; ++pc) {
                            const int ub = q_used % kQueue;
                            const int my_at = piece_at[ub], my_span = piece_span[ub];
                            const int kk0 = piece_kb0[ub] * kBlockK - ck0, my_nkb = piece_nkb[ub];
                            ok = wait_bar(&my_bars[ub], (uint32_t)(q_used / kQueue) & 1u);
                            ok = __all_sync(0xffffffffu, ok);
                            if (!ok) break;
                            // A: x rows (tokens); rows past tokp read the zero row. B: weight rows, 8 rows of 128 bytes to a
                            // block of K, the 16-byte pieces of row n at (piece ^ n): the 128-byte swizzle of the copy.
                            const int arow = lane & 15;
                            const uint32_t a_addr = arow < tokp ? smem_u32(xs + (size_t)arow * XS + kk0 + (lane >> 4) * 8) : smem_u32(zero_row);
                            const uint32_t a_step = arow < tokp ? 32u : 0u;
                            const uint32_t n = (uint32_t)(lane & 7), which = (uint32_t)(lane >> 3);
                            const uint32_t b_row = smem_u32(my_ring + my_at) + n * 128u;
                            const uint32_t set_b = (uint32_t)p.bk * 1024u;
                            const int steps = my_nkb * (kBlockK / 16);     // a multiple of 4
                            // four chains of sums per set (the tensor core's result comes back after ~30 cycles: one chain
                            // would wait for each), added up at the piece's end in a fixed order
                            float pa[4][4], pb[4][4];
#pragma unroll
                            for (int ch = 0; ch < 4; ++ch)
#pragma unroll
                                for (int e = 0; e < 4; ++e) pa[ch][e] = pb[ch][e] = 0.f;
                            for (int st = 0; st < steps; st += 4) {
                                uint32_t af[4][4], bfr[2][4];
#pragma unroll
                                for (int u = 0; u < 4; ++u) ldmatrix_x4(af[u], a_addr + a_step * (uint32_t)(st + u));
                                const uint32_t b_blk = b_row + (uint32_t)(st >> 2) * 1024u;
                                ldmatrix_x4(bfr[0], b_blk + ((which ^ n) << 4));
                                ldmatrix_x4(bfr[1], b_blk + (((4u + which) ^ n) << 4));
                                mma16816(pa[0], af[0], bfr[0][0], bfr[0][1]);
                                mma16816(pa[1], af[1], bfr[0][2], bfr[0][3]);
                                mma16816(pa[2], af[2], bfr[1][0], bfr[1][1]);
                                mma16816(pa[3], af[3], bfr[1][2], bfr[1][3]);
                                if (two_sets) {
                                    uint32_t bu[2][4];
                                    ldmatrix_x4(bu[0], b_blk + set_b + ((which ^ n) << 4));
                                    ldmatrix_x4(bu[1], b_blk + set_b + (((4u + which) ^ n) << 4));
                                    mma16816(pb[0], af[0], bu[0][0], bu[0][1]);
                                    mma16816(pb[1], af[1], bu[0][2], bu[0][3]);
                                    mma16816(pb[2], af[2], bu[1][0], bu[1][1]);
                                    mma16816(pb[3], af[3], bu[1][2], bu[1][3]);
                                }
                            }
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                c[0][e] += (pa[0][e] + pa[1][e]) + (pa[2][e] + pa[3][e]);
                                c[1][e] += (pb[0][e] + pb[1][e]) + (pb[2][e] + pb[3][e]);
                            }
                            // (the copy that reuses these bytes is issued after the loads above have returned their values:
                            // a proxy fence here would wait for every copy the CTA has in flight, a trip to memory per piece)
                            __syncwarp();
                            ++q_used;
                            ring_in_flight -= my_span;
                            issue_more();
                        }
                    }
                    if (last_chunk) {
                        // sums of the warps that share a unit, in warp order, then the epilogue by the first of them
                        if (s.wpu > 1) {
                            __syncthreads();     // (the same for every warp of the CTA: rounds and wpu are the CTA's)
                            float* mine_red = red + (size_t)warp * 256;
#pragma unroll
                            for (int e = 0; e < 4; ++e) { mine_red[e * 32 + lane] = c[0][e]; mine_red[128 + e * 32 + lane] = c[1][e]; }
                            __syncthreads();
                            if (ksub == 0) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) { c[0][e] = 0.f; c[1][e] = 0.f; }
                                for (int w2 = 0; w2 < s.wpu; ++w2) {
                                    const float* other = red + (size_t)(warp + w2) * 256;
#pragma unroll
                                    for (int e = 0; e < 4; ++e) { c[0][e] += other[e * 32 + lane]; c[1][e] += other[128 + e * 32 + lane]; }
                                }
                            }
                        }
                        if (mine && ksub == 0 && ok) epilogue(s.u0 + idx, c);
                        if (s.n_chunks == 1) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) c[0][e] = c[1][e] = 0.f;
                        }
                    }
                }
            };
            for (int round = 0; round < s.rounds; ++round) {
                if (s.n_chunks > 1 && round == 1) run_round(round, acc[1]);
                else run_round(round, acc[0]);
            }
        }
        if (!ok && lane == 0) {
            atomicExch(&a.barrier[3], 1u);
            if (a.error) atomicExch(a.error, 8);
        }
    };

    // ---- attention of one layer: this step's tokens over the cache --------------------------------------------------
    uint32_t att_uses[2] = {0, 0};     // uses of this warp's two tile buffers, over all layers: their barriers' phases
    auto run_attention = [&](int layer) {
        const FusedLayer& L = a.layers[layer];
        const int hd = a.head_dim, group = a.heads / a.kv_heads;
        const int n_items = T * a.kv_heads, S = a.att_splits;
        const int row_bytes = hd * 2 + 16;                     // padded rows: ldmatrix without bank conflicts
        const int tile_bytes = 16 * row_bytes;                 // keys of 16 positions (values: the same again)
        const int buffers = (kFlexBytes / kWarps) / (2 * tile_bytes) >= 2 ? 2 : 1;
        unsigned char* my_kv = flex + (size_t)warp * (kFlexBytes / kWarps);
        const int g = lane >> 2, q4 = lane & 3;
        const int KT = hd / 16, NT = hd / 8;
        PagedKV paged{L.page_table, L.table_stride, L.ring, a.kv_heads, hd};
        bool ok = true;
        // the newest keys and values were written by other CTAs' stores and are read by bulk copies
        asm volatile("fence.proxy.async.global;" ::: "memory");
        for (int work = cta; work < n_items * S; work += n_ctas) {
            const int item = work / S, part = work - item * S;
            const int t = item / a.kv_heads, kvh = item - t * a.kv_heads;
            const int pos = a.positions[t], slot_id = a.token_slot[t];
            const int start = (L.window > 0 && pos >= L.window) ? pos - L.window + 1 : 0;
            const int base0 = start / 16 * 16;
            const int n_tiles = (pos - base0) / 16 + 1;
            const int per_part = (n_tiles + S - 1) / S;
            const int tile_lo = min(n_tiles, part * per_part), tile_hi = min(n_tiles, tile_lo + per_part);
            // q of the group's heads (rows of the tile; rows past the group are zero)
            uint32_t qf[8][4];
            {
                const __nv_bfloat16* qb = a.q + ((size_t)t * a.heads + (size_t)kvh * group) * hd;
#pragma unroll
                for (int kt = 0; kt < 8; ++kt) {
                    if (kt < KT) {
                        const int d = kt * 16 + q4 * 2;
                        qf[kt][0] = g < group ? __ldcg(reinterpret_cast<const unsigned int*>(qb + (size_t)g * hd + d)) : 0u;
                        qf[kt][1] = g + 8 < group ? __ldcg(reinterpret_cast<const unsigned int*>(qb + (size_t)(g + 8) * hd + d)) : 0u;
                        qf[kt][2] = g < group ? __ldcg(reinterpret_cast<const unsigned int*>(qb + (size_t)g * hd + d + 8)) : 0u;
                        qf[kt][3] = g + 8 < group ? __ldcg(reinterpret_cast<const unsigned int*>(qb + (size_t)(g + 8) * hd + d + 8)) : 0u;
                    }
                }
            }
            float o[16][4];
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
            float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
            // this warp's tiles: tile_lo + warp, + 8, ...
            auto request = [&](int tile, int buf) {
                unsigned char* kt_ = my_kv + (size_t)buf * 2 * tile_bytes;
                unsigned char* vt_ = kt_ + tile_bytes;
                if (lane == 0) mbar_expect_tx(&att_bars[buf], 32u * (uint32_t)hd * 2u);
                __syncwarp();
                const int p0 = base0 + tile * 16 + (lane & 15);
                const size_t off = paged.row_offset(slot_id, p0, kvh);
                if (lane < 16) bulk_load(kt_ + (size_t)lane * row_bytes, L.k_pool + off, (uint32_t)hd * 2u, &att_bars[buf]);
                else bulk_load(vt_ + (size_t)(lane - 16) * row_bytes, L.v_pool + off, (uint32_t)hd * 2u, &att_bars[buf]);
            };
            int next_tile = tile_lo + warp;
            if (buffers == 2) {
                if (next_tile < tile_hi) request(next_tile, 0);
                if (next_tile + kWarps < tile_hi) request(next_tile + kWarps, 1);
            }
            int buf = 0;
            for (int tile = tile_lo + warp; tile < tile_hi && ok; tile += kWarps) {
                if (buffers == 1) request(tile, 0);
                ok = wait_bar(&att_bars[buf], att_uses[buf] & 1u);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ++att_uses[buf];
                const uint32_t kbase = smem_u32(my_kv + (size_t)buf * 2 * tile_bytes), vbase = kbase + (uint32_t)tile_bytes;
                // S = Q K^T: heads x 16 positions
                float sc[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
                    for (int kt = 0; kt < 8; ++kt) {
                        if (kt < KT) {
                            uint32_t b0, b1;
                            ldmatrix_x2(b0, b1, kbase + (uint32_t)(j * 8 + (lane & 7)) * (uint32_t)row_bytes + (uint32_t)(kt * 32) + (uint32_t)((lane >> 3) & 1) * 16u);
                            mma16816(sc[j], qf[kt], b0, b1);
                        }
                    }
                }
                const int p_first = base0 + tile * 16;
                float mx0 = m0, mx1 = m1;
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int pp = p_first + j * 8 + q4 * 2 + (e & 1);
                        const bool vis = pp >= start && pp <= pos;
                        const float x = vis ? sc[j][e] * a.scale_log2 : -CUDART_INF_F;
                        sc[j][e] = x;
                        if (e & 2) mx1 = fmaxf(mx1, x); else mx0 = fmaxf(mx0, x);
                    }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float ref0 = mx0 == -CUDART_INF_F ? 0.f : mx0, ref1 = mx1 == -CUDART_INF_F ? 0.f : mx1;
                const float c0 = exp2f(m0 - ref0), c1 = exp2f(m1 - ref1);
                m0 = mx0;
                m1 = mx1;
                uint32_t pf[4];
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float p0 = exp2f(sc[j][0] - ref0), p1 = exp2f(sc[j][1] - ref0);
                    const float p2 = exp2f(sc[j][2] - ref1), p3 = exp2f(sc[j][3] - ref1);
                    sum0 += p0 + p1;
                    sum1 += p2 + p3;
                    pf[j * 2] = pack2(p0, p1);
                    pf[j * 2 + 1] = pack2(p2, p3);
                }
                l0 = l0 * c0 + sum0;
                l1 = l1 * c1 + sum1;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (i < NT) {
                        o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
                        uint32_t b0, b1;
                        ldmatrix_x2_trans(b0, b1, vbase + (uint32_t)(lane & 15) * (uint32_t)row_bytes + (uint32_t)(i * 16));
                        mma16816(o[i], pf, b0, b1);
                    }
                }
                __syncwarp();
                if (buffers == 2) {
                    if (tile + 2 * kWarps < tile_hi) request(tile + 2 * kWarps, buf);
                    buf ^= 1;
                }
            }
            // ---- the CTA's warps merge in shared memory: [warp][16 heads][hd + 2] --------------------------------
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            __syncthreads();       // every warp has read its last tile: the tiles' space takes the warps' results
            float* merge = reinterpret_cast<float*>(flex);
            const int MS = hd + 2;
            {
                float* mine = merge + (size_t)warp * 16 * MS;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (i < NT) {
                        const int d = i * 8 + q4 * 2;
                        mine[g * MS + d] = o[i][0]; mine[g * MS + d + 1] = o[i][1];
                        mine[(g + 8) * MS + d] = o[i][2]; mine[(g + 8) * MS + d + 1] = o[i][3];
                    }
                }
                if (q4 == 0) {
                    mine[g * MS + hd] = m0; mine[g * MS + hd + 1] = l0;
                    mine[(g + 8) * MS + hd] = m1; mine[(g + 8) * MS + hd + 1] = l1;
                }
            }
            __syncthreads();
            // one thread per (head of the group, dimension): over the warps in order
            float* part_out = a.att_parts + ((size_t)item * S + part) * 16 * MS;
            for (int idx = threadIdx.x; idx < group * hd; idx += kThreads) {
                const int hrow = idx / hd, d = idx - hrow * hd;
                float M = -CUDART_INF_F;
                for (int w2 = 0; w2 < kWarps; ++w2) M = fmaxf(M, merge[((size_t)w2 * 16 + hrow) * MS + hd]);
                float Ls = 0.f, Os = 0.f;
                for (int w2 = 0; w2 < kWarps; ++w2) {
                    const float mw = merge[((size_t)w2 * 16 + hrow) * MS + hd];
                    if (mw == -CUDART_INF_F) continue;
                    const float f = exp2f(mw - M);
                    Ls += merge[((size_t)w2 * 16 + hrow) * MS + hd + 1] * f;
                    Os += merge[((size_t)w2 * 16 + hrow) * MS + d] * f;
                }
                if (S == 1) {
                    a.att[((size_t)t * a.heads + (size_t)kvh * group + hrow) * hd + d] = __float2bfloat16_rn(Os / Ls);
                } else {
                    part_out[hrow * MS + d] = Os;
                    if (d == 0) { part_out[hrow * MS + hd] = M; part_out[hrow * MS + hd + 1] = Ls; }
                }
            }
            if (S > 1) {
                // the part that finishes last adds the parts up, in part order
                __threadfence();
                __syncthreads();
                if (threadIdx.x == 0) {
                    const int done = atomicAdd(&a.att_counters[item], 1);
                    last_flag = done == S - 1;
                    if (last_flag) a.att_counters[item] = 0;     // ready for the next layer
                    __threadfence();
                }
                __syncthreads();
                if (last_flag) {
                    const float* parts = a.att_parts + (size_t)item * S * 16 * MS;
                    for (int idx = threadIdx.x; idx < group * hd; idx += kThreads) {
                        const int hrow = idx / hd, d = idx - hrow * hd;
                        float M = -CUDART_INF_F;
                        for (int s2 = 0; s2 < S; ++s2) M = fmaxf(M, __ldcg(parts + ((size_t)s2 * 16 + hrow) * MS + hd));
                        float Ls = 0.f, Os = 0.f;
                        for (int s2 = 0; s2 < S; ++s2) {
                            const float ms = __ldcg(parts + ((size_t)s2 * 16 + hrow) * MS + hd);
                            if (ms == -CUDART_INF_F) continue;
                            const float f = exp2f(ms - M);
                            Ls += __ldcg(parts + ((size_t)s2 * 16 + hrow) * MS + hd + 1) * f;
                            Os += __ldcg(parts + ((size_t)s2 * 16 + hrow) * MS + d) * f;
                        }
                        a.att[((size_t)t * a.heads + (size_t)kvh * group + hrow) * hd + d] = __float2bfloat16_rn(Os / Ls);
                    }
                }
            }
            __syncthreads();       // the merge space is free again
        }
        if (!ok && lane == 0) {
            atomicExch(&a.barrier[3], 1u);
            if (a.error) atomicExch(a.error, 9);
        }
    };

    // ---- the step ----------------------------------------------------------------------------------------------------
    int marks = 0;
    auto mark = [&]() {
        if (a.trace && cta == 0 && threadIdx.x == 0) {
            long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            a.trace[marks] = now;
        }
        ++marks;
    };
    mark();
    for (int layer = 0; layer < a.n_layers && alive; ++layer) {
        run_product(4 * layer + K_QKV);
        mark();
        if (!(alive = grid_sync(gb, a.error, &aborted))) break;
        mark();
        run_attention(layer);
        mark();
        if (!(alive = grid_sync(gb, a.error, &aborted))) break;
        mark();
        run_product(4 * layer + K_OUT);
        mark();
        if (!(alive = grid_sync(gb, a.error, &aborted))) break;
        mark();
        run_product(4 * layer + K_GATE_UP);
        mark();
        if (!(alive = grid_sync(gb, a.error, &aborted))) break;
        mark();
        run_product(4 * layer + K_DOWN);
        mark();
        alive = grid_sync(gb, a.error, &aborted);
        mark();
    }
    if (alive && a.n_rows > 0) run_product(4 * a.n_layers);
    mark();

    // Bulk copies this warp still has in flight must land before the CTA's shared memory is given up.
    {
        // pieces asked for and not used: wait for their bytes (bounded)
        for (; q_used < q_issued; ++q_used) wait_bar(&my_bars[q_used % kQueue], (uint32_t)(q_used / kQueue) & 1u);
    }
    __syncthreads();
    // the last CTA to leave puts the barrier's words back for the next launch
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int left = atomicAdd(&a.barrier[2], 1u);
        if (left == (unsigned)n_ctas - 1) {
            a.barrier[0] = 0;
            a.barrier[2] = 0;
            __threadfence();
        }
    }
}

int sm_count() {
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

int decode_fused_ctas() { return sm_count(); }

int decode_fused_splits(int T, int kv_heads) {
    const int items = T * kv_heads;
    int s = items > 0 ? sm_count() / items : 1;
    if (s > 16) s = 16;
    if (s < 1) s = 1;
    return s;
}

const char* decode_fused_refusal(int T, int D, int H, int heads, int kv_heads, int head_dim, int V) {
    if (T < 1 || T > 16) return "1 to 16 tokens";
    if (D % kBlockK || H % kBlockK || (heads * head_dim) % kBlockK) return "widths that are multiples of 64";
    if (head_dim % 16 || head_dim > 128 || head_dim < 16) return "head sizes that are multiples of 16 up to 128";
    if (heads % kv_heads || heads / kv_heads > 16) return "at most 16 heads per kv head";
    if (V < 1) return "a vocabulary";
    // K in several chunks: a warp holds the sums of at most kMaxRounds units
    const int chunk = T <= 8 ? 2048 : 1024;
    const int g = sm_count();
    struct { int units, K; } prods[4] = {{(heads + kv_heads) * head_dim / 16 + kv_heads * head_dim / 8, D}, {(D + 7) / 8, heads * head_dim},
                                         {(H + 7) / 8, D}, {(D + 7) / 8, H}};
    for (auto& p : prods) {
        if (p.K <= chunk) continue;
        const int n_u = (p.units + g - 1) / g;
        const int wpu = n_u >= 5 ? 1 : (n_u >= 3 ? 2 : (n_u == 2 ? 4 : 8));
        if ((n_u + kWarps / wpu - 1) / (kWarps / wpu) > kMaxRounds) return "layers whose products fit its accumulators";
    }
    if (D > chunk) {
        const int n_u = ((V + 7) / 8 + g - 1) / g;
        if ((n_u + kWarps - 1) / kWarps > kMaxRounds) return "an output head whose width fits one chunk";
    }
    return nullptr;
}

// Blocks of K a weight copy of each kind of product brings: what a warp of the CTAs with the fewest units takes of a
// chunk of 1024 elements, at most 8 KB a copy (one or two sets of 8 rows).
void decode_fused_blocks(int D, int H, int heads, int kv_heads, int head_dim, int V, int bk[5]) {
    const int g = sm_count();
    const int units[5] = {(heads + kv_heads) * head_dim / 16 + kv_heads * head_dim / 8, (D + 7) / 8, (H + 7) / 8, (D + 7) / 8, (V + 7) / 8};
    const int K[5] = {D, heads * head_dim, D, H, D};
    const int cap[5] = {4, 8, 4, 8, 8};
    for (int kind = 0; kind < 5; ++kind) {
        int n_u = units[kind] / g;
        if (n_u < 1) n_u = 1;
        const int wpu = n_u >= 5 ? 1 : (n_u >= 3 ? 2 : (n_u == 2 ? 4 : 8));
        int blocks = K[kind] / kBlockK;
        if (blocks > 1024 / kBlockK) blocks = 1024 / kBlockK;
        int per = (blocks + wpu - 1) / wpu;
        if (per > cap[kind]) per = (per + 1) / 2 > cap[kind] ? cap[kind] : (per + 1) / 2;
        bk[kind] = per < 1 ? 1 : per;
    }
}

// The tensor map of a [rows, K] bfloat16 weight matrix as [rows][K / 64][64]: a copy brings 8 rows by `bk` blocks of 64
// elements, each 8 x 64 block a 1024-byte atom of 128-byte swizzled rows. Written to `out` (128 bytes, host memory).
void decode_fused_encode_map(void* out, const void* w, long long rows, int K, int bk) {
    if (K % kBlockK || bk < 1 || bk > 16 || ((uintptr_t)w & 15))
        throw std::invalid_argument("decode_fused: a weight matrix needs K a multiple of 64 and a 16-byte aligned start");
    cuuint64_t dims[3] = {(cuuint64_t)kBlockK, (cuuint64_t)rows, (cuuint64_t)(K / kBlockK)};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)kBlockK * 2};
    cuuint32_t box[3] = {(cuuint32_t)kBlockK, 8, (cuuint32_t)bk};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = tc5::tensor_map_encoder()(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w),
                                           dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        throw std::runtime_error("decode_fused: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r) + " for a " +
                                 std::to_string(rows) + " x " + std::to_string(K) + " matrix");
}

void decode_fused(const FusedArgs& a, cudaStream_t stream) {
    const char* why = decode_fused_refusal(a.T, a.D, a.H, a.heads, a.kv_heads, a.head_dim, a.V);
    if (why) throw std::invalid_argument(std::string("decode_fused takes ") + why);
    if (a.att_splits < 1 || a.att_splits > 16) throw std::invalid_argument("decode_fused: 1 to 16 parts per sequence and kv head");
    if (a.maps == nullptr || ((uintptr_t)a.maps & 63)) throw std::invalid_argument("decode_fused: the tensor maps must lie on a 64-byte boundary");
    for (int k = 0; k < 5; ++k)
        if (a.bk[k] < 1 || a.bk[k] * 2048 > kWarpRing) throw std::invalid_argument("decode_fused: a copy of more blocks than a warp's ring holds");
    static std::once_flag once;
    static int max_blocks = 0;
    std::call_once(once, [] {
        cudaFuncSetAttribute(decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&max_blocks, decode_fused_kernel, kThreads, kSmemBytes);
    });
    if (max_blocks < 1) throw std::runtime_error("decode_fused: the kernel does not fit an SM");
    note_launch();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)sm_count());
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident at once, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_fused_kernel, a);
    if (e != cudaSuccess) throw std::runtime_error(std::string("decode_fused: launch failed: ") + cudaGetErrorString(e));
}

}  // namespace sm
