// Causal attention of whole prompts over their own keys for bfloat16 (prefill): packed
// sequences of unequal lengths, grouped heads, optional window, running softmax so that no
// score matrix is stored (the reference scans [start, pos] per query and head:
// src/model.c:459-491, src/kernels.c:1156-1176).
//
// A second form of the same kernel serves sequences that go on from the cache with any number of
// tokens (a prompt in portions, a later message of a conversation, single tokens mixed with prompts:
// the reference's model_forward(tokens, n, pos0), src/model.c:664-690): keys and values of positions
// before the first one a sequence brings in this step are read from the paged cache, the step's own
// from the packed tensors.
//
// One CTA per (tile of 64 queries of one sequence, head); 4 warps of 16 queries each. Keys
// and values come through shared memory in tiles of 64 positions; both products run on
// the tensor cores (mma.sync m16n8k16, bfloat16 in, float accumulate); maximum, sum and
// the rescaling are float. Key tiles that a query tile cannot see are skipped.
#include <math_constants.h>

#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels.h"

namespace sm {

namespace {

constexpr int kBM = 64, kBN = 64, kWarps = 4;

struct PrefillArgs {
    const __nv_bfloat16* q;   // [T, heads, HD]
    const __nv_bfloat16* k;   // [T, kv_heads, HD]
    const __nv_bfloat16* v;
    __nv_bfloat16* out;       // [T, heads, HD]
    const int32_t* tiles;     // [n_tiles, 3]: packed index of the sequence's first token, its length, first query;
                              // going on from the cache [n_tiles, 5]: ... its tokens in this step, first query among
                              // them, the position of its first token of this step, its slot
    int heads, kv_heads, window;
    float scale_log2;         // scale * log2(e)
    const __nv_bfloat16* k_pool;   // one layer's page pools (null: whole prompts)
    const __nv_bfloat16* v_pool;
    const int32_t* page_table;
    int table_stride, ring;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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

template <int HD, bool CACHED>
__global__ void __launch_bounds__(kWarps * 32) prefill_attention_kernel(PrefillArgs a) {
    constexpr int LD = HD + 8;            // padded row: conflict-free fragment loads
    constexpr int KT = HD / 16;           // k-steps of Q K^T
    constexpr int NT = HD / 8;            // n-tiles of P V
    __shared__ __align__(16) __nv_bfloat16 ks[kBN][LD];
    __shared__ __align__(16) __nv_bfloat16 vs[kBN][LD];

    // Queries are counted among the sequence's tokens of this step (0 .. seq_len-1), keys by their absolute
    // position; the two differ by pos0, the position of the step's first token of the sequence.
    const int tile = blockIdx.x, h = blockIdx.y;
    constexpr int TS = CACHED ? 5 : 3;
    const int seq_start = a.tiles[TS * tile], seq_len = a.tiles[TS * tile + 1], q0 = a.tiles[TS * tile + 2];
    const int pos0 = CACHED ? a.tiles[TS * tile + 3] : 0, slot = CACHED ? a.tiles[TS * tile + 4] : 0;
    const int seq_end = pos0 + seq_len;   // the sequence's length after this step
    const int kvh = h / (a.heads / a.kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = lane >> 2, tq = lane & 3;
    const int r0 = q0 + warp * 16 + quad, r1 = r0 + 8;   // this thread's two query positions

    // Q fragments straight from global memory (rows beyond the sequence read as zero)
    uint32_t qf[KT][4];
    {
        const __nv_bfloat16* qb = a.q + ((size_t)seq_start * a.heads + h) * HD;
        const size_t stride = (size_t)a.heads * HD;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            int d = kt * 16 + tq * 2;
            qf[kt][0] = r0 < seq_len ? *reinterpret_cast<const uint32_t*>(qb + r0 * stride + d) : 0u;
            qf[kt][1] = r1 < seq_len ? *reinterpret_cast<const uint32_t*>(qb + r1 * stride + d) : 0u;
            qf[kt][2] = r0 < seq_len ? *reinterpret_cast<const uint32_t*>(qb + r0 * stride + d + 8) : 0u;
            qf[kt][3] = r1 < seq_len ? *reinterpret_cast<const uint32_t*>(qb + r1 * stride + d + 8) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

    const int q_last = pos0 + min(q0 + kBM, seq_len) - 1;
    const int first_key = a.window > 0 ? max(0, pos0 + q0 - a.window + 1) : 0;
    PagedKV paged{a.page_table, a.table_stride, a.ring, a.kv_heads, HD};
    const __nv_bfloat16* kb = a.k + ((size_t)seq_start * a.kv_heads + kvh) * HD;
    const __nv_bfloat16* vb = a.v + ((size_t)seq_start * a.kv_heads + kvh) * HD;
    const size_t kv_stride = (size_t)a.kv_heads * HD;

    for (int n0 = (first_key / kBN) * kBN; n0 <= q_last; n0 += kBN) {
        __syncthreads();   // the previous tile has been read
        for (int c = threadIdx.x; c < kBN * (HD / 8); c += kWarps * 32) {
            int row = c / (HD / 8), col = (c % (HD / 8)) * 8;
            const int p = n0 + row;
            bool in = p < seq_end;
            if (CACHED && p < pos0) {
                in = in && p >= first_key;   // older rows of a ring may be gone; they are masked below anyway
                size_t g = in ? paged.row_offset(slot, p, kvh) + col : 0;
                cp_async16(&ks[row][col], a.k_pool + g, in);
                cp_async16(&vs[row][col], a.v_pool + g, in);
                continue;
            }
            size_t g = in ? (size_t)(p - pos0) * kv_stride + col : 0;
            cp_async16(&ks[row][col], kb + g, in);
            cp_async16(&vs[row][col], vb + g, in);
        }
        asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        // S = Q K^T for 16 queries x 64 keys
        float s[kBN / 8][4];
#pragma unroll
        for (int j = 0; j < kBN / 8; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kt = 0; kt < KT; ++kt) {
                const __nv_bfloat16* kr = &ks[j * 8 + quad][kt * 16 + tq * 2];
                uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr);
                uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + 8);
                mma_bf16(s[j], qf[kt], b0, b1);
            }
        }
        // scale, mask (causal, window, end of sequence), running maximum
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int j = 0; j < kBN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int key = n0 + j * 8 + tq * 2 + (e & 1);
                int qp = pos0 + ((e & 2) ? r1 : r0);
                bool vis = key <= qp && key < seq_end && (a.window <= 0 || key > qp - a.window);
                float x = vis ? s[j][e] * a.scale_log2 : -CUDART_INF_F;
                s[j][e] = x;
                if (e & 2) mx1 = fmaxf(mx1, x); else mx0 = fmaxf(mx0, x);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // a row that has seen no key yet keeps m = -inf; use 0 as its reference to avoid inf - inf
        const float ref0 = mx0 == -CUDART_INF_F ? 0.f : mx0, ref1 = mx1 == -CUDART_INF_F ? 0.f : mx1;
        const float c0 = exp2f(m0 - ref0), c1 = exp2f(m1 - ref1);
        m0 = mx0;
        m1 = mx1;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pf[kBN / 16][4];
#pragma unroll
        for (int j = 0; j < kBN / 8; ++j) {
            float p0 = exp2f(s[j][0] - ref0), p1 = exp2f(s[j][1] - ref0);
            float p2 = exp2f(s[j][2] - ref1), p3 = exp2f(s[j][3] - ref1);
            sum0 += p0 + p1;
            sum1 += p2 + p3;
            pf[j / 2][(j & 1) * 2] = pack_bf16(p0, p1);
            pf[j / 2][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l0 = l0 * c0 + sum0;
        l1 = l1 * c1 + sum1;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                uint32_t b0, b1;
                ldmatrix_x2_trans(b0, b1, &vs[kk * 16 + (lane & 15)][i * 8]);
                mma_bf16(o[i], pf[kk], b0, b1);
            }
        }
    }
    // the row sums live spread over the four threads of a quad
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
    __nv_bfloat16* ob = a.out + ((size_t)seq_start * a.heads + h) * HD;
    const size_t stride = (size_t)a.heads * HD;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        int d = i * 8 + tq * 2;
        if (r0 < seq_len) *reinterpret_cast<uint32_t*>(ob + r0 * stride + d) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        if (r1 < seq_len) *reinterpret_cast<uint32_t*>(ob + r1 * stride + d) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

template <int HD>
void launch(const PrefillArgs& a, int n_tiles, cudaStream_t stream) {
    dim3 grid(n_tiles, a.heads);
    if (a.k_pool != nullptr) prefill_attention_kernel<HD, true><<<grid, kWarps * 32, 0, stream>>>(a);
    else prefill_attention_kernel<HD, false><<<grid, kWarps * 32, 0, stream>>>(a);
}

void dispatch(const PrefillArgs& a, int n_tiles, int head_dim, cudaStream_t stream) {
    switch (head_dim) {
        case 16: launch<16>(a, n_tiles, stream); break;
        case 32: launch<32>(a, n_tiles, stream); break;
        case 48: launch<48>(a, n_tiles, stream); break;
        case 64: launch<64>(a, n_tiles, stream); break;
        case 80: launch<80>(a, n_tiles, stream); break;
        case 96: launch<96>(a, n_tiles, stream); break;
        case 112: launch<112>(a, n_tiles, stream); break;
        default: launch<128>(a, n_tiles, stream); break;
    }
}

void check(const char* what, int heads, int kv_heads, int head_dim) {
    if (!attention_prefill_supports(head_dim))
        throw std::invalid_argument(std::string(what) + ": head_dim " + std::to_string(head_dim) +
                                    " is not a multiple of 16 between 16 and 128 (the plain kernel takes it)");
    if (heads % kv_heads) throw std::invalid_argument(std::string(what) + ": kv_heads must divide heads");
    if (heads > 65535) throw std::invalid_argument(std::string(what) + ": more than 65535 heads");
}

}  // namespace

bool attention_prefill_supports(int head_dim) { return head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128; }

void attention_prefill(const void* q, const void* k, const void* v, void* out, const int32_t* tiles, int n_tiles,
                       int heads, int kv_heads, int head_dim, float scale, int window, cudaStream_t stream) {
    if (n_tiles <= 0) return;
    check("attention_prefill", heads, kv_heads, head_dim);
    note_launch();
    PrefillArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, tiles,
                  heads, kv_heads, window, scale * 1.4426950408889634f, nullptr, nullptr, nullptr, 0, 0};
    dispatch(a, n_tiles, head_dim, stream);
}

void attention_extend(const void* q, const void* k, const void* v, void* out, const int32_t* tiles, int n_tiles,
                      int heads, int kv_heads, int head_dim, float scale, int window, const void* k_pool,
                      const void* v_pool, const int32_t* page_table, int table_stride, int ring, cudaStream_t stream) {
    if (n_tiles <= 0) return;
    check("attention_extend", heads, kv_heads, head_dim);
    if (k_pool == nullptr || v_pool == nullptr || page_table == nullptr)
        throw std::invalid_argument("attention_extend: the cache's pools and page table are needed");
    note_launch();
    PrefillArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, tiles,
                  heads, kv_heads, window, scale * 1.4426950408889634f, (const __nv_bfloat16*)k_pool,
                  (const __nv_bfloat16*)v_pool, page_table, table_stride, ring};
    dispatch(a, n_tiles, head_dim, stream);
}

}  // namespace sm
