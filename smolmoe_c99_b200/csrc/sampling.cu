// Token selection on the GPU: greedy argmax, and temperature sampling with optional top-k
// and top-p, with the rules of the reference's sampler (src/sampler.c:57-127):
//   * candidates are ranked by (logit descending, id ascending); banned ids never appear;
//   * top-k keeps the k best; p_i = exp((l_i - l_max) / T) in double; top-p keeps the
//     shortest prefix whose mass reaches top_p of the total;
//   * u = (xorshift32(state) >> 8) / 2^24; the token is the first in rank order whose
//     cumulative mass exceeds u times the kept mass.
// One block per row. Masses are held as 64-bit fixed point (2^40 = the best candidate), so
// sums are exact integers and no result depends on the order threads add in. "The first
// element in rank order at which the cumulative weight reaches X" is found by a radix
// descent over the 56-bit rank (inverted logit bits, then id), 8 bits a pass.
#include <math_constants.h>

#include <stdexcept>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace sm {

constexpr int kSampleThreads = 1024;
constexpr unsigned long long kAllRanks = ~0ull;

// Larger logit -> smaller rank value; equal logits -> smaller id first. -0 counts as +0.
__device__ __forceinline__ unsigned long long rank_of(float logit, int id) {
    if (logit == 0.f) logit = 0.f;
    uint32_t bits = __float_as_uint(logit);
    uint32_t key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);  // ascending with the value
    return ((unsigned long long)(~key) << 24) | (unsigned long long)(uint32_t)id;
}

// Greedy choice in one launch over (chunks of the vocabulary, rows): every CTA finds the
// best rank of its chunk and lowers the row's 64-bit scratch word with atomicMin (a
// minimum does not depend on the order of arrival); the CTA that arrives last for a row
// writes the token and puts the scratch word and the counter back to their idle values.
constexpr int kArgmaxThreads = 256;
constexpr int kArgmaxChunks = 128;   // a vocabulary of 150 k: 1.2 k logits a CTA, one batch of loads a thread

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_kernel(const float* __restrict__ logits, const uint8_t* __restrict__ banned, int32_t* __restrict__ out, int V,
              unsigned long long* scratch, int* counters) {
    __shared__ unsigned long long best_shared[kArgmaxThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const float* row = logits + (size_t)b * V;
    const int per = (V + kArgmaxChunks - 1) / kArgmaxChunks;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    unsigned long long best = kAllRanks;
    for (int i0 = lo + threadIdx.x; i0 < hi; i0 += 4 * kArgmaxThreads) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            int i = i0 + u * kArgmaxThreads;
            v[u] = i < hi ? row[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            int i = i0 + u * kArgmaxThreads;
            if (i < hi && !(banned && banned[i])) {
                unsigned long long r = rank_of(v[u], i);
                best = r < best ? r : best;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other < best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) best_shared[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < kArgmaxThreads / 32; ++i) best = best_shared[i] < best ? best_shared[i] : best;
        atomicMin(&scratch[b], best);
        __threadfence();
        if (atomicAdd(&counters[b], 1) == kArgmaxChunks - 1) {
            __threadfence();
            unsigned long long final_rank = atomicExch(&scratch[b], kAllRanks);
            counters[b] = 0;
            out[b] = final_rank == kAllRanks ? -1 : (int32_t)(final_rank & 0xffffffu);
        }
    }
}

void argmax(const float* logits, const uint8_t* banned, int32_t* out, int B, int V, unsigned long long* scratch,
            int* counters, cudaStream_t stream) {
    if (B <= 0) return;
    if (V <= 0 || V > (1 << 24)) throw std::invalid_argument("argmax: vocabulary must be in [1, 2^24]");
    if (B > 65535) throw std::invalid_argument("argmax: more than 65535 rows");
    note_launch();
    launch_kernel("argmax", argmax_kernel, dim3(kArgmaxChunks, B), dim3(kArgmaxThreads), 0, stream, 1,
                  dependent_launch_enabled(), logits, banned, out, V, scratch, counters);
}

// ---------------------------------------------------------------------------------------
struct SearchState {
    unsigned long long hist[256];
    unsigned long long prefix;      // digits chosen so far (high part of the rank)
    unsigned long long cum_before;  // weight of all members ranked before the prefix
    unsigned long long reduce[kSampleThreads / 32];
    float lmax;
    int none_allowed;
};

__device__ __forceinline__ unsigned long long mass_of(float logit, float lmax, float temperature) {
    double x = ((double)logit - (double)lmax) / (double)temperature;
    return __double2ull_rn(exp(x) * 1099511627776.0);  // 2^40
}

// Finds the first member (rank <= cut) at which the cumulative weight reaches `want`.
// Returns its rank in st->prefix and the cumulative weight including it in *cum_inclusive.
template <bool UNIT>
__device__ void rank_search(const float* row, const uint8_t* banned, int V, unsigned long long cut,
                            unsigned long long want, float temperature, SearchState* st,
                            unsigned long long* cum_inclusive) {
    if (threadIdx.x == 0) { st->prefix = 0; st->cum_before = 0; }
    for (int pass = 0; pass < 7; ++pass) {
        int shift = 48 - 8 * pass;
        for (int i = threadIdx.x; i < 256; i += kSampleThreads) st->hist[i] = 0;
        __syncthreads();
        unsigned long long prefix = st->prefix;
        for (int i = threadIdx.x; i < V; i += kSampleThreads) {
            if (banned && banned[i]) continue;
            float l = row[i];
            unsigned long long r = rank_of(l, i);
            if (r > cut) continue;
            if (pass > 0 && (r >> (shift + 8)) != prefix) continue;
            unsigned long long w = UNIT ? 1ull : mass_of(l, st->lmax, temperature);
            if (w) atomicAdd(&st->hist[(r >> shift) & 255u], w);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long cum = st->cum_before;
            int digit = -1, last_nonempty = 0;
            for (int b = 0; b < 256; ++b) {
                if (!st->hist[b]) continue;
                last_nonempty = b;
                if (cum + st->hist[b] >= want) { digit = b; break; }
                cum += st->hist[b];
            }
            if (digit < 0) {  // want exceeds the total: end at the last member
                digit = last_nonempty;
                cum -= st->hist[digit];
            }
            st->cum_before = cum;
            st->prefix = (prefix << 8) | (unsigned long long)digit;
            if (pass == 6) *cum_inclusive = cum + st->hist[digit];
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, const uint8_t* __restrict__ banned, int32_t* __restrict__ out,
              uint32_t* __restrict__ rng_state, int V, float temperature, int top_k, float top_p) {
    __shared__ SearchState st;
    __shared__ unsigned long long result;
    const float* row = logits + (size_t)blockIdx.x * V;

    // the best allowed logit
    float lmax = -CUDART_INF_F;
    int any = 0;
    for (int i = threadIdx.x; i < V; i += kSampleThreads) {
        if (banned && banned[i]) continue;
        lmax = fmaxf(lmax, row[i]);
        any = 1;
    }
    lmax = warp_max(lmax);
    any = __any_sync(0xffffffffu, any);
    if ((threadIdx.x & 31) == 0) st.reduce[threadIdx.x >> 5] = ((unsigned long long)any << 32) | __float_as_uint(lmax);
    __syncthreads();
    if (threadIdx.x == 0) {
        float best = -CUDART_INF_F;
        int some = 0;
        for (int i = 0; i < kSampleThreads / 32; ++i) {
            best = fmaxf(best, __uint_as_float((uint32_t)st.reduce[i]));
            some |= (int)(st.reduce[i] >> 32);
        }
        st.lmax = best;
        st.none_allowed = !some;
    }
    __syncthreads();
    if (st.none_allowed) {
        if (threadIdx.x == 0) out[blockIdx.x] = -1;
        return;
    }

    unsigned long long cut = kAllRanks;
    if (top_k > 0 && top_k < V) {  // src/sampler.c:13: top-k at or above the vocabulary is off
        rank_search<true>(row, banned, V, cut, (unsigned long long)top_k, temperature, &st, &result);
        cut = st.prefix;
        __syncthreads();
    }
    // kept mass under the cut
    unsigned long long total = 0;
    for (int i = threadIdx.x; i < V; i += kSampleThreads) {
        if (banned && banned[i]) continue;
        float l = row[i];
        if (rank_of(l, i) > cut) continue;
        total += mass_of(l, st.lmax, temperature);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if ((threadIdx.x & 31) == 0) st.reduce[threadIdx.x >> 5] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long sum = 0;
        for (int i = 0; i < kSampleThreads / 32; ++i) sum += st.reduce[i];
        result = sum;
    }
    __syncthreads();
    total = result;
    __syncthreads();
    if (top_p < 1.0f) {
        double want = ceil((double)top_p * (double)total);
        unsigned long long want_int = want < 1.0 ? 1ull : (unsigned long long)want;
        rank_search<false>(row, banned, V, cut, want_int, temperature, &st, &result);
        cut = st.prefix;
        total = result;
        __syncthreads();
    }
    // one draw: the first member whose cumulative mass exceeds u * total, u = r / 2^24
    uint32_t x = rng_state[blockIdx.x];
    x ^= x << 13;
    x ^= x >> 17;
    x ^= x << 5;
    unsigned long long r = x >> 8;
    unsigned long long target = (__umul64hi(r, total) << 40) | ((r * total) >> 24);  // floor(r * total / 2^24)
    rank_search<false>(row, banned, V, cut, target + 1, temperature, &st, &result);
    if (threadIdx.x == 0) {
        out[blockIdx.x] = (int32_t)(st.prefix & 0xffffffu);
        rng_state[blockIdx.x] = x;
    }
}

void sample(const float* logits, const uint8_t* banned, int32_t* out, uint32_t* rng_state, int B, int V,
            float temperature, int top_k, float top_p, cudaStream_t stream) {
    if (B <= 0) return;
    if (V <= 0 || V > (1 << 24)) throw std::invalid_argument("sample: vocabulary must be in [1, 2^24]");
    if (!(temperature > 0.f)) throw std::invalid_argument("sample: temperature must be positive (0 is argmax)");
    if (!(top_p > 0.f && top_p <= 1.0f)) throw std::invalid_argument("sample: top_p must be in (0, 1]");
    note_launch();
    sample_kernel<<<B, kSampleThreads, 0, stream>>>(logits, banned, out, rng_state, V, temperature, top_k, top_p);
}

}  // namespace sm
