// Host-side launchers of every kernel in this library. Pointers are device pointers; each
// call enqueues on `stream` and returns. Arithmetic is float everywhere; `DType` names the
// storage of a tensor. A launcher that cannot take a size throws std::invalid_argument
// with the size in the message rather than compute a wrong result.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm {

enum DType : int { F32 = 0, BF16 = 1 };

// Every launcher reports the kernels it enqueues (capi.cu keeps the count).
void note_launch(int kernels = 1);
long long launch_count();

// Whether the kernels of the decode chain are launched as programmatic dependents of their
// predecessors (see launch.cuh). On by default.
bool dependent_launch_enabled();
void set_dependent_launch(bool on);

// A device int that kernels whose bounded waits ran out write a code into (0: nothing
// happened); null until the host gives one. Kernels skip the write when it is null.
int* error_word();
void set_error_word(int* word);

// ---- elementwise.cu -------------------------------------------------------------------
// out[t, :] = table[tokens[t], :] as float. A token outside [0, V) sets *status |= 1 and
// its row is zeroed.
void embedding(const void* table, DType table_dt, const int32_t* tokens, float* out, int T, int D,
               int V, int32_t* status, cudaStream_t stream);

// y = x * (1 / sqrtf(mean(x^2) + eps)) * w for each row (src/model.c:334-342 of the reference).
// `rows` (nullable) picks the input rows: out[r] = norm(x[rows[r]]).
void rmsnorm(const float* x, const void* w, DType w_dt, float eps, void* out, DType out_dt,
             const int32_t* rows, int n_rows, int D, cudaStream_t stream);

// out[t, j] = up[t, j] * act(gate[t, j]), gate = gate_up[t, j], up = gate_up[t, H + j]; act 0: SiLU, g / (1 + exp(-g))
// (src/vecmath.c:78-81), 1: tanh-GELU (Activation in common.cuh).
void swiglu(const float* gate_up, void* out, DType out_dt, int T, int H, int act, cudaStream_t stream);

// Steps of a model that belong to no layer: x *= scale (an embedding scale); x = cap * tanh(x / cap) (a cap on the
// logits); x[t, :] += table[rows[t], :] (a table of position vectors added to the embeddings; rows outside it add nothing).
void scale_inplace(float* x, size_t total, float scale, cudaStream_t stream);
void softcap_inplace(float* x, size_t total, float cap, cudaStream_t stream);
void add_rows(float* x, const void* table, DType table_dt, const int32_t* rows, int T, int D, int n_table_rows, cudaStream_t stream);

struct RopeStoreArgs {
    const float* qkv;           // [T, (heads + 2 kv_heads) * head_dim], bias already added
    int T, heads, kv_heads, head_dim, rotary_dim;
    const int32_t* positions;   // [T] absolute positions
    const float* cos_table;     // [max_positions, rotary_dim / 2]
    const float* sin_table;
    void* q_out;                // [T, heads, head_dim]
    void* k_packed;             // [T, kv_heads, head_dim] or null
    void* v_packed;
    DType dt;                   // storage of q_out, k_packed, v_packed and the pools
    void* k_pool;               // one layer's page pool or null
    void* v_pool;
    const int32_t* page_table;  // [slots, table_stride]
    int table_stride;
    int ring;                   // 0, or the number of positions a windowed group keeps
    const int32_t* token_slot;  // [T]
    const int32_t* token_end;   // [T] the sequence's length after this step
};
// Rotates q and k (pairs (i, i + rotary_dim/2), src/model.c:439-450 with the converter's
// permutation undone), writes q, and writes k and v to the packed buffers and the cache.
void rope_store(const RopeStoreArgs& a, cudaStream_t stream);

// Writes packed keys and values [T, kv_heads, head_dim] (already rotated) to the cache, for steps whose attention
// must still read what the new rows replace in a windowed group's ring. A token whose place a later token of the
// same step takes (position < token_end - ring) is not stored.
void kv_store(const void* k_packed, const void* v_packed, DType dt, int T, int kv_heads, int head_dim, void* k_pool,
              void* v_pool, const int32_t* positions, const int32_t* page_table, int table_stride, int ring,
              const int32_t* token_slot, const int32_t* token_end, cudaStream_t stream);

// ---- gemm_simt.cu ---------------------------------------------------------------------
// out[t, n] (+)= sum_k x[t, k] * w[n, k] + bias[n]; float FMA in ascending k for every
// element, whatever T is. x: F32 or BF16; w, bias: F32 or BF16; out: F32 or BF16.
void gemm_simt(const void* x, DType x_dt, const void* w, DType w_dt, const void* bias, DType bias_dt,
               void* out, DType out_dt, int T, int N, int K, bool accumulate, cudaStream_t stream);

// ---- gemm_tc.cu -----------------------------------------------------------------------
// The same product for bfloat16 x and w on the tcgen05 tensor cores (TMA-fed, accumulator
// in tensor memory). mode 0: out = x w^T + bias (out F32 or BF16); 1: float out += x w^T;
// 2: out = act(x w_gate^T) * (x w_up^T) where w holds the gate rows [0, N) and the up rows
// [up_offset, up_offset + N); the activation (Activation in common.cuh) travels in mode's second byte: 2 | act << 8. Shapes whose K is split over several CTAs need a workspace
// of gemm_tc_workspace_bytes(). *error becomes non-zero if a bounded wait ran out.
bool gemm_tc_supports(int T, int N, int K);
size_t gemm_tc_workspace_bytes(int T, int N, int K, bool dual);
// q/k/v rows of up to 160 tokens with bias, rotation and the cache write in the product's epilogue (q to rope.q_out,
// rotated keys and values into the paged pools): x [T, K] bfloat16, w [(heads + 2 kv_heads) * head_dim, K]. Returns
// false, having done nothing, where the shape is not taken (heads that straddle tiles of 128 rows, K split more
// than a cluster's ways): the caller then runs the product and rope_store().
struct SkinnyRope;
bool gemm_tc_qkv_rope(const void* x, const void* w, const void* bias, DType bias_dt, int T, int K, const SkinnyRope& rope,
                      int* error, cudaStream_t stream);
// How a product of these sizes is cut: tokens per tile and CTAs along K.
void gemm_tc_plan(int T, int N, int K, bool dual, int* tile_n, int* splits);
void gemm_tc(const void* x, const void* w, const void* bias, DType bias_dt, void* out, DType out_dt, int T, int N,
             int K, int mode, int up_offset, float* workspace, int* error, cudaStream_t stream);

// ---- gemm_pair.cu ---------------------------------------------------------------------
// The same product (modes 0, 1, 2 of gemm_tc) for many tokens: two CTAs on one tile of 256 tokens with the two-CTA
// tcgen05.mma. gemm_tc() goes this way by itself where gemm_pair_takes() says so (more than 160 tokens, operands and
// output on 16 bytes, output rows a multiple of 16 bytes); gemm_pair_enable(false) keeps every product on the
// one-CTA kernel, for comparisons.
bool gemm_pair_takes(const void* x, const void* w, const void* out, DType out_dt, int T, int N, int K, int mode);
void gemm_pair_enable(bool on);
void gemm_pair(const void* x, const void* w, const void* bias, DType bias_dt, void* out, DType out_dt, int T, int N, int K,
               int mode, int up_offset, int* error, cudaStream_t stream);
// q/k/v rows of many tokens with bias, rotation and the cache write in the product's epilogue: rotated queries to q_out,
// rotated keys and the values to the step's packed tensors (where given) and into the paged pools (where given, and
// where the ring still has a place for the position). Head sizes 64 and 128, every dimension rotated. Returns false,
// having done nothing, where the product is not taken.
struct PairRope {
    int heads, kv_heads, head_dim;
    const int32_t* positions;   // [T]
    const float* cos_table;     // [positions, head_dim / 2]
    const float* sin_table;
    void* q_out;                // bfloat16 [T, heads, head_dim]
    void* k_packed;             // bfloat16 [T, kv_heads, head_dim] or null
    void* v_packed;
    void* k_pool;               // or null: nothing is written to the cache
    void* v_pool;
    const int32_t* page_table;
    int table_stride, ring;
    const int32_t* token_slot;  // [T]
    const int32_t* token_end;   // [T]
};
bool gemm_pair_qkv(const void* x, const void* w, const void* bias, DType bias_dt, int T, int K, const PairRope& rope, int* error,
                   cudaStream_t stream);

// ---- gemm_skinny.cu -------------------------------------------------------------------
// The product for a handful of tokens (T <= 32) and bfloat16 weights, with the layer's
// surroundings folded in. x is bfloat16 [T, K], or -- when norm_w is given -- the float
// residual [T, K], normalised on the fly (RMSNorm with norm_w and eps). mode 0: out = x w^T
// + bias; 1: float out += x w^T; 2: out = act(x w[:N]^T) * (x w[up_offset:up_offset+N]^T);
// 3: q/k/v rows with bias, rotation of q and k, q written to rope->q_out and k, v to the cache.
struct SkinnyRope {
    int heads, kv_heads, head_dim, rotary_dim;
    const int32_t* positions;   // [T]
    const float* cos_table;
    const float* sin_table;
    void* q_out;                // bfloat16 [T, heads, head_dim]
    void* k_pool;
    void* v_pool;
    const int32_t* page_table;
    int table_stride, ring;
    const int32_t* token_slot;  // [T]
    // null where a step has no use for them:
    void* k_packed = nullptr;   // bfloat16 [T, kv_heads, head_dim]: rotated keys of the step, beside (or instead of) the cache
    void* v_packed = nullptr;
    const int32_t* token_end = nullptr;   // [T] the token's sequence length after the step: with a ring, older positions are not stored
};
bool gemm_skinny_supports(int T, int N, int K);
// Rounds in which a CTA of the kernel takes its share of K for these sizes (1: all of its weights are in
// flight at once, which is what the kernel is good at).
int gemm_skinny_rounds(int T, int N, int K, bool gated);
void gemm_skinny(const void* x, const void* norm_w, DType norm_w_dt, float eps, const void* w, int T, int N, int K,
                 int mode, const void* bias, DType bias_dt, void* out, DType out_dt, int up_offset,
                 const SkinnyRope* rope, cudaStream_t stream);

// ---- attention_plain.cu ---------------------------------------------------------------
struct AttentionArgs {
    const void* q;              // [T, heads, head_dim]
    void* out;                  // [T, heads, head_dim]
    DType dt;
    int T, heads, kv_heads, head_dim;
    float scale;
    int window;                 // 0: every key up to the query's position
    const int32_t* positions;   // [T]
    // keys and values packed for this step's own tokens ...
    const void* k_packed;       // [T, kv_heads, head_dim] or null
    const void* v_packed;
    const int32_t* token_seq_start;  // [T] packed index of the first token the token's sequence brings in this step
    // ... and/or in the cache. With both, a key at a position before the first one its sequence brings in this
    // step is read from the cache and every later one from the packed tensors.
    const void* k_pool;
    const void* v_pool;
    const int32_t* page_table;
    int table_stride;
    int ring;
    const int32_t* token_slot;  // [T]
};
// One warp per (token, head); keys in ascending order in groups of 32 from the first
// visible key, so the result depends only on the query, the visible keys and the window.
void attention_plain(const AttentionArgs& a, cudaStream_t stream);

// ---- attention_prefill.cu -------------------------------------------------------------
// Causal attention of packed whole prompts for bfloat16 on the tensor cores. `tiles` lists
// the 64-query tiles: [n_tiles, 3] = (packed index of the sequence's first token, the
// sequence's length, first query of the tile). head_dim: multiples of 16 up to 128.
bool attention_prefill_supports(int head_dim);
void attention_prefill(const void* q, const void* k, const void* v, void* out, const int32_t* tiles, int n_tiles,
                       int heads, int kv_heads, int head_dim, float scale, int window, cudaStream_t stream);

// The same for sequences that go on from the cache by any number of tokens: `tiles` is [n_tiles, 5] = (packed index
// of the sequence's first token of this step, its tokens in this step, first query of the tile among them, the
// position of its first token of this step, its slot). Keys and values at earlier positions come from the page
// pools, the step's own from k and v; the cache need not hold the step's own tokens yet.
void attention_extend(const void* q, const void* k, const void* v, void* out, const int32_t* tiles, int n_tiles,
                      int heads, int kv_heads, int head_dim, float scale, int window, const void* k_pool,
                      const void* v_pool, const int32_t* page_table, int table_stride, int ring, cudaStream_t stream);

// ---- attention_prefill_tc.cu ----------------------------------------------------------
// The same as attention_prefill on the tcgen05 tensor cores (TMA operands, S and PV in tensor
// memory) for head sizes 64 and 128. q, k, v are the packed [T, heads or kv_heads, head_dim]
// tensors; `tiles` is the list attention_prefill takes (tiles of 64 queries; the kernel pairs
// them). A bounded wait that runs out writes a code into *error (nullable).
bool attention_prefill_tc_supports(int heads, int kv_heads, int head_dim);
// `longest`: the longest sequence (0: unknown); `variant`: -1 lets the launcher choose between one CTA an SM
// (0) and two (1, head size 64 only; it wins on long prompts).
void attention_prefill_tc(const void* q, const void* k, const void* v, void* out, const int32_t* tiles, int n_tiles, int T,
                          int heads, int kv_heads, int head_dim, float scale, int window, int longest, int variant,
                          int* error, cudaStream_t stream);

// The same kernel for sequences that go on from the cache by many tokens (prompt portions): keys and values come from
// the paged pools, which must hold the step's own tokens already; `tiles` [n_tiles, 5] as attention_extend takes them,
// `longest` the longest sequence after the step. No windowed group (its ring is written after the attention).
bool attention_extend_tc_supports(int heads, int kv_heads, int head_dim, long long pool_pages);
void attention_extend_tc(const void* q, void* out, const int32_t* tiles, int n_tiles, int T, int heads, int kv_heads, int head_dim,
                         float scale, int window, const void* k_pool, const void* v_pool, const int32_t* page_table,
                         int table_stride, long long pool_pages, int longest, int variant, int* error, cudaStream_t stream);

// ---- attention_decode.cu --------------------------------------------------------------
// One new token per sequence over the paged cache for bfloat16: a cluster of CTAs per
// (sequence, kv head) splits the visible positions and merges through distributed shared
// memory; no workspace. `max_len` (the longest sequence of the batch, or a bound of it) only
// sizes the clusters; `pool_pages` is the number of pages of the two pools (long shares of head sizes 64 and 128
// come in through a tensor map over them). head_dim: multiples of 16 up to 128; at most 16 heads per kv head.
bool attention_decode_supports(int heads, int kv_heads, int head_dim);
// How a launch for these sizes would be cut: plan[0..3] = CTAs per (sequence, kv head), positions per
// buffer, buffers, bytes of shared memory per CTA; for shares that are streamed tile by tile: CTAs, 0, tiles a
// warp keeps in flight, bytes of shared memory.
void attention_decode_plan(int B, int heads, int kv_heads, int head_dim, int window, int max_len, int* plan);
// `late`: the rows are not one new token per sequence but several new positions of a sequence (a short later message):
// the kernel before wrote more of the cache than each row's newest position, so nothing is read before the wait for it.
void attention_decode(const void* q, void* out, int B, int heads, int kv_heads, int head_dim, float scale, int window,
                      const int32_t* positions, const int32_t* slots, const void* k_pool, const void* v_pool,
                      const int32_t* page_table, int table_stride, int ring, int max_len, long long pool_pages, bool late,
                      cudaStream_t stream);

// ---- decode_fused.cu ------------------------------------------------------------------
// One decode step (every sequence goes on by one token) of a stack of standard layers -- RMSNorm, attention with
// q/k/v bias and full rotation over the paged cache, RMSNorm, gated feed-forward with SiLU -- with final norm and
// output head, in one persistent kernel for up to 16 tokens; bfloat16 weights, norm weights, biases and cache.
struct FusedLayer {                  // one per run of a layer, in run order, in device memory
    const __nv_bfloat16* w_qkv;      // [(heads + 2 kv_heads) * head_dim, D]
    const __nv_bfloat16* b_qkv;      // [(heads + 2 kv_heads) * head_dim] or null
    const __nv_bfloat16* w_o;        // [D, heads * head_dim]
    const __nv_bfloat16* w_gate_up;  // [2 H, D]: gate rows, then up rows
    const __nv_bfloat16* w_down;     // [D, H]
    const __nv_bfloat16* norm1;      // [D] before the attention
    const __nv_bfloat16* norm2;      // [D] before the feed-forward
    __nv_bfloat16* k_pool;           // this run's page pools
    __nv_bfloat16* v_pool;
    const int32_t* page_table;       // [slots, table_stride]
    const float* cos_table;          // [positions, head_dim / 2]
    const float* sin_table;
    int table_stride, ring, window;  // window 0: every key
    float eps1, eps2;
    int pad_;
};
struct FusedArgs {
    const FusedLayer* layers;
    int n_layers;
    const void* maps;                // device array of 4 * n_layers + 1 tensor maps (decode_fused_encode_map), 128 bytes each:
                                     // per layer q/k/v, o, gate/up, down; then the head
    int bk[5];                       // blocks of K a copy of each kind brings (decode_fused_blocks; the maps' boxes)
    int T, D, H, heads, kv_heads, head_dim, V;
    const __nv_bfloat16* embed;      // [V, D]
    const __nv_bfloat16* head;       // [V, D] (the embedding again when tied)
    const __nv_bfloat16* norm_f;     // [D]
    float eps_f;
    float scale_log2;                // attention scale * log2(e)
    const int32_t* tokens;           // [T]
    const int32_t* positions;        // [T]
    const int32_t* token_slot;       // [T]
    const int32_t* rows;             // [n_rows] tokens whose logits are wanted
    int n_rows;
    int att_splits;                  // parts a (sequence, kv head) is cut into (decode_fused_splits)
    // scratch, all in device memory: float residual [T, D]; q, att [T, heads * head_dim]; h [T, H];
    // att_parts [T * kv_heads * att_splits * 16 * (head_dim + 2)] floats; att_counters [T * kv_heads] zeros;
    // barrier: 4 words, zero before the first launch (and after a launch that reported an error)
    float* residual;
    __nv_bfloat16* q;
    __nv_bfloat16* att;
    __nv_bfloat16* h;
    float* att_parts;
    int* att_counters;
    unsigned int* barrier;
    float* logits;                   // [n_rows, V]
    int* error;                      // a bounded wait that ran out leaves a code here (nullable)
    int32_t* status;                 // |= 1 for a token outside the vocabulary (nullable)
    long long* trace;                // nullable: CTA 0 leaves the GPU's nanosecond timer here after every phase
};
// null if the kernel takes these sizes, else what it takes instead (for the caller's message or fallback)
const char* decode_fused_refusal(int T, int D, int H, int heads, int kv_heads, int head_dim, int V);
int decode_fused_splits(int T, int kv_heads);
void decode_fused_blocks(int D, int H, int heads, int kv_heads, int head_dim, int V, int bk[5]);
void decode_fused_encode_map(void* out, const void* w, long long rows, int K, int bk);
void decode_fused(const FusedArgs& a, cudaStream_t stream);

// ---- sampling.cu ----------------------------------------------------------------------
// out[b] = argmax over the allowed ids of logits[b, :], the lowest id on ties
// (src/sampler.c:57-63). `banned` (nullable) is one byte per id. `scratch` holds B words
// that are all ones and `counters` B zeros before the first launch; the kernel leaves them so.
void argmax(const float* logits, const uint8_t* banned, int32_t* out, int B, int V, unsigned long long* scratch,
            int* counters, cudaStream_t stream);

// Temperature sampling with optional top-k (0 or >= V: off) and top-p (1: off), one
// xorshift32 state per row, advanced once per call (src/sampler.c:103-127). out[b] = -1
// when every id is banned.
void sample(const float* logits, const uint8_t* banned, int32_t* out, uint32_t* rng_state, int B, int V,
            float temperature, int top_k, float top_p, cudaStream_t stream);

}  // namespace sm
