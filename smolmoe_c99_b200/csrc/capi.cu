// The C interface of the kernel library: plain functions over device pointers, so that it
// can be loaded with dlopen/ctypes and has no dependency beyond the CUDA runtime. Each
// function returns 0 or a non-zero status and leaves a message for sm_last_error(), in the
// manner of the reference's status channel (src/util.h:28-70): after an error the next call
// still works.
#include <cuda_runtime.h>

#include <atomic>
#include <exception>
#include <string>

#include "common.cuh"
#include "drain.cuh"
#include "kernels.h"

namespace {
thread_local std::string g_last_error;

template <typename F>
int guarded(F&& body) {
    try {
        body();
        cudaError_t e = cudaPeekAtLastError();
        if (e != cudaSuccess) {
            g_last_error = std::string("CUDA: ") + cudaGetErrorString(e);
            cudaGetLastError();
            return 2;
        }
        return 0;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return 1;
    } catch (...) {
        g_last_error = "unknown error";
        return 1;
    }
}
}  // namespace

namespace sm {
static std::atomic<long long> g_launches{0};
void note_launch(int kernels) { g_launches.fetch_add(kernels, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }
static std::atomic<bool> g_dependent_launch{true};
bool dependent_launch_enabled() { return g_dependent_launch.load(std::memory_order_relaxed); }
void set_dependent_launch(bool on) { g_dependent_launch.store(on, std::memory_order_relaxed); }
static std::atomic<int*> g_error_word{nullptr};
int* error_word() { return g_error_word.load(std::memory_order_relaxed); }
void set_error_word(int* word) { g_error_word.store(word, std::memory_order_relaxed); }
}  // namespace sm

namespace sm {
// For entry points that live in other files and report through the same message channel.
void set_last_error(const std::string& message) { g_last_error = message; }
}  // namespace sm

#define SM_API extern "C" __attribute__((visibility("default")))

SM_API const char* sm_last_error() { return g_last_error.c_str(); }

// Programmatic dependent launch of the decode chain's kernels: 1 on (default), 0 off.
SM_API void sm_set_dependent_launch(int on) { sm::set_dependent_launch(on != 0); }

// The device int that kernels report a bounded wait that ran out into.
SM_API void sm_set_error_word(int* word) { sm::set_error_word(word); }

// Positions per page of the key/value cache that the kernels are compiled for; the host's cache must use the same.
SM_API int sm_page_size() { return sm::kPageSize; }

// The bookkeeping of a CTA's way out after a bounded wait ran out (drain.cuh): which stage barriers, at which parity,
// still have copies in flight. Host arithmetic, here for tests. Returns their number (at most `stages`).
SM_API int sm_outstanding_fills(long long issued, long long consumed, int stages, int* stage_out, int* parity_out) {
    sm::OutstandingFill left[64];
    if (stages > 64) stages = 64;
    const int n = sm::outstanding_fills(issued, consumed, stages, left);
    for (int i = 0; i < n; ++i) { stage_out[i] = left[i].stage; parity_out[i] = (int)left[i].parity; }
    return n;
}

// Kernels enqueued by this library since it was loaded.
SM_API long long sm_launch_count() { return sm::launch_count(); }

SM_API int sm_embedding(const void* table, int table_dt, const int32_t* tokens, float* out, int T, int D, int V,
                        int32_t* status, void* stream) {
    return guarded([&] { sm::embedding(table, (sm::DType)table_dt, tokens, out, T, D, V, status, (cudaStream_t)stream); });
}

SM_API int sm_rmsnorm(const float* x, const void* w, int w_dt, float eps, void* out, int out_dt,
                      const int32_t* rows, int n_rows, int D, void* stream) {
    return guarded([&] {
        sm::rmsnorm(x, w, (sm::DType)w_dt, eps, out, (sm::DType)out_dt, rows, n_rows, D, (cudaStream_t)stream);
    });
}

SM_API int sm_swiglu(const float* gate_up, void* out, int out_dt, int T, int H, int act, void* stream) {
    return guarded([&] { sm::swiglu(gate_up, out, (sm::DType)out_dt, T, H, act, (cudaStream_t)stream); });
}

SM_API int sm_scale_inplace(float* x, long long total, float scale, void* stream) {
    return guarded([&] { sm::scale_inplace(x, (size_t)total, scale, (cudaStream_t)stream); });
}

SM_API int sm_softcap_inplace(float* x, long long total, float cap, void* stream) {
    return guarded([&] { sm::softcap_inplace(x, (size_t)total, cap, (cudaStream_t)stream); });
}

SM_API int sm_add_rows(float* x, const void* table, int table_dt, const int32_t* rows, int T, int D, int n_table_rows, void* stream) {
    return guarded([&] { sm::add_rows(x, table, (sm::DType)table_dt, rows, T, D, n_table_rows, (cudaStream_t)stream); });
}

SM_API int sm_rope_store(const float* qkv, int T, int heads, int kv_heads, int head_dim, int rotary_dim,
                         const int32_t* positions, const float* cos_table, const float* sin_table, void* q_out,
                         void* k_packed, void* v_packed, int dt, void* k_pool, void* v_pool,
                         const int32_t* page_table, int table_stride, int ring, const int32_t* token_slot,
                         const int32_t* token_end, void* stream) {
    return guarded([&] {
        sm::RopeStoreArgs a{qkv, T, heads, kv_heads, head_dim, rotary_dim, positions, cos_table, sin_table,
                            q_out, k_packed, v_packed, (sm::DType)dt, k_pool, v_pool, page_table, table_stride,
                            ring, token_slot, token_end};
        sm::rope_store(a, (cudaStream_t)stream);
    });
}

SM_API int sm_kv_store(const void* k_packed, const void* v_packed, int dt, int T, int kv_heads, int head_dim,
                       void* k_pool, void* v_pool, const int32_t* positions, const int32_t* page_table,
                       int table_stride, int ring, const int32_t* token_slot, const int32_t* token_end, void* stream) {
    return guarded([&] {
        sm::kv_store(k_packed, v_packed, (sm::DType)dt, T, kv_heads, head_dim, k_pool, v_pool, positions, page_table,
                     table_stride, ring, token_slot, token_end, (cudaStream_t)stream);
    });
}

SM_API int sm_gemm_simt(const void* x, int x_dt, const void* w, int w_dt, const void* bias, int bias_dt, void* out,
                        int out_dt, int T, int N, int K, int accumulate, void* stream) {
    return guarded([&] {
        sm::gemm_simt(x, (sm::DType)x_dt, w, (sm::DType)w_dt, bias, (sm::DType)bias_dt, out, (sm::DType)out_dt, T, N,
                      K, accumulate != 0, (cudaStream_t)stream);
    });
}

SM_API int sm_attention_plain(const void* q, void* out, int dt, int T, int heads, int kv_heads, int head_dim,
                              float scale, int window, const int32_t* positions, const void* k_packed,
                              const void* v_packed, const int32_t* token_seq_start, const void* k_pool,
                              const void* v_pool, const int32_t* page_table, int table_stride, int ring,
                              const int32_t* token_slot, void* stream) {
    return guarded([&] {
        sm::AttentionArgs a{q, out, (sm::DType)dt, T, heads, kv_heads, head_dim, scale, window, positions,
                            k_packed, v_packed, token_seq_start, k_pool, v_pool, page_table, table_stride, ring,
                            token_slot};
        sm::attention_plain(a, (cudaStream_t)stream);
    });
}

SM_API int sm_argmax(const float* logits, const uint8_t* banned, int32_t* out, int B, int V,
                     unsigned long long* scratch, int* counters, void* stream) {
    return guarded([&] { sm::argmax(logits, banned, out, B, V, scratch, counters, (cudaStream_t)stream); });
}

SM_API int sm_sample(const float* logits, const uint8_t* banned, int32_t* out, uint32_t* rng_state, int B, int V,
                     float temperature, int top_k, float top_p, void* stream) {
    return guarded([&] {
        sm::sample(logits, banned, out, rng_state, B, V, temperature, top_k, top_p, (cudaStream_t)stream);
    });
}

SM_API int sm_gemm_tc_supports(int T, int N, int K) { return sm::gemm_tc_supports(T, N, K) ? 1 : 0; }

SM_API long long sm_gemm_tc_workspace_bytes(int T, int N, int K, int dual) {
    return (long long)sm::gemm_tc_workspace_bytes(T, N, K, dual != 0);
}

SM_API void sm_gemm_pair_enable(int on) { sm::gemm_pair_enable(on != 0); }

SM_API int sm_gemm_pair_takes(const void* x, const void* w, const void* out, int out_dt, int T, int N, int K, int mode) {
    return sm::gemm_pair_takes(x, w, out, (sm::DType)out_dt, T, N, K, mode) ? 1 : 0;
}

SM_API int sm_gemm_tc_plan(int T, int N, int K, int dual, int* tile_n, int* splits) {
    return guarded([&] { sm::gemm_tc_plan(T, N, K, dual != 0, tile_n, splits); });
}

SM_API int sm_gemm_tc(const void* x, const void* w, const void* bias, int bias_dt, void* out, int out_dt, int T,
                      int N, int K, int mode, int up_offset, float* workspace, int* error, void* stream) {
    return guarded([&] {
        sm::gemm_tc(x, w, bias, (sm::DType)bias_dt, out, (sm::DType)out_dt, T, N, K, mode, up_offset, workspace, error,
                    (cudaStream_t)stream);
    });
}

SM_API int sm_attention_prefill_supports(int head_dim) { return sm::attention_prefill_supports(head_dim) ? 1 : 0; }

SM_API int sm_attention_prefill(const void* q, const void* k, const void* v, void* out, const int32_t* tiles,
                                int n_tiles, int heads, int kv_heads, int head_dim, float scale, int window,
                                void* stream) {
    return guarded([&] {
        sm::attention_prefill(q, k, v, out, tiles, n_tiles, heads, kv_heads, head_dim, scale, window, (cudaStream_t)stream);
    });
}

SM_API int sm_attention_extend(const void* q, const void* k, const void* v, void* out, const int32_t* tiles,
                               int n_tiles, int heads, int kv_heads, int head_dim, float scale, int window,
                               const void* k_pool, const void* v_pool, const int32_t* page_table, int table_stride,
                               int ring, void* stream) {
    return guarded([&] {
        sm::attention_extend(q, k, v, out, tiles, n_tiles, heads, kv_heads, head_dim, scale, window, k_pool, v_pool,
                             page_table, table_stride, ring, (cudaStream_t)stream);
    });
}

SM_API int sm_attention_prefill_tc_supports(int heads, int kv_heads, int head_dim) {
    return sm::attention_prefill_tc_supports(heads, kv_heads, head_dim) ? 1 : 0;
}

SM_API int sm_attention_prefill_tc(const void* q, const void* k, const void* v, void* out, const int32_t* tiles,
                                   int n_tiles, int T, int heads, int kv_heads, int head_dim, float scale, int window,
                                   int longest, int variant, int* error, void* stream) {
    return guarded([&] {
        sm::attention_prefill_tc(q, k, v, out, tiles, n_tiles, T, heads, kv_heads, head_dim, scale, window, longest,
                                 variant, error, (cudaStream_t)stream);
    });
}

SM_API int sm_attention_extend_tc_supports(int heads, int kv_heads, int head_dim, long long pool_pages) {
    return sm::attention_extend_tc_supports(heads, kv_heads, head_dim, pool_pages) ? 1 : 0;
}

SM_API int sm_attention_extend_tc(const void* q, void* out, const int32_t* tiles, int n_tiles, int T, int heads, int kv_heads,
                                  int head_dim, float scale, int window, const void* k_pool, const void* v_pool,
                                  const int32_t* page_table, int table_stride, long long pool_pages, int longest, int variant,
                                  int* error, void* stream) {
    return guarded([&] {
        sm::attention_extend_tc(q, out, tiles, n_tiles, T, heads, kv_heads, head_dim, scale, window, k_pool, v_pool, page_table,
                                table_stride, pool_pages, longest, variant, error, (cudaStream_t)stream);
    });
}

SM_API int sm_attention_decode_supports(int heads, int kv_heads, int head_dim) {
    return sm::attention_decode_supports(heads, kv_heads, head_dim) ? 1 : 0;
}

SM_API int sm_attention_decode_plan(int B, int heads, int kv_heads, int head_dim, int window, int max_len, int* plan) {
    return guarded([&] { sm::attention_decode_plan(B, heads, kv_heads, head_dim, window, max_len, plan); });
}

SM_API int sm_attention_decode(const void* q, void* out, int B, int heads, int kv_heads, int head_dim, float scale,
                               int window, const int32_t* positions, const int32_t* slots, const void* k_pool,
                               const void* v_pool, const int32_t* page_table, int table_stride, int ring, int max_len,
                               long long pool_pages, int late, void* stream) {
    return guarded([&] {
        sm::attention_decode(q, out, B, heads, kv_heads, head_dim, scale, window, positions, slots, k_pool, v_pool,
                             page_table, table_stride, ring, max_len, pool_pages, late != 0, (cudaStream_t)stream);
    });
}

// *taken = 1 if the fused kernel ran, 0 if the shape is not its own (nothing was done).
SM_API int sm_gemm_tc_qkv(const void* x, const void* w, int T, int K, const void* bias, int bias_dt, int heads, int kv_heads,
                          int head_dim, int rotary_dim, const int32_t* positions, const float* cos_table,
                          const float* sin_table, void* q_out, void* k_pool, void* v_pool, const int32_t* page_table,
                          int table_stride, int ring, const int32_t* token_slot, void* k_packed, void* v_packed,
                          const int32_t* token_end, int* error, int* taken, void* stream) {
    return guarded([&] {
        sm::SkinnyRope rope{heads, kv_heads, head_dim, rotary_dim, positions, cos_table, sin_table, q_out,
                            k_pool, v_pool, page_table, table_stride, ring, token_slot, k_packed, v_packed, token_end};
        *taken = sm::gemm_tc_qkv_rope(x, w, bias, (sm::DType)bias_dt, T, K, rope, error, (cudaStream_t)stream) ? 1 : 0;
    });
}

SM_API int sm_gemm_pair_qkv(const void* x, const void* w, int T, int K, const void* bias, int bias_dt, int heads, int kv_heads,
                            int head_dim, const int32_t* positions, const float* cos_table, const float* sin_table, void* q_out,
                            void* k_packed, void* v_packed, void* k_pool, void* v_pool, const int32_t* page_table,
                            int table_stride, int ring, const int32_t* token_slot, const int32_t* token_end, int* error,
                            int* taken, void* stream) {
    return guarded([&] {
        sm::PairRope rope{heads, kv_heads, head_dim, positions, cos_table, sin_table, q_out, k_packed, v_packed, k_pool, v_pool,
                          page_table, table_stride, ring, token_slot, token_end};
        *taken = sm::gemm_pair_qkv(x, w, bias, (sm::DType)bias_dt, T, K, rope, error, (cudaStream_t)stream) ? 1 : 0;
    });
}

SM_API int sm_gemm_skinny_supports(int T, int N, int K) { return sm::gemm_skinny_supports(T, N, K) ? 1 : 0; }

SM_API int sm_gemm_skinny_rounds(int T, int N, int K, int gated) { return sm::gemm_skinny_rounds(T, N, K, gated != 0); }

SM_API int sm_gemm_skinny(const void* x, const void* norm_w, int norm_w_dt, float eps, const void* w, int T, int N,
                          int K, int mode, const void* bias, int bias_dt, void* out, int out_dt, int up_offset,
                          void* stream) {
    return guarded([&] {
        sm::gemm_skinny(x, norm_w, (sm::DType)norm_w_dt, eps, w, T, N, K, mode, bias, (sm::DType)bias_dt, out,
                        (sm::DType)out_dt, up_offset, nullptr, (cudaStream_t)stream);
    });
}

SM_API int sm_gemm_skinny_qkv(const void* x, const void* norm_w, int norm_w_dt, float eps, const void* w, int T, int K,
                              const void* bias, int bias_dt, int heads, int kv_heads, int head_dim, int rotary_dim,
                              const int32_t* positions, const float* cos_table, const float* sin_table, void* q_out,
                              void* k_pool, void* v_pool, const int32_t* page_table, int table_stride, int ring,
                              const int32_t* token_slot, void* k_packed, void* v_packed, const int32_t* token_end,
                              void* stream) {
    return guarded([&] {
        sm::SkinnyRope rope{heads, kv_heads, head_dim, rotary_dim, positions, cos_table, sin_table, q_out,
                            k_pool, v_pool, page_table, table_stride, ring, token_slot, k_packed, v_packed, token_end};
        sm::gemm_skinny(x, norm_w, (sm::DType)norm_w_dt, eps, w, T, (heads + 2 * kv_heads) * head_dim, K, 3, bias,
                        (sm::DType)bias_dt, nullptr, sm::BF16, 0, &rope, (cudaStream_t)stream);
    });
}

// The fused decode step. `layers` points at a device array of n_layers records of 16 8-byte words each:
// w_qkv, b_qkv, w_o, w_gate_up, w_down, norm1, norm2, k_pool, v_pool, page_table, cos, sin (pointers), then
// (table_stride, ring), (window, eps1 as float bits), (eps2 as float bits, 0) packed as pairs of 32-bit words.
SM_API int sm_decode_fused_refusal(int T, int D, int H, int heads, int kv_heads, int head_dim, int V) {
    const char* why = sm::decode_fused_refusal(T, D, H, heads, kv_heads, head_dim, V);
    if (why) g_last_error = std::string("decode_fused takes ") + why;
    return why ? 1 : 0;
}

SM_API int sm_decode_fused_splits(int T, int kv_heads) { return sm::decode_fused_splits(T, kv_heads); }

SM_API int sm_decode_fused_layer_bytes() { return (int)sizeof(sm::FusedLayer); }

SM_API int sm_decode_fused_blocks(int D, int H, int heads, int kv_heads, int head_dim, int V, int* bk) {
    return guarded([&] { sm::decode_fused_blocks(D, H, heads, kv_heads, head_dim, V, bk); });
}

// Writes the 128-byte tensor map of a [rows, K] bfloat16 weight matrix to host memory at `out`.
SM_API int sm_decode_fused_encode_map(void* out, const void* w, long long rows, int K, int bk) {
    return guarded([&] { sm::decode_fused_encode_map(out, w, rows, K, bk); });
}

SM_API int sm_decode_fused(const void* layers, const void* maps, const int* bk, int n_layers, int T, int D, int H, int heads, int kv_heads, int head_dim, int V,
                           const void* embed, const void* head, const void* norm_f, float eps_f, float scale,
                           const int32_t* tokens, const int32_t* positions, const int32_t* token_slot, const int32_t* rows,
                           int n_rows, int att_splits, float* residual, void* q, void* att, void* h, float* att_parts,
                           int* att_counters, unsigned int* barrier, float* logits, int* error, int32_t* status,
                           long long* trace, void* stream) {
    return guarded([&] {
        sm::FusedArgs a{};
        a.layers = (const sm::FusedLayer*)layers; a.n_layers = n_layers;
        a.maps = maps;
        for (int k = 0; k < 5; ++k) a.bk[k] = bk[k];
        a.T = T; a.D = D; a.H = H; a.heads = heads; a.kv_heads = kv_heads; a.head_dim = head_dim; a.V = V;
        a.embed = (const __nv_bfloat16*)embed; a.head = (const __nv_bfloat16*)head; a.norm_f = (const __nv_bfloat16*)norm_f;
        a.eps_f = eps_f; a.scale_log2 = scale * 1.4426950408889634f;
        a.tokens = tokens; a.positions = positions; a.token_slot = token_slot; a.rows = rows; a.n_rows = n_rows;
        a.att_splits = att_splits; a.residual = residual; a.q = (__nv_bfloat16*)q; a.att = (__nv_bfloat16*)att;
        a.h = (__nv_bfloat16*)h; a.att_parts = att_parts; a.att_counters = att_counters; a.barrier = barrier;
        a.logits = logits; a.error = error; a.status = status; a.trace = trace;
        sm::decode_fused(a, (cudaStream_t)stream);
    });
}
