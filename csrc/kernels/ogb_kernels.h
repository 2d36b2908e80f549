// C entry points of the sm_100a kernel library (libogb_cuda.so).  Every function takes raw
// device pointers plus a CUDA stream handle and returns 0 on success, a cudaError_t (>0) from
// the launch, or a negative code for an argument the kernel cannot serve.  No function here
// allocates device memory: scratch buffers are passed in by the caller.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int ogb_num_sms(void);

// C[M,N] = A[M,K] * W[N,K]^T, bf16 in, fp32 accumulate (tcgen05), bf16 (C) or fp32 (C_f32) out.
// epilogue: 0 = (+bias), 1 = (+bias) + residual[M,N] (may alias C), 2 = SwiGLU over column-interleaved
// gate|up tiles (output [M, N/2]).  bn = 0 picks the tile width; status = device int32 word.
int ogb_gemm_bf16(const void* A, const void* W, void* C, const void* bias, const void* residual, void* C_f32, int M,
                  int N, int K, int lda, int ldw, int ldc, int ldr, int epilogue, int bn, int* status, void* stream);

// ogb_gemm_bf16 whose A rows are delivered by other GPUs: `a_ready` holds one counter per 128-row tile of A, bumped
// once per 8 rows that land; the TMA producer waits (at most a_wait_ns nanoseconds, 0 = default) for a tile before
// loading it, and the last CTA to finish clears the counters (a_done: a zeroed word).
int ogb_gemm_bf16_wait(const void* A, const void* W, void* C, const void* bias, const void* residual, void* C_f32, int M,
                       int N, int K, int lda, int ldw, int ldc, int ldr, int epilogue, int bn, uint32_t* a_ready,
                       uint32_t* a_done, unsigned long long a_wait_ns, int* status, void* stream);

// Stream-K decomposition of the GEMMs (on by default; OGB_STREAM_K=0 disables it): 1 / 0 sets it, the old value is returned.
int ogb_gemm_set_stream_k(int on);
// Programmatic dependent launch along scatter GEMM -> exchange kernel -> consuming GEMM (off by default; OGB_TP_PDL=1
// enables it at start-up): the follower starts while the leader is still running and finds its rows through the per-tile
// counters.  1 / 0 sets it, the old value is returned.
int ogb_tp_set_pdl(int on);

// out[r,:] = x[r,:] * rsqrt(mean(x^2) + eps) * w ; if delta != NULL first x += delta (written back to x).
int ogb_rmsnorm_bf16(void* x, const void* delta, const void* weight, void* out, int rows, int hidden, int ldx, int ldo,
                     float eps, void* stream);
int ogb_embedding_bf16(const int* ids, const void* table, void* out, int tokens, int hidden, int vocab, int* status,
                       void* stream);
int ogb_silu_mul_bf16(const void* gate_up, void* out, int rows, int inter, void* stream);

// Rotary embedding on q and k (in place on the packed qkv rows) + append of k, v into the paged pool.
// qkv: [tokens, (hq + 2*hkv) * d]; pool: [pages, hkv, 2, page_size, d] bf16; slot = page * page_size + offset.
int ogb_rope_kv_append_bf16(void* qkv, const int* positions, const int* slots, const float* cos_sin, void* pool,
                            int tokens, int hq, int hkv, int d, int rotary_dim, int interleaved, int page_size,
                            int64_t num_slots, int max_pos, int* status, void* stream);
// Same with e4m3 pages and one fp32 scale per (page, head, k|v): scales [pages, hkv, 2].
int ogb_rope_kv_append_fp8(void* qkv, const int* positions, const int* slots, const float* cos_sin, void* pool,
                           float* scales, int tokens, int hq, int hkv, int d, int rotary_dim, int interleaved,
                           int page_size, int64_t num_slots, int max_pos, int* status, void* stream);

// Paged GQA attention.  q rows live inside the packed qkv buffer (row stride q_stride elements).  window > 0: a query
// sees only its last `window` keys, plus -- attention sinks -- the first `sink` keys of the sequence; the page-table
// entries of pages that lie wholly between the two are never read (the scheduler may have released them).
int ogb_paged_prefill_bf16(const void* q, void* out, const void* pool, const int* page_table, const int* ctx_len,
                           const int* cu_q, const int* tile_seq, const int* tile_q0, int num_tiles, int num_seqs,
                           int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride, int o_stride,
                           float scale, int window, int sink, int* status, void* stream);
// Prefill attention on tcgen05 / TMEM: the contract of ogb_paged_prefill_bf16 plus `q_rows`, the number of rows of
// the packed query buffer the kernel's tensor map may read; each 128-row aligned pair of 64-row tiles is one CTA.
int ogb_paged_prefill_tc_bf16(const void* q, void* out, const void* pool, const int* page_table, const int* ctx_len,
                              const int* cu_q, const int* tile_seq, const int* tile_q0, int num_tiles, int num_seqs,
                              int q_rows, int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride,
                              int o_stride, float scale, int window, int sink, int* status, void* stream);
int ogb_paged_decode_bf16(const void* q, void* out, const void* pool, const int* page_table, const int* ctx_len,
                          int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride,
                          int o_stride, float scale, int num_splits, float* part_o, float* part_ml, int window,
                          int sink, int* status, void* stream);

// Same over e4m3 pages [pages, hkv, 2, 16, 128] uint8 with scales [pages, hkv, 2] fp32 (head_dim 128 only).
int ogb_paged_decode_fp8(const void* q, void* out, const void* pool, const float* scales, const int* page_table,
                         const int* ctx_len, int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d,
                         int q_stride, int o_stride, float scale, int num_splits, float* part_o, float* part_ml, int* status,
                         void* stream);
int ogb_paged_prefill_fp8(const void* q, void* out, const void* pool, const float* scales, const int* page_table,
                          const int* ctx_len, const int* cu_q, const int* tile_seq, const int* tile_q0, int num_tiles,
                          int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride, int o_stride,
                          float scale, int* status, void* stream);

// One-byte pages (kv_format 0 = e4m3, 1 = symmetric int8, 2 = e5m2), same pool and scale layout.
int ogb_rope_kv_append_q8(void* qkv, const int* positions, const int* slots, const float* cos_sin, void* pool, float* scales,
                          int kv_format, int tokens, int hq, int hkv, int d, int rotary_dim, int interleaved, int page_size,
                          int64_t num_slots, int max_pos, int* status, void* stream);
// How decode reads e4m3 pages when a KV head serves at most 8 query heads: 2 = tcgen05 kernel with the raw bytes as
// kind::f8f6f4 operands (default), 1 = mma.sync e4m3 kernel, 0 = expand pages to bf16 first.  OGB_E4M3_MMA=0|1|2 picks
// it at start-up; this call sets it and returns the old value.
int ogb_attn_set_e4m3_mma(int mode);
int ogb_paged_decode_q8(const void* q, void* out, const void* pool, const float* scales, int kv_format, const int* page_table,
                        const int* ctx_len, int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d,
                        int q_stride, int o_stride, float scale, int num_splits, float* part_o, float* part_ml, int window,
                        int sink, int* status, void* stream);
int ogb_paged_prefill_q8(const void* q, void* out, const void* pool, const float* scales, int kv_format, const int* page_table,
                         const int* ctx_len, const int* cu_q, const int* tile_seq, const int* tile_q0, int num_tiles,
                         int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride, int o_stride,
                         float scale, int window, int sink, int* status, void* stream);

// Sampling.  logits [rows, vocab] bf16 (ld = row stride).  out_tokens int32 [rows].
int ogb_argmax_bf16(const void* logits, int* out_tokens, int rows, int vocab, int ld, void* stream);
// Fused temperature -> top-k -> top-p -> min-p -> inverse-CDF draw (u in [0,1) per row).
// work: uint32 [rows, vocab] scratch.  Rows with temperature <= 0 take the argmax.
int ogb_sample_bf16(const void* logits, int* out_tokens, const float* temperature, const int* top_k, const float* top_p,
                    const float* min_p, const float* uniform, uint32_t* work, int rows, int vocab, int ld, void* stream);
// Greedy speculative verification: argmax over (k+1) logits rows per sequence, accepted-prefix length, next token.
int ogb_spec_verify_greedy(const void* logits, const int* draft_tokens, int* accept_len, int* out_tokens, int num_seqs,
                           int k, int vocab, int ld, void* stream);

// KV page utilities.
int ogb_kv_page_copy(void* pool, const int64_t* src_pages, const int64_t* dst_pages, int n, int64_t page_bytes,
                     void* stream);
int ogb_kv_gather_pages(const void* pool, void* staging, const int64_t* pages, int n, int64_t page_bytes, void* stream);
int ogb_kv_scatter_pages(void* pool, const void* staging, const int64_t* pages, int n, int64_t page_bytes, void* stream);
// Moves n pages of every one of `layers` page arrays in one launch (swap out / swap in / copy-on-write across the
// whole model).  Either side may be pinned host memory; int32 page ids are bounds-checked against the two counts.
int ogb_kv_move_pages(const uint64_t* dst_bases, const uint64_t* src_bases, int layers, const int* src_pages,
                      const int* dst_pages, int n, int64_t page_bytes, int64_t src_count, int64_t dst_count, int* status,
                      void* stream);

// MatMulNBits int4 (block 32, optional nibble zero points) weight-only GEMM, in-kernel dequant.
// qweight [N, K/32, 16] uint8 (low nibble = even k), scales [N, K/32] bf16 or fp32, zp [N, ceil(K/32/2)] or NULL.
int ogb_w4a16_gemv(const void* x, const void* qweight, const void* scales, const void* zp, const void* bias, void* y,
                   int M, int N, int K, int ldx, int ldy, int scales_fp32, void* stream);
int ogb_w4a16_gemv_fused(const void* x, const void* qweight, const void* scales, const void* zp, const void* bias,
                         const void* norm_w, const void* residual, void* y, int M, int N, int K, int ldx, int ldy, int ldr,
                         float eps, int prologue, int scales_fp32, void* stream);
int ogb_w4a16_dequant(const void* qweight, const void* scales, const void* zp, void* w_bf16, int N, int K,
                      int scales_fp32, void* stream);
// The same product for any M on the tensor cores: int4 tiles are dequantised to bf16 in shared memory in front of
// tcgen05.mma, so no bf16 copy of the weights exists.  K a multiple of 32; ldx, ldc multiples of 8.
int ogb_w4a16_gemm(const void* x, const void* qweight, const void* scales, const void* zp, const void* bias, void* out,
                   int M, int N, int K, int ldx, int ldc, int scales_fp32, int* status, void* stream);

// Operators of hybrid and sparse decoders (fp32 math; dtype 0 = fp32, 1 = bf16, 2 = fp16; all tensors contiguous).
// Linear attention: q [B,T,Hq*dk], k [B,T,Nk*dk], v [B,T,Hkv*dv], past / state_out [B,Hkv,dk,dv], decay [B,T,Hkv] or
// [B,T,Hkv*dk] (log decay), beta [B,T,Hkv] or [B,T,1]; out [B,T,max(Hq,Hkv)*dv].  Returns -2 for key widths other than 32, 64, 128.
int ogb_linear_attention(const void* q, const void* k, const void* v, const void* past, const void* decay, const void* beta,
                         void* out, void* state_out, int B, int T, int Hq, int Nk, int Hkv, int dk, int dv, int decay_per_dim,
                         int beta_heads, int use_decay, int use_delta, float scale, int dtype, void* stream);
// Depthwise causal convolution over concat(past, x): x / y [B,C,L], w [C,K], past / state_out [B,C,K-1].
int ogb_causal_conv_state(const void* x, const void* w, const void* bias, const void* past, void* y, void* state_out, int B,
                          int C, int L, int K, int silu, int dtype, void* stream);
// Attention of each query row over the positions listed for it: q / out [B,N,Sq,D], k / v [B,Nkv,total,D], sel int64
// [B, sel_heads (1 or N), Sq, Ksel] increasing with -1 as trailing padding, bias with four element strides or NULL.
int ogb_index_share_attention(const void* q, const void* k, const void* v, const void* sel, const void* bias, void* out, int B,
                              int N, int Nkv, int Sq, int total, int D, int Ksel, int sel_heads, const long long* bias_strides,
                              float scale, int dtype, int* status, void* stream);
// cache [B,G,C,row] and int64 idx [B,G,Q,K] -> out [B,G,Q,K,row]; an index outside the row's valid length sets the status word.
int ogb_sparse_kv_gather(const void* cache, const void* idx, const void* lengths, void* out, int B, int G, int C, int Q, int K,
                         int row_bytes, int* status, void* stream);

// MoE: softmax router with top-k (renormalised), device-side permutation by expert, grouped GEMM, combine.
int ogb_moe_route_topk(const void* router_logits, int* topk_ids, float* topk_w, int tokens, int experts, int k,
                       int renormalize, int ld, void* stream);
int ogb_moe_permute(const int* topk_ids, int* counts, int* offsets, int* cursor, int* sorted_route, int* route_pos,
                    int* tile_tab, int* meta, int tokens, int k, int e0, int experts, int max_mtiles, void* stream);
int ogb_moe_gather_rows(const void* x, const int* sorted_route, const int* meta, void* xs, int max_routes, int k, int hidden,
                        void* stream);
int ogb_moe_combine(const void* ys, const int* route_pos, const float* topk_w, void* out, int tokens, int k, int hidden,
                    int accumulate, void* stream);
int ogb_grouped_gemm_bf16(const void* A, const void* W, void* C, const int* group_tab, const int* group_mtiles, int experts,
                          int max_rows, int max_mtiles, int N, int K, int epilogue, int bn, int* status, void* stream);

// Tensor parallelism over peer-mapped memory (CUDA IPC): row-parallel GEMM whose epilogue publishes tiles to
// the owner rank, and the owner-side reduce + residual add + broadcast.  `sc` / `rp` are device-resident
// TpScatter / TpReduce structs (tp_comm.cuh).
int ogb_gemm_bf16_scatter(const void* A, const void* W, int M, int N, int K, int lda, int ldw, const void* sc, int bn,
                          int* status, void* stream);
int ogb_tp_signal_rows(const void* sc, int rows, void* stream);
int ogb_tp_reduce_bcast(const void* rp, int rows, int n, int chunk, int tp, int nvls, int* status, void* stream);

#ifdef __cplusplus
}
#endif
