// Native step executor: launches the whole decoder stack of one engine step from a single call.
//
// The reference's counterpart is the nxrt session executor with its pre-bound device buffers and
// static plan (crates/onnx-runtime-session/src/executor/{build,run,bindings}.rs) driven by
// DecodeCudaState (crates/onnx-genai-engine/src/native_decode/cuda.rs:2958-3031).  Here the plan is
// the fused layer recipe itself, not an op list: per layer
//   rmsnorm -> qkv GEMM(+bias) -> RoPE + KV-page append -> paged decode / prefill attention ->
//   o_proj GEMM(+residual) -> rmsnorm -> gate_up GEMM(SwiGLU) -> down GEMM(+residual)
// then a gather of the rows that sample, the final norm and the lm_head GEMM.  All buffers are
// bound once at plan creation; a step passes only the shape of the batch and the device
// addresses of the plan sections.  Host cost per step is ~10 kernel launches per layer from C++
// (no interpreter in the loop), which keeps the GPU queue full.
#include <vector>

#include "common.cuh"
#include "ogb_kernels.h"

namespace ogb {

struct LayerPtrs {
  const void *ln1, *qkv_w, *qkv_b, *o_w, *ln2, *gate_up_w, *down_w;
  void* kv_pool;
};

// Weight paging: the matrices of the layers from `first` on live in pinned host memory, one contiguous pack per layer
// (qkv_w | o_w | gate_up_w | down_w), and pass through two device slots.  While layer l runs out of one slot the copy
// stream fills the other with layer l + 1; `copied` orders a layer's first GEMM after its copy, `consumed` orders the
// next copy into a slot after the layer that used it.  Role of the reference's weight paging for models larger than
// device memory (crates/onnx-runtime-ep-cuda/src/weight_paging.rs), done with two streams and four events.
struct WeightPaging {
  int first = -1;
  std::vector<const void*> host;
  void* slot[2] = {nullptr, nullptr};
  size_t bytes = 0, off[4] = {0, 0, 0, 0};
  cudaStream_t copy = nullptr;
  cudaEvent_t copied[2] = {nullptr, nullptr}, consumed[2] = {nullptr, nullptr};
  long long copies = 0;
};

struct DecoderPlan {
  int num_layers, hidden, hq, hkv, d, rotary_dim, interleaved, inter_local, vocab, swiglu_bn, window, sink, max_pages, max_pos;
  int tp, prefill_tc;
  int64_t num_pages;
  float eps, scale;
  const void *embed, *final_norm, *lm_head;
  const float* cos_sin;
  void *x, *h, *qkv, *attn, *act, *x_last, *h_last, *logits, *partial;
  float *part_o, *part_ml;
  int* status;
  std::vector<LayerPtrs> layers;
  long long launches = 0;
  long long launches_scatter = 0, launches_exchange = 0;   // row-parallel GEMMs with the scatter epilogue / exchange kernels
  WeightPaging wp;
};

}  // namespace ogb

using namespace ogb;

#define STEP_CHECK(expr)          \
  do {                            \
    int _rc = (expr);             \
    ++p->launches;                \
    if (_rc != 0) return _rc;     \
  } while (0)

// iparams: num_layers, hidden, hq, hkv, d, rotary_dim, interleaved, inter_local, vocab, swiglu_bn, window, max_pages,
//          max_pos, tp, prefill_tc (1: prefill attention on the tcgen05 kernel), sink (attention-sink keys kept by a window)
// fparams: eps, scale
// gptrs  : embed, final_norm, lm_head, cos_sin, x, h, qkv, attn, act, x_last, h_last, logits, partial, part_o, part_ml, status
// lptrs  : per layer 8 pointers (ln1, qkv_w, qkv_b, o_w, ln2, gate_up_w, down_w, kv_pool)
extern "C" void* ogb_decoder_create(const int* iparams, int64_t num_pages, const float* fparams, const uint64_t* gptrs,
                                    const uint64_t* lptrs) {
  DecoderPlan* p = new DecoderPlan();
  p->num_layers = iparams[0]; p->hidden = iparams[1]; p->hq = iparams[2]; p->hkv = iparams[3]; p->d = iparams[4];
  p->rotary_dim = iparams[5]; p->interleaved = iparams[6]; p->inter_local = iparams[7]; p->vocab = iparams[8];
  p->swiglu_bn = iparams[9]; p->window = iparams[10]; p->max_pages = iparams[11]; p->max_pos = iparams[12];
  p->tp = iparams[13];
  p->prefill_tc = iparams[14];
  p->sink = iparams[15];
  p->num_pages = num_pages;
  p->eps = fparams[0]; p->scale = fparams[1];
  auto P = [&](int i) { return reinterpret_cast<void*>(gptrs[i]); };
  p->embed = P(0); p->final_norm = P(1); p->lm_head = P(2); p->cos_sin = static_cast<const float*>(P(3));
  p->x = P(4); p->h = P(5); p->qkv = P(6); p->attn = P(7); p->act = P(8); p->x_last = P(9); p->h_last = P(10);
  p->logits = P(11); p->partial = P(12); p->part_o = static_cast<float*>(P(13)); p->part_ml = static_cast<float*>(P(14));
  p->status = static_cast<int*>(P(15));
  p->layers.resize(p->num_layers);
  for (int l = 0; l < p->num_layers; ++l) {
    const uint64_t* q = lptrs + 8 * l;
    LayerPtrs& L = p->layers[l];
    L.ln1 = reinterpret_cast<void*>(q[0]); L.qkv_w = reinterpret_cast<void*>(q[1]); L.qkv_b = reinterpret_cast<void*>(q[2]);
    L.o_w = reinterpret_cast<void*>(q[3]); L.ln2 = reinterpret_cast<void*>(q[4]); L.gate_up_w = reinterpret_cast<void*>(q[5]);
    L.down_w = reinterpret_cast<void*>(q[6]); L.kv_pool = reinterpret_cast<void*>(q[7]);
  }
  return p;
}

extern "C" void ogb_decoder_destroy(void* plan) {
  DecoderPlan* p = static_cast<DecoderPlan*>(plan);
  if (p != nullptr && p->wp.copy != nullptr) {
    cudaStreamSynchronize(p->wp.copy);
    for (int i = 0; i < 2; ++i) { cudaEventDestroy(p->wp.copied[i]); cudaEventDestroy(p->wp.consumed[i]); }
    cudaStreamDestroy(p->wp.copy);
  }
  delete p;
}

// Page the matrices of layers [first_layer, num_layers) through two device slots (see WeightPaging).  host_packs: one
// pinned pointer per paged layer; slots: two device buffers of `bytes`; offsets: qkv_w, o_w, gate_up_w, down_w inside a pack.
extern "C" int ogb_decoder_set_weight_paging(void* plan, int first_layer, const uint64_t* host_packs, const uint64_t* slots,
                                             int64_t bytes, const int64_t* offsets) {
  DecoderPlan* p = static_cast<DecoderPlan*>(plan);
  if (p == nullptr || first_layer < 0 || first_layer >= p->num_layers || bytes <= 0 || p->wp.copy != nullptr) return -3;
  WeightPaging& w = p->wp;
  for (int l = first_layer; l < p->num_layers; ++l) w.host.push_back(reinterpret_cast<const void*>(host_packs[l - first_layer]));
  w.slot[0] = reinterpret_cast<void*>(slots[0]);
  w.slot[1] = reinterpret_cast<void*>(slots[1]);
  w.bytes = static_cast<size_t>(bytes);
  for (int i = 0; i < 4; ++i) w.off[i] = static_cast<size_t>(offsets[i]);
  OGB_CUDA_CHECK(cudaStreamCreateWithFlags(&w.copy, cudaStreamNonBlocking));
  for (int i = 0; i < 2; ++i) {
    OGB_CUDA_CHECK(cudaEventCreateWithFlags(&w.copied[i], cudaEventDisableTiming));
    OGB_CUDA_CHECK(cudaEventCreateWithFlags(&w.consumed[i], cudaEventDisableTiming));
  }
  w.first = first_layer;
  return 0;
}
extern "C" long long ogb_decoder_weight_copies(void* plan) { return static_cast<DecoderPlan*>(plan)->wp.copies; }
extern "C" long long ogb_decoder_launches(void* plan) { return static_cast<DecoderPlan*>(plan)->launches; }
// which: 0 = all kernels, 1 = GEMMs with the tensor-parallel scatter epilogue, 2 = tensor-parallel exchange kernels
extern "C" long long ogb_decoder_counter(void* plan, int which) {
  DecoderPlan* p = static_cast<DecoderPlan*>(plan);
  return which == 1 ? p->launches_scatter : which == 2 ? p->launches_exchange : p->launches;
}
// The KV pool is a reserved address range of which `num_pages` pages are backed; the kernels bound page ids by it.
extern "C" void ogb_decoder_set_num_pages(void* plan, int64_t num_pages) { static_cast<DecoderPlan*>(plan)->num_pages = num_pages; }
extern "C" void ogb_decoder_set_split_scratch(void* plan, float* part_o, float* part_ml) {
  DecoderPlan* p = static_cast<DecoderPlan*>(plan);
  p->part_o = part_o;
  p->part_ml = part_ml;
}

// One forward pass of a dense decoder.  Section pointers address the device copy of the packed
// step plan.
extern "C" int ogb_gemm_bf16_scatter(const void* A, const void* W, int M, int N, int K, int lda, int ldw, const void* sc,
                                     int bn, int* status, void* stream_);
extern "C" int ogb_tp_reduce_bcast(const void* rp, int rows, int n, int chunk, int tp, int nvls, int* status, void* stream);
extern "C" int ogb_tp_exchange_norm(const void* rp, const void* norm_w, float eps, int rows, int n, int chunk, int tp, int nvls,
                                    int pushed, int* status, void* stream);
extern "C" int ogb_tp_wait_ready(const void* rp, int rows, int* status, void* stream);
extern "C" int ogb_gemm_bf16_wait(const void* A, const void* W, void* C, const void* bias, const void* residual, void* C_f32,
                                  int M, int N, int K, int lda, int ldw, int ldc, int ldr, int epilogue, int bn,
                                  uint32_t* a_ready, uint32_t* a_done, unsigned long long a_wait_ns, int* status, void* stream_);

// tp > 1: `tp_structs` = {scatter slot 0, reduce slot 0, scatter slot 1, reduce slot 1} device structs for this
// step's row chunk, one flag word (bit 0: the reduce structs carry NVSwitch multicast pointers, bit 1: the scatter
// epilogue pushes partials into the owners' buffers), then the
// local addresses of the two slots' per-tile ready counters.  The residual stream p->x is then owned by rows
// (each rank keeps its own chunk), p->h lives in the peer-mapped region, and a row-parallel projection is
//   GEMM with the scatter epilogue  ->  exchange (reduce-scatter + residual + RMSNorm + all-gather of h)
// followed by a column-parallel GEMM whose TMA producer waits tile by tile for the rows of h.
extern "C" int ogb_decoder_step(void* plan, const int* token_ids, const int* positions, const int* slots,
                                const int* ctx_len, const int* page_table, const int* cu_q, const int* tile_seq,
                                const int* tile_q0, const int* logit_rows, int T, int Nd, int Np, int num_tiles, int R,
                                int decode_splits, void* stream, const uint64_t* tp_structs, int tp_chunk) {
  DecoderPlan* p = static_cast<DecoderPlan*>(plan);
  if (T <= 0) return 0;
  if (p->tp != 1 && tp_structs == nullptr) return -10;
  const void* sc[2] = {nullptr, nullptr};
  const void* rd[2] = {nullptr, nullptr};
  uint32_t* ready[2] = {nullptr, nullptr};      // per-tile ready counters of the two slots; [k] + 64 is the slot's GEMM-done word
  int nvls = 0, pushed = 0;
  const bool tp = p->tp != 1;
  if (tp) {
    sc[0] = reinterpret_cast<const void*>(tp_structs[0]); rd[0] = reinterpret_cast<const void*>(tp_structs[1]);
    sc[1] = reinterpret_cast<const void*>(tp_structs[2]); rd[1] = reinterpret_cast<const void*>(tp_structs[3]);
    nvls = (tp_structs[4] & 1) != 0 ? 1 : 0;
    pushed = (tp_structs[4] & 2) != 0 ? 1 : 0;
    ready[0] = reinterpret_cast<uint32_t*>(tp_structs[5]);
    ready[1] = reinterpret_cast<uint32_t*>(tp_structs[6]);
  }
  const int hid = p->hidden, d = p->d, hq = p->hq, hkv = p->hkv;
  const int qkv_n = (hq + 2 * hkv) * d;
  const int attn_n = hq * d;
  char* qkv_prefill = static_cast<char*>(p->qkv) + static_cast<size_t>(Nd) * qkv_n * 2;
  char* attn_prefill = static_cast<char*>(p->attn) + static_cast<size_t>(Nd) * attn_n * 2;
  STEP_CHECK(ogb_embedding_bf16(token_ids, p->embed, p->x, T, hid, p->vocab, p->status, stream));
  if (tp) {
    // every rank embeds and norms all rows once; from here on a rank only updates the residual rows it owns
    STEP_CHECK(ogb_rmsnorm_bf16(p->x, nullptr, p->layers[0].ln1, p->h, T, hid, hid, hid, p->eps, stream));
  }
  WeightPaging& wp = p->wp;
  cudaStream_t cstream = static_cast<cudaStream_t>(stream);
  auto page_in = [&](int l) -> int {          // start the copy of layer l into its slot, behind the slot's last reader
    const int i = l - wp.first, s = i & 1;
    OGB_CUDA_CHECK(cudaStreamWaitEvent(wp.copy, wp.consumed[s], 0));
    OGB_CUDA_CHECK(cudaMemcpyAsync(wp.slot[s], wp.host[i], wp.bytes, cudaMemcpyHostToDevice, wp.copy));
    OGB_CUDA_CHECK(cudaEventRecord(wp.copied[s], wp.copy));
    ++wp.copies;
    return 0;
  };
  if (wp.first >= 0) STEP_CHECK(page_in(wp.first));
  for (int l = 0; l < p->num_layers; ++l) {
    LayerPtrs L = p->layers[l];
    const bool paged = wp.first >= 0 && l >= wp.first;
    if (paged) {
      const int s = (l - wp.first) & 1;
      if (l + 1 < p->num_layers) STEP_CHECK(page_in(l + 1));      // one layer ahead: it lands while this layer computes
      OGB_CUDA_CHECK(cudaStreamWaitEvent(cstream, wp.copied[s], 0));
      const char* base = static_cast<const char*>(wp.slot[s]);
      L.qkv_w = base + wp.off[0]; L.o_w = base + wp.off[1]; L.gate_up_w = base + wp.off[2]; L.down_w = base + wp.off[3];
    }
    if (!tp) STEP_CHECK(ogb_rmsnorm_bf16(p->x, nullptr, L.ln1, p->h, T, hid, hid, hid, p->eps, stream));
    STEP_CHECK(ogb_gemm_bf16_wait(p->h, L.qkv_w, p->qkv, L.qkv_b, nullptr, nullptr, T, qkv_n, hid, hid, hid, qkv_n, 0, 0, 0,
                                  (tp && l > 0) ? ready[1] : nullptr, (tp && l > 0) ? ready[1] + 64 : nullptr, 0, p->status, stream));
    STEP_CHECK(ogb_rope_kv_append_bf16(p->qkv, positions, slots, p->cos_sin, L.kv_pool, T, hq, hkv, d, p->rotary_dim,
                                       p->interleaved, 16, p->num_pages * 16, p->max_pos, p->status, stream));
    if (Nd > 0) {
      STEP_CHECK(ogb_paged_decode_bf16(p->qkv, p->attn, L.kv_pool, page_table, ctx_len, Nd, p->max_pages, p->num_pages, hq,
                                       hkv, d, qkv_n, attn_n, p->scale, decode_splits, p->part_o, p->part_ml, p->window,
                                       p->sink, p->status, stream));
    }
    if (Np > 0) {
      if (p->prefill_tc && (d == 64 || d == 128) && attn_n % 8 == 0) {
        STEP_CHECK(ogb_paged_prefill_tc_bf16(qkv_prefill, attn_prefill, L.kv_pool, page_table + static_cast<size_t>(Nd) * p->max_pages,
                                             ctx_len + Nd, cu_q, tile_seq, tile_q0, num_tiles, Np, T - Nd, p->max_pages,
                                             p->num_pages, hq, hkv, d, qkv_n, attn_n, p->scale, p->window, p->sink, p->status, stream));
      } else {
        STEP_CHECK(ogb_paged_prefill_bf16(qkv_prefill, attn_prefill, L.kv_pool, page_table + static_cast<size_t>(Nd) * p->max_pages,
                                          ctx_len + Nd, cu_q, tile_seq, tile_q0, num_tiles, Np, p->max_pages, p->num_pages, hq,
                                          hkv, d, qkv_n, attn_n, p->scale, p->window, p->sink, p->status, stream));
      }
    }
    if (!tp) {
      STEP_CHECK(ogb_gemm_bf16(p->attn, L.o_w, p->x, nullptr, p->x, nullptr, T, hid, attn_n, attn_n, attn_n, hid, hid, 1, 0,
                               p->status, stream));
      STEP_CHECK(ogb_rmsnorm_bf16(p->x, nullptr, L.ln2, p->h, T, hid, hid, hid, p->eps, stream));
    } else {
      STEP_CHECK(ogb_gemm_bf16_scatter(p->attn, L.o_w, T, hid, attn_n, attn_n, attn_n, sc[0], 0, p->status, stream));
      STEP_CHECK(ogb_tp_exchange_norm(rd[0], L.ln2, p->eps, T, hid, tp_chunk, p->tp, nvls, pushed, p->status, stream));
      p->launches_scatter += 2;     // this layer's two row-parallel projections (the second one follows below)
      p->launches_exchange += 2;
    }
    STEP_CHECK(ogb_gemm_bf16_wait(p->h, L.gate_up_w, p->act, nullptr, nullptr, nullptr, T, 2 * p->inter_local, hid, hid, hid,
                                  p->inter_local, 0, 2, p->swiglu_bn, tp ? ready[0] : nullptr, tp ? ready[0] + 64 : nullptr, 0,
                                  p->status, stream));
    if (!tp) {
      STEP_CHECK(ogb_gemm_bf16(p->act, L.down_w, p->x, nullptr, p->x, nullptr, T, hid, p->inter_local, p->inter_local,
                               p->inter_local, hid, hid, 1, 0, p->status, stream));
    } else {
      STEP_CHECK(ogb_gemm_bf16_scatter(p->act, L.down_w, T, hid, p->inter_local, p->inter_local, p->inter_local, sc[1], 0,
                                       p->status, stream));
      const void* next_norm = (l + 1 < p->num_layers) ? p->layers[l + 1].ln1 : p->final_norm;
      STEP_CHECK(ogb_tp_exchange_norm(rd[1], next_norm, p->eps, T, hid, tp_chunk, p->tp, nvls, pushed, p->status, stream));
    }
    if (paged) OGB_CUDA_CHECK(cudaEventRecord(wp.consumed[(l - wp.first) & 1], cstream));
  }
  if (R > 0) {
    if (!tp) {
      // rows that sample: x_last[r] = x[logit_rows[r]] (the embedding gather doubles as a row gather)
      STEP_CHECK(ogb_embedding_bf16(logit_rows, p->x, p->x_last, R, hid, T, p->status, stream));
      STEP_CHECK(ogb_rmsnorm_bf16(p->x_last, nullptr, p->final_norm, p->h_last, R, hid, hid, hid, p->eps, stream));
    } else {
      // the last exchange already applied the final norm: wait for every owner's rows, then gather the rows that sample
      STEP_CHECK(ogb_tp_wait_ready(rd[1], T, p->status, stream));
      STEP_CHECK(ogb_embedding_bf16(logit_rows, p->h, p->h_last, R, hid, T, p->status, stream));
    }
    STEP_CHECK(ogb_gemm_bf16(p->h_last, p->lm_head, p->logits, nullptr, nullptr, nullptr, R, p->vocab, hid, hid, hid,
                             p->vocab, 0, 0, 0, p->status, stream));
  } else if (tp) {
    // nothing samples in this step, but the slot's counters must still be consumed before the next step reuses them
    STEP_CHECK(ogb_tp_wait_ready(rd[1], T, p->status, stream));
  }
  return 0;
}
