// Shared pieces of the paged attention kernels (bf16 pages in attention.cu, e4m3 pages in
// attention_fp8.cu): tile geometry, swizzled shared-memory addressing, ldmatrix / mma.sync wrappers,
// the kernel parameter block and the TMA producer loop.
#pragma once
#include "common.cuh"

namespace ogb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);
int make_tmap_u8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t box_cols);

constexpr int kKvBlock = 64;
constexpr int kPageTokens = 16;
constexpr int kAttnThreads = 160;

// STAGES / QROWS: prefill keeps 64 query rows and a 2-deep ring (two CTAs fit per SM); decode
// keeps 16 query rows and a 3-deep ring.
template <int D, int STAGES, int QROWS>
struct AttnCfg {
  static constexpr int kStages = STAGES;
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = kKvBlock * D * 2;
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kQBytes = QROWS * D * 2;
  static constexpr int kSmemBytes = STAGES * kStageBytes + kQBytes + 1024 /*align*/ + 1024 /*barriers, merge stats*/;
};

OGB_DEVICE void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
OGB_DEVICE void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
OGB_DEVICE void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
OGB_DEVICE void compute_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
template <int THREADS>
OGB_DEVICE void compute_bar_sync_n() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }

// byte offset of (token t, dim d) inside a 64-token K or V tile made of swizzled 2 KB boxes
template <int D>
OGB_DEVICE uint32_t kv_tile_off(int t, int d) {
  return static_cast<uint32_t>((((t >> 4) * (D / 64) + (d >> 6)) << 11) + ((t & 15) << 7) +
                               (((((d & 63) >> 3) ^ (t & 7))) << 4));
}
// byte offset of (row, dim d) inside the Q tile: [half][ROWS][128 B], same swizzle
template <int ROWS>
OGB_DEVICE uint32_t q_tile_off(int row, int d) {
  return static_cast<uint32_t>((((d >> 6) * ROWS + row) << 7) + (((((d & 63) >> 3) ^ (row & 7))) << 4));
}

struct AttnParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int* page_table;
  const int* ctx_len;
  const int* cu_q;
  const int* tile_seq;
  const int* tile_q0;
  int num_tiles;
  int num_seqs;
  int max_pages;
  int64_t num_pages;
  int hq, hkv, group;
  int q_stride, o_stride;
  float scale_log2e;
  int window;               // > 0: a query sees only the last `window` keys ...
  int sink;                 // ... and, with window > 0, the first `sink` keys as well (attention sinks)
  int num_splits;
  float* part_o;
  float* part_ml;
  int* status;
  const float* kv_scales;   // one-byte pages only: [pages, kv_heads, 2] fp32 (K scale, V scale)
  int kv_fmt;               // one-byte pages only: 0 = e4m3, 1 = int8
  unsigned long long* dbg;  // optional (tcgen05 prefill): per-role wait / work nanoseconds of the CTA (dbg_tile, head 0)
  int dbg_tile;
};

// Sliding window with attention sinks (the retention policy of crates/onnx-genai-kv/src/paged_cache.rs:483-585, done
// here as a mask plus a block walk instead of a compacted buffer): a query at position qpos sees keys
// [0, sink) and (qpos - window, qpos].
OGB_DEVICE bool key_visible(int col, int qpos, int ctx, int window, int sink) {
  return col <= qpos && col < ctx && (window <= 0 || col > qpos - window || col < sink);
}
// The scheduler may release the pages that lie wholly between the sinks and the window (their page-table entries
// become -1).  `kv_lo` is the first key any query of the CTA sees inside its window; a page index in the gap is replaced
// by the window's first page, whose keys are masked where they stand in for gap keys.
OGB_DEVICE int skip_gap_page(int pi, int window, int sink, int kv_lo) {
  if (window > 0) {
    const int gap_lo = (sink + kPageTokens - 1) / kPageTokens, gap_hi = kv_lo / kPageTokens;
    if (pi >= gap_lo && pi < gap_hi) pi = gap_hi;
  }
  return pi;
}
// The key blocks a CTA walks: the sink blocks, then the blocks from the window's first key to the last key.
struct KvBlocks {
  int nsink, first, count, kv_lo;
  OGB_DEVICE int phys(int j) const { return j < nsink ? j : first + (j - nsink); }
};
OGB_DEVICE KvBlocks make_kv_blocks(int window, int sink, int kv_lo, int kv_end, int block) {
  KvBlocks r;
  const int last = (kv_end + block - 1) / block;
  r.kv_lo = (window > 0) ? kv_lo : 0;
  r.first = r.kv_lo / block;
  r.nsink = (window > 0 && sink > 0) ? (min(sink, kv_end) + block - 1) / block : 0;
  if (r.first <= r.nsink) { r.first = 0; r.nsink = 0; }      // the window reaches the sinks: one contiguous walk
  r.count = r.nsink + last - r.first;
  return r;
}

// Producer: stream logical blocks [j_begin, j_end) of one sequence / kv head into the ring.
template <class Cfg>
OGB_DEVICE bool attn_produce(const CUtensorMap* kv_map, const AttnParams& p, uint8_t* stages, uint64_t* full_bar,
                             uint64_t* empty_bar, int seq, int kvh, int ctx, const KvBlocks& blocks, int j_begin, int j_end) {
  const int n_pages = (ctx + kPageTokens - 1) / kPageTokens;
  const int* table = p.page_table + static_cast<size_t>(seq) * p.max_pages;
  int stage = 0;
  uint32_t phase = 0;
  for (int j = j_begin; j < j_end; ++j) {
    const int b = blocks.phys(j);
    if (!mbar_wait(&empty_bar[stage], phase ^ 1)) return false;
    uint8_t* sk = stages + stage * Cfg::kStageBytes;
    uint8_t* sv = sk + Cfg::kTileBytes;
    mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int pi = b * 4 + i;
      if (pi > n_pages - 1) pi = n_pages - 1;  // tail: re-read the last page, masked later
      if (pi > p.max_pages - 1) pi = p.max_pages - 1;
      pi = skip_gap_page(pi, p.window, p.sink, blocks.kv_lo);
      int64_t page = table[pi];
      if (page < 0 || page >= p.num_pages) {
        atomicOr(p.status, kStatusIndexOutOfRange);
        page = 0;
      }
      const int row_k = static_cast<int>(((page * p.hkv + kvh) * 2) * kPageTokens);
#pragma unroll
      for (int h = 0; h < Cfg::kHalves; ++h) {
        tma_load_2d(sk + ((i * Cfg::kHalves + h) << 11), kv_map, &full_bar[stage], h * 64, row_k);
        tma_load_2d(sv + ((i * Cfg::kHalves + h) << 11), kv_map, &full_bar[stage], h * 64, row_k + kPageTokens);
      }
    }
    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
  }
  return true;
}

// tcgen05 decode over e4m3 pages (attention_fp8_tc.cu): `p` fully filled, at most 8 query heads per KV head, head_dim 128.
int launch_decode_e4m3_tc(const AttnParams& p, const void* pool, void* stream);

}  // namespace ogb
