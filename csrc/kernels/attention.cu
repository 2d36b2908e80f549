// Paged grouped-query attention for sm_100a, reading KV pages in place.
//
// The reference keeps device KV as one contiguous buffer per layer and only *materialises*
// pages (crates/onnx-genai-kv/src/paged_cache.rs:298-420); its attention kernels are
// flash_attention_{f32,f16,bf16,f16_tc} for prefill (crates/onnx-runtime-ep-cuda/src/kernels/
// flash_attention.rs:1-60,280-345) and gqa_decode_attention_* split-K + merge for decode
// (kernels/gqa_decode.rs:1-57, gqa_decode_bf16.rs).  Here both phases walk a page table:
//
//   pool layout  [pages, kv_heads, 2 (K|V), 16 tokens, head_dim]  bf16
//   a KV "block" 64 tokens = 4 pages; each page half (16 tokens x 64 dims = 2 KB) is one TMA
//                box, landed 128-byte swizzled so ldmatrix reads it bank-conflict free
//   warp 4       producer: one lane looks up page ids and issues the TMA loads into a 3-stage ring
//   warps 0..3   consumers: QK^T and PV on tensor cores (m16n8k16 bf16, fp32 accumulate),
//                online softmax in the log2 domain
//   prefill      one CTA = 64 query rows of one head; causal (+ optional sliding window)
//   decode       one CTA = (sequence, kv head, KV split); the G query heads of the group are the
//                MMA rows, each warp takes one page of every block, warps merge at the end;
//                splits > 1 write partials that paged_decode_merge_kernel combines
// Page ids are bounds-checked: a bad id raises kStatusIndexOutOfRange and page 0 is read instead.
#include <mutex>
#include <unordered_map>

#include "attention_common.cuh"
#include "ogb_kernels.h"

namespace ogb {

// ------------------------------------------------------------------------------------------
// prefill: ROWS query rows x one head per CTA.  The scheduler emits 64-row tiles; ROWS = 64 gives one CTA per
// tile, ROWS = 32 / 16 give two / four CTAs per tile with two / one compute warps each.  A warp's work is
// the same in every variant (16 query rows against each 64-key block), so when tiles x heads cannot fill the
// machine -- few heads per rank under tensor parallelism, or one short prompt -- the narrower variants cut
// the kernel's duration by spreading the same warps over more SMs.
// ------------------------------------------------------------------------------------------
template <int D, int ROWS>
__global__ void __launch_bounds__((ROWS / 16 + 1) * 32, 2) paged_prefill_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                              const AttnParams p) {
  using Cfg = AttnCfg<D, 2, 64>;
  constexpr int kWarps = ROWS / 16;          // compute warps; warp kWarps is the TMA producer
  constexpr int kSub = 64 / ROWS;            // CTAs per 64-row tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* sq = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sq + Cfg::kQBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;

  const int tile = blockIdx.x / kSub;
  if (tile >= p.num_tiles) return;
  const int head = blockIdx.y;
  const int kvh = head / p.group;
  const int seq = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile] + (blockIdx.x % kSub) * ROWS;
  const int q_begin = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - q_begin;
  const int ctx = p.ctx_len[seq];
  const int rows = min(ROWS, q_len - q0);
  const int pos0 = ctx - q_len + q0;
  if (rows <= 0 || ctx <= 0) return;
  const int kv_end = min(ctx, pos0 + rows);
  const KvBlocks blocks = make_kv_blocks(p.window, p.sink, max(0, pos0 - p.window + 1), kv_end, kKvBlock);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], kWarps); }
    mbar_fence_init();
    tma_prefetch_desc(&kv_map);
  }
  __syncthreads();

  if (warp == kWarps) {
    if (lane == 0) {
      if (!attn_produce<Cfg>(&kv_map, p, stages, full_bar, empty_bar, seq, kvh, ctx, blocks, 0, blocks.count))
        atomicOr(p.status, kStatusWaitTimeout);
    }
    return;
  }

  // ---- stage Q (swizzled) and pull the A fragments into registers ----
  {
    const __nv_bfloat16* qsrc = p.q + static_cast<size_t>(q_begin + q0) * p.q_stride + head * D;
    for (int idx = threadIdx.x; idx < ROWS * (D / 8); idx += kWarps * 32) {
      const int row = idx / (D / 8), ch = idx % (D / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < rows) v = *reinterpret_cast<const uint4*>(qsrc + static_cast<size_t>(row) * p.q_stride + ch * 8);
      *reinterpret_cast<uint4*>(sq + q_tile_off<64>(row, ch * 8)) = v;
    }
  }
  compute_bar_sync_n<kWarps * 32>();
  uint32_t qf[D / 16][4];
  {
    const uint32_t sq_u = smem_u32(sq);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int row = 16 * warp + (lane & 15);
      const int d = 16 * kk + 8 * (lane >> 4);
      ldsm_x4(sq_u + q_tile_off<64>(row, d), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
  }

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_a = 16 * warp + (lane >> 2);
  const int qpos_a = pos0 + row_a, qpos_b = pos0 + row_a + 8;

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int jb = 0; jb < blocks.count; ++jb) {
    const int b = blocks.phys(jb);
    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase))) { ok = false; break; }
    const uint32_t sk = smem_u32(stages + stage * Cfg::kStageBytes);
    const uint32_t sv = sk + Cfg::kTileBytes;
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        const int mi = lane >> 3;
        const int t = 16 * jp + 8 * (mi >> 1) + (lane & 7);
        const int d = 16 * kk + 8 * (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sk + kv_tile_off<D>(t, d), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * jp], qf[kk], b0, b1);
        mma_bf16_16816(s[2 * jp + 1], qf[kk], b2, b3);
      }
    }
    // scale into the log2 domain and mask
    const int kv_base = b * kKvBlock;
    const bool need_mask = (kv_base + kKvBlock - 1 > pos0 + 16 * warp) || (kv_base + kKvBlock > ctx) || (p.window > 0);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[j][e] * p.scale_log2e;
        if (need_mask) {
          const int col = kv_base + 8 * j + 2 * (lane & 3) + (e & 1);
          const int qpos = (e < 2) ? qpos_a : qpos_b;
          if (!key_visible(col, qpos, ctx, p.window, p.sink)) v = -INFINITY;
        }
        s[j][e] = v;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * r], s[j][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run[r] - m_use);
      m_run[r] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j][2 * r] = exp2f(s[j][2 * r] - m_use);
        s[j][2 * r + 1] = exp2f(s[j][2 * r + 1] - m_use);
        sum += s[j][2 * r] + s[j][2 * r + 1];
      }
      l_run[r] = l_run[r] * alpha + sum;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) { o[j][2 * r] *= alpha; o[j][2 * r + 1] *= alpha; }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jd = 0; jd < D / 16; ++jd) {
        const int mi = lane >> 3;
        const int t = 16 * kk + 8 * (mi & 1) + (lane & 7);
        const int d = 16 * jd + 8 * (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sv + kv_tile_off<D>(t, d), b0, b1, b2, b3);
        mma_bf16_16816(o[2 * jd], a, b0, b1);
        mma_bf16_16816(o[2 * jd + 1], a, b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
  }
  if (!ok) {
    if (lane == 0) atomicOr(p.status, kStatusWaitTimeout);
    return;
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = (l > 0.f) ? 1.f / l : 0.f;
    const int row = row_a + 8 * r;
    if (row < rows) {
      __nv_bfloat16* dst = p.out + static_cast<size_t>(q_begin + q0 + row) * p.o_stride + head * D + 2 * (lane & 3);
#pragma unroll
      for (int j = 0; j < D / 8; ++j)
        *reinterpret_cast<uint32_t*>(dst + 8 * j) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------------
// decode: one query token per sequence; MMA rows = the G query heads sharing a kv head
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kAttnThreads, 2) paged_decode_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                     const AttnParams p) {
  using Cfg = AttnCfg<D, 3, 16>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* sq = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sq + Cfg::kQBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  float* sm_ml = reinterpret_cast<float*>(empty_bar + Cfg::kStages);  // [4 warps][16 rows][2]

  const int seq = blockIdx.x / p.num_splits;
  const int split = blockIdx.x % p.num_splits;
  const int kvh = blockIdx.y;
  const int G = p.group;
  const int ctx = p.ctx_len[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  int b_begin = 0, b_end = 0;            // logical blocks of this split (sink blocks first, then the window's)
  KvBlocks blocks{0, 0, 0, 0};
  if (ctx > 0) {
    blocks = make_kv_blocks(p.window, p.sink, max(0, ctx - p.window), ctx, kKvBlock);
    const int per = (blocks.count + p.num_splits - 1) / p.num_splits;
    b_begin = split * per;
    b_end = min(b_begin + per, blocks.count);
  }
  const int kv_lo = blocks.kv_lo;
  if (b_begin >= b_end) {
    // nothing to do for this split (or an inactive row): publish an empty partial
    if (p.num_splits > 1 && ctx > 0) {
      for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
        const int r = idx / D, d = idx % D;
        const size_t slot = (static_cast<size_t>(seq) * p.hq + kvh * G + r) * p.num_splits + split;
        p.part_o[slot * D + d] = 0.f;
        if (d == 0) { p.part_ml[slot * 2] = -INFINITY; p.part_ml[slot * 2 + 1] = 0.f; }
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 4); }
    mbar_fence_init();
    tma_prefetch_desc(&kv_map);
  }
  __syncthreads();

  if (warp == 4) {
    if (lane == 0) {
      if (!attn_produce<Cfg>(&kv_map, p, stages, full_bar, empty_bar, seq, kvh, ctx, blocks, b_begin, b_end))
        atomicOr(p.status, kStatusWaitTimeout);
    }
    return;
  }

  {
    const __nv_bfloat16* qsrc = p.q + static_cast<size_t>(seq) * p.q_stride + kvh * G * D;
    for (int idx = threadIdx.x; idx < 16 * (D / 8); idx += 128) {
      const int row = idx / (D / 8), ch = idx % (D / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < G) v = *reinterpret_cast<const uint4*>(qsrc + row * D + ch * 8);
      *reinterpret_cast<uint4*>(sq + q_tile_off<16>(row, ch * 8)) = v;
    }
  }
  compute_bar_sync();
  uint32_t qf[D / 16][4];
  {
    const uint32_t sq_u = smem_u32(sq);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int row = (lane & 15);
      const int d = 16 * kk + 8 * (lane >> 4);
      ldsm_x4(sq_u + q_tile_off<16>(row, d), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  const int sink = (p.window > 0) ? p.sink : 0;
  for (int jb = b_begin; jb < b_end; ++jb) {
    const int b = blocks.phys(jb);
    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase))) { ok = false; break; }
    const int tok0 = b * kKvBlock + 16 * warp;  // first token of this warp's page in the block
    if (tok0 < ctx && (tok0 + 16 > kv_lo || tok0 < sink)) {
      const uint32_t sk = smem_u32(stages + stage * Cfg::kStageBytes);
      const uint32_t sv = sk + Cfg::kTileBytes;
      float s[2][4];
      s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int mi = lane >> 3;
        const int t = 16 * warp + 8 * (mi >> 1) + (lane & 7);
        const int d = 16 * kk + 8 * (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sk + kv_tile_off<D>(t, d), b0, b1, b2, b3);
        mma_bf16_16816(s[0], qf[kk], b0, b1);
        mma_bf16_16816(s[1], qf[kk], b2, b3);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = tok0 + 8 * j + 2 * (lane & 3) + (e & 1);
          const bool valid = (col < ctx) && (col >= kv_lo || col < sink);
          s[j][e] = valid ? s[j][e] * p.scale_log2e : -INFINITY;
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[r], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_run[r] - m_use);
        m_run[r] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          s[j][2 * r] = exp2f(s[j][2 * r] - m_use);
          s[j][2 * r + 1] = exp2f(s[j][2 * r + 1] - m_use);
          sum += s[j][2 * r] + s[j][2 * r + 1];
        }
        l_run[r] = l_run[r] * alpha + sum;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) { o[j][2 * r] *= alpha; o[j][2 * r + 1] *= alpha; }
      }
      uint32_t a[4];
      a[0] = pack_bf16(s[0][0], s[0][1]);
      a[1] = pack_bf16(s[0][2], s[0][3]);
      a[2] = pack_bf16(s[1][0], s[1][1]);
      a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int jd = 0; jd < D / 16; ++jd) {
        const int mi = lane >> 3;
        const int t = 16 * warp + 8 * (mi & 1) + (lane & 7);
        const int d = 16 * jd + 8 * (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sv + kv_tile_off<D>(t, d), b0, b1, b2, b3);
        mma_bf16_16816(o[2 * jd], a, b0, b1);
        mma_bf16_16816(o[2 * jd + 1], a, b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
  }
  if (!ok && lane == 0) atomicOr(p.status, kStatusWaitTimeout);

  // ---- merge the four warps (each saw a disjoint quarter of the keys) ----
  compute_bar_sync();  // every stage has been consumed: the ring can be reused as scratch
  float* sm_o = reinterpret_cast<float*>(stages);  // [4][16][D] fp32
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = (lane >> 2) + 8 * r;
    if ((lane & 3) == 0) {
      sm_ml[(warp * 16 + row) * 2] = m_run[r];
      sm_ml[(warp * 16 + row) * 2 + 1] = l;
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      float* dst = sm_o + (static_cast<size_t>(warp * 16 + row)) * D + 8 * j + 2 * (lane & 3);
      dst[0] = o[j][2 * r];
      dst[1] = o[j][2 * r + 1];
    }
  }
  compute_bar_sync();
  for (int idx = threadIdx.x; idx < G * D; idx += 128) {
    const int row = idx / D, d = idx % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, sm_ml[(w * 16 + row) * 2]);
    const float m_use = (mx == -INFINITY) ? 0.f : mx;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = exp2f(sm_ml[(w * 16 + row) * 2] - m_use);
      acc += wgt * sm_o[(static_cast<size_t>(w * 16 + row)) * D + d];
      l += wgt * sm_ml[(w * 16 + row) * 2 + 1];
    }
    const int head = kvh * G + row;
    if (p.num_splits == 1) {
      p.out[static_cast<size_t>(seq) * p.o_stride + head * D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
    } else {
      const size_t slot = (static_cast<size_t>(seq) * p.hq + head) * p.num_splits + split;
      p.part_o[slot * D + d] = acc;
      if (d == 0) { p.part_ml[slot * 2] = mx; p.part_ml[slot * 2 + 1] = l; }
    }
  }
}

__global__ void paged_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out, int hq, int D,
                                          int num_splits, int o_stride) {
  const int seq = blockIdx.x, head = blockIdx.y;
  if (ctx_len[seq] <= 0) return;
  const size_t base = (static_cast<size_t>(seq) * hq + head) * num_splits;
  float mx = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mx = fmaxf(mx, part_ml[(base + s) * 2]);
  const float m_use = (mx == -INFINITY) ? 0.f : mx;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float w = exp2f(part_ml[(base + s) * 2] - m_use);
      acc += w * part_o[(base + s) * D + d];
      l += w * part_ml[(base + s) * 2 + 1];
    }
    out[static_cast<size_t>(seq) * o_stride + head * D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
  }
}

// ------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------
struct TmapKey {
  const void* base;
  uint64_t rows;
  int d;
  bool operator==(const TmapKey& o) const { return base == o.base && rows == o.rows && d == o.d; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (std::hash<uint64_t>()(k.rows) * 1315423911u) ^ static_cast<size_t>(k.d);
  }
};

static int get_pool_tmap(const void* pool, int64_t num_pages, int hkv, int d, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const uint64_t rows = static_cast<uint64_t>(num_pages) * hkv * 2 * kPageTokens;
  TmapKey key{pool, rows, d};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  CUtensorMap m;
  int rc = make_tmap_bf16_2d(&m, pool, rows, d, d, kPageTokens, 64);
  if (rc != 0) return rc;
  cache.emplace(key, m);
  *out = m;
  return 0;
}

template <int D, int ROWS>
static int launch_prefill_rows(const CUtensorMap& map, const AttnParams& p, cudaStream_t stream) {
  using Cfg = AttnCfg<D, 2, 64>;
  static bool attr_set = false;
  if (!attr_set) {
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_prefill_kernel<D, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_prefill_kernel<D, ROWS>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    attr_set = true;
  }
  dim3 grid(p.num_tiles * (64 / ROWS), p.hq);
  paged_prefill_kernel<D, ROWS><<<grid, (ROWS / 16 + 1) * 32, Cfg::kSmemBytes, stream>>>(map, p);
  return static_cast<int>(cudaGetLastError());
}

template <int D>
static int launch_prefill(const CUtensorMap& map, const AttnParams& p, cudaStream_t stream) {
  // two CTAs fit per SM: below ~3/4 of that many 64-row CTAs, narrower CTAs finish sooner (see the kernel comment)
  const long ctas64 = static_cast<long>(p.num_tiles) * p.hq;
  const long slots = 2L * ogb_num_sms();
  if (4 * ctas64 >= 3 * slots) return launch_prefill_rows<D, 64>(map, p, stream);
  if (8 * ctas64 >= 3 * slots) return launch_prefill_rows<D, 32>(map, p, stream);
  return launch_prefill_rows<D, 16>(map, p, stream);
}
template <int D>
static int launch_decode(const CUtensorMap& map, const AttnParams& p, cudaStream_t stream) {
  using Cfg = AttnCfg<D, 3, 16>;
  static bool attr_set = false;
  if (!attr_set) {
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_kernel<D>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    attr_set = true;
  }
  dim3 grid(p.num_seqs * p.num_splits, p.hkv);
  paged_decode_kernel<D><<<grid, kAttnThreads, Cfg::kSmemBytes, stream>>>(map, p);
  int rc = static_cast<int>(cudaGetLastError());
  if (rc != 0) return rc;
  if (p.num_splits > 1) {
    dim3 mgrid(p.num_seqs, p.hq);
    paged_decode_merge_kernel<<<mgrid, D, 0, stream>>>(p.part_o, p.part_ml, p.ctx_len, p.out, p.hq, D, p.num_splits, p.o_stride);
    rc = static_cast<int>(cudaGetLastError());
  }
  return rc;
}

}  // namespace ogb

using namespace ogb;

extern "C" int ogb_paged_prefill_bf16(const void* q, void* out, const void* pool, const int* page_table, const int* ctx_len,
                                      const int* cu_q, const int* tile_seq, const int* tile_q0, int num_tiles, int num_seqs,
                                      int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride, int o_stride,
                                      float scale, int window, int sink, int* status, void* stream) {
  if (num_tiles <= 0) return 0;
  if ((d != 64 && d != 128) || hkv <= 0 || hq % hkv != 0 || (q_stride % 8) != 0 || (o_stride % 2) != 0) return -3;
  CUtensorMap map;
  int rc = get_pool_tmap(pool, num_pages, hkv, d, &map);
  if (rc != 0) return rc;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.page_table = page_table; p.ctx_len = ctx_len; p.cu_q = cu_q; p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.num_tiles = num_tiles; p.num_seqs = num_seqs; p.max_pages = max_pages; p.num_pages = num_pages;
  p.hq = hq; p.hkv = hkv; p.group = hq / hkv; p.q_stride = q_stride; p.o_stride = o_stride;
  p.scale_log2e = scale * 1.4426950408889634f; p.window = window; p.sink = window > 0 ? sink : 0; p.num_splits = 1; p.status = status;
  return d == 128 ? launch_prefill<128>(map, p, static_cast<cudaStream_t>(stream))
                  : launch_prefill<64>(map, p, static_cast<cudaStream_t>(stream));
}

extern "C" int ogb_paged_decode_bf16(const void* q, void* out, const void* pool, const int* page_table, const int* ctx_len,
                                     int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride,
                                     int o_stride, float scale, int num_splits, float* part_o, float* part_ml, int window,
                                     int sink, int* status, void* stream) {
  if (num_seqs <= 0) return 0;
  if ((d != 64 && d != 128) || hkv <= 0 || hq % hkv != 0 || hq / hkv > 16 || (q_stride % 8) != 0) return -3;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return -4;
  CUtensorMap map;
  int rc = get_pool_tmap(pool, num_pages, hkv, d, &map);
  if (rc != 0) return rc;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.page_table = page_table; p.ctx_len = ctx_len;
  p.num_seqs = num_seqs; p.max_pages = max_pages; p.num_pages = num_pages;
  p.hq = hq; p.hkv = hkv; p.group = hq / hkv; p.q_stride = q_stride; p.o_stride = o_stride;
  p.scale_log2e = scale * 1.4426950408889634f; p.window = window; p.sink = window > 0 ? sink : 0; p.num_splits = num_splits;
  p.part_o = part_o; p.part_ml = part_ml; p.status = status;
  return d == 128 ? launch_decode<128>(map, p, static_cast<cudaStream_t>(stream))
                  : launch_decode<64>(map, p, static_cast<cudaStream_t>(stream));
}
