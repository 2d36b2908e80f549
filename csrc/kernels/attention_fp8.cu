// Paged GQA attention over e4m3 KV pages with one fp32 scale per (page, kv head, K|V).
//
// The reference quantises KV only in host page storage with a software codec (one scale per
// (head, token slot), crates/onnx-genai-kv/src/page_table.rs:250-297,776-832, src/fp8.rs:5-198) and
// its attention kernels never read quantised KV (group_query_attention.rs:1140-1200 rejects
// k/v_quant_type != NONE).  Here the pages stay e4m3 in HBM (half the bytes of bf16 on the decode
// critical path) and are expanded on chip:
//   pool   [pages, kv_heads, 2, 16 tokens, 128] uint8 e4m3, scales [pages, kv_heads, 2] fp32
//   TMA    one 2 KB box per (page, K|V), 128-byte swizzled, 3-stage (decode) / 2-stage (prefill) ring
//   expand each consumer warp turns fp8 pairs into bf16 (exact: every e4m3 value is a bf16 value) and
//          writes them in the bf16 tile layout the shared ldmatrix / mma.sync code reads
//   scale  K scale multiplies the scores of the page's 16 keys, V scale multiplies their
//          probabilities before P.V; the running row sum uses the unscaled probabilities
// Head dimension 128 only.  Same bounded waits and status word as the bf16 kernels.
#include <cuda_fp8.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "attention_common.cuh"
#include "ogb_kernels.h"

namespace ogb {

constexpr int kD = 128;
constexpr int kRawPage = kPageTokens * kD;           // 2 KB of e4m3 per page side
constexpr int kRawStage = 4 * 2 * kRawPage;          // 4 pages x (K, V) = 16 KB
constexpr int kWorkPage = kPageTokens * kD * 2;      // 4 KB of bf16 per page side

// One-byte values -> bf16 with integer and half-rate-free arithmetic only (no cvt instructions, which issue at a quarter
// of the ALU rate and made the expansion, not HBM, the limit of these kernels).
//
// e4m3 (s eeee mmm, bias 7): the seven magnitude bits dropped at bit 4 of a bf16 (s eeeeeeee mmmmmmm, bias 127) read as the
// same number times 2^-120 -- for subnormals too, which land on bf16 subnormals -- so one exact multiply by 2^120 finishes
// the conversion.  Input word t holds the two bytes at bits 15:8 and 31:24.
OGB_DEVICE uint32_t e4m3x2_to_bf16x2(uint32_t t) {
  uint32_t bits = (t & 0x80008000u) | ((t >> 4) & 0x07f007f0u);
  const uint32_t two120 = 0x7B807B80u;
  __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&bits), *reinterpret_cast<const __nv_bfloat162*>(&two120));
  return *reinterpret_cast<uint32_t*>(&v);
}
// int8 (two's complement): with u = low seven bits, bf16(128 + u) is 0x4300 | u exactly, and the value is that minus
// 128 (byte >= 0) or 256 (byte < 0), i.e. minus bf16 bits 0x4300 | (byte & 0x80).  Input word t holds the two bytes at
// bits 7:0 and 23:16.
OGB_DEVICE uint32_t i8x2_to_bf16x2(uint32_t t) {
  uint32_t x = 0x43004300u | (t & 0x007f007fu);
  uint32_t c = 0x43004300u | (t & 0x00800080u);
  __nv_bfloat162 v = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&x), *reinterpret_cast<__nv_bfloat162*>(&c));
  return *reinterpret_cast<uint32_t*>(&v);
}

// e5m2 (s eeeee mm, bias 15): the seven magnitude bits dropped at bit 5 of a bf16 read as the same number times 2^-112
// (subnormals land on bf16 subnormals), so one exact multiply by 2^112 finishes the conversion.  Input word as for e4m3.
OGB_DEVICE uint32_t e5m2x2_to_bf16x2(uint32_t t) {
  uint32_t bits = (t & 0x80008000u) | ((t >> 3) & 0x0fe00fe0u);
  const uint32_t two112 = 0x77807780u;
  __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&bits), *reinterpret_cast<const __nv_bfloat162*>(&two112));
  return *reinterpret_cast<uint32_t*>(&v);
}
OGB_DEVICE void cvt16_e5m2_bf16(const uint4& raw, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = e5m2x2_to_bf16x2(__byte_perm(w[i], 0, 0x1404));
    o[2 * i + 1] = e5m2x2_to_bf16x2(__byte_perm(w[i], 0, 0x3424));
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// 16 e4m3 bytes -> 16 bf16, as two 16-byte vectors
OGB_DEVICE void cvt16_e4m3_bf16(const uint4& raw, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = e4m3x2_to_bf16x2(__byte_perm(w[i], 0, 0x1404));       // bytes 0, 1 -> bits 15:8, 31:24
    o[2 * i + 1] = e4m3x2_to_bf16x2(__byte_perm(w[i], 0, 0x3424));   // bytes 2, 3
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// 16 int8 bytes -> 16 bf16 (exact: |v| <= 128 fits bf16's 8 significant bits)
OGB_DEVICE void cvt16_i8_bf16(const uint4& raw, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = i8x2_to_bf16x2(__byte_perm(w[i], 0, 0x4140));         // bytes 0, 1 -> bits 7:0, 23:16
    o[2 * i + 1] = i8x2_to_bf16x2(__byte_perm(w[i], 0, 0x4342));     // bytes 2, 3
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// Expand one raw page side (16 tokens x 128 one-byte values, 128-byte swizzled rows) into a bf16 page tile
// ([2 halves][16 rows][128 B], same swizzle), using `nthreads` threads starting at `tid`.  fmt 0: e4m3, 1: int8, 2: e5m2.
OGB_DEVICE void expand_page(const uint8_t* raw, uint8_t* work, int tid, int nthreads, int fmt) {
  for (int i = tid; i < kPageTokens * 8; i += nthreads) {   // 16 rows x 8 chunks of 16 bytes
    const int r = i >> 3, c = i & 7;
    const uint4 v = *reinterpret_cast<const uint4*>(raw + r * 128 + ((c ^ (r & 7)) << 4));
    uint4 lo, hi;
    if (fmt == 0) cvt16_e4m3_bf16(v, lo, hi);
    else if (fmt == 1) cvt16_i8_bf16(v, lo, hi);
    else cvt16_e5m2_bf16(v, lo, hi);
    const int d0 = c * 16;
    *reinterpret_cast<uint4*>(work + kv_tile_off<kD>(r, d0)) = lo;
    *reinterpret_cast<uint4*>(work + kv_tile_off<kD>(r, d0 + 8)) = hi;
  }
}

OGB_DEVICE bool fp8_produce(const CUtensorMap* kv_map, const AttnParams& p, uint8_t* stages, uint64_t* full_bar,
                            uint64_t* empty_bar, int nstages, int seq, int kvh, int ctx, int b_begin, int b_end, int kv_lo) {
  const int n_pages = (ctx + kPageTokens - 1) / kPageTokens;
  const int* table = p.page_table + static_cast<size_t>(seq) * p.max_pages;
  int stage = 0;
  uint32_t phase = 0;
  for (int b = b_begin; b < b_end; ++b) {
    if (!mbar_wait(&empty_bar[stage], phase ^ 1)) return false;
    uint8_t* s = stages + stage * kRawStage;
    mbar_expect_tx(&full_bar[stage], kRawStage);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int pi = min(min(b * 4 + i, n_pages - 1), p.max_pages - 1);
      pi = skip_gap_page(pi, p.window, p.sink, kv_lo);
      int64_t page = table[pi];
      if (page < 0 || page >= p.num_pages) { atomicOr(p.status, kStatusIndexOutOfRange); page = 0; }
      const int row_k = static_cast<int>(((page * p.hkv + kvh) * 2) * kPageTokens);
      tma_load_2d(s + i * kRawPage, kv_map, &full_bar[stage], 0, row_k);
      tma_load_2d(s + (4 + i) * kRawPage, kv_map, &full_bar[stage], 0, row_k + kPageTokens);
    }
    if (++stage == nstages) { stage = 0; phase ^= 1; }
  }
  return true;
}

OGB_DEVICE int64_t page_of(const AttnParams& p, int seq, int ctx, int pi, int kv_lo) {
  const int n_pages = (ctx + kPageTokens - 1) / kPageTokens;
  pi = skip_gap_page(min(min(pi, n_pages - 1), p.max_pages - 1), p.window, p.sink, kv_lo);
  int64_t page = p.page_table[static_cast<size_t>(seq) * p.max_pages + pi];
  return (page < 0 || page >= p.num_pages) ? 0 : page;
}

// ------------------------------------------------------------------------------------------
// decode
// ------------------------------------------------------------------------------------------
constexpr int kDecStages = 3;
constexpr int kDecSmem = kDecStages * kRawStage + 4 * 2 * kWorkPage + 16 * kD * 2 + 1024 + 1024;

__global__ void __launch_bounds__(kAttnThreads) paged_decode_fp8_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                         const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* work = smem + kDecStages * kRawStage;          // [4 warps][K 4 KB | V 4 KB]
  uint8_t* sq = work + 4 * 2 * kWorkPage;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sq + 16 * kD * 2);
  uint64_t* empty_bar = full_bar + kDecStages;
  float* sm_ml = reinterpret_cast<float*>(empty_bar + kDecStages);

  const int seq = blockIdx.x / p.num_splits, split = blockIdx.x % p.num_splits, kvh = blockIdx.y;
  const int G = p.group;
  const int ctx = p.ctx_len[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int b_begin = 0, b_end = 0;
  const int kv_lo = (p.window > 0) ? max(0, ctx - p.window) : 0;     // first key inside the window
  const int sink = (p.window > 0) ? p.sink : 0;
  if (ctx > 0) {
    const int first = (sink > 0) ? 0 : kv_lo / kKvBlock;            // with sinks the walk starts at key 0 (gap blocks are masked)
    const int last = (ctx + kKvBlock - 1) / kKvBlock;
    const int per = (last - first + p.num_splits - 1) / p.num_splits;
    b_begin = first + split * per;
    b_end = min(b_begin + per, last);
  }
  if (b_begin >= b_end) {
    if (p.num_splits > 1 && ctx > 0) {
      for (int idx = threadIdx.x; idx < G * kD; idx += blockDim.x) {
        const int r = idx / kD, d = idx % kD;
        const size_t slot = (static_cast<size_t>(seq) * p.hq + kvh * G + r) * p.num_splits + split;
        p.part_o[slot * kD + d] = 0.f;
        if (d == 0) { p.part_ml[slot * 2] = -INFINITY; p.part_ml[slot * 2 + 1] = 0.f; }
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < kDecStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 4); }
    mbar_fence_init();
    tma_prefetch_desc(&kv_map);
  }
  __syncthreads();
  if (warp == 4) {
    if (lane == 0 && !fp8_produce(&kv_map, p, stages, full_bar, empty_bar, kDecStages, seq, kvh, ctx, b_begin, b_end, kv_lo))
      atomicOr(p.status, kStatusWaitTimeout);
    return;
  }
  {
    const __nv_bfloat16* qsrc = p.q + static_cast<size_t>(seq) * p.q_stride + kvh * G * kD;
    for (int idx = threadIdx.x; idx < 16 * (kD / 8); idx += 128) {
      const int row = idx / (kD / 8), ch = idx % (kD / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < G) v = *reinterpret_cast<const uint4*>(qsrc + row * kD + ch * 8);
      *reinterpret_cast<uint4*>(sq + q_tile_off<16>(row, ch * 8)) = v;
    }
  }
  compute_bar_sync();
  uint32_t qf[kD / 16][4];
  {
    const uint32_t sq_u = smem_u32(sq);
#pragma unroll
    for (int kk = 0; kk < kD / 16; ++kk)
      ldsm_x4(sq_u + q_tile_off<16>(lane & 15, 16 * kk + 8 * (lane >> 4)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
  float o[kD / 8][4];
#pragma unroll
  for (int j = 0; j < kD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  uint8_t* wk = work + warp * 2 * kWorkPage;
  uint8_t* wv = wk + kWorkPage;
  const uint32_t sk = smem_u32(wk), sv = smem_u32(wv);

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  // The scales of a page sit behind two dependent global loads (page table, then scale table).  They are fetched one
  // block ahead so that their latency overlaps the expansion and the MMAs of the current block instead of stalling it.
  float ks_next, vs_next;
  {
    const int64_t page = page_of(p, seq, ctx, b_begin * 4 + warp, kv_lo);
    ks_next = p.kv_scales[(page * p.hkv + kvh) * 2];
    vs_next = p.kv_scales[(page * p.hkv + kvh) * 2 + 1];
  }
  for (int b = b_begin; b < b_end; ++b) {
    const float ks = ks_next * p.scale_log2e, vs = vs_next;
    if (b + 1 < b_end) {
      const int64_t page = page_of(p, seq, ctx, (b + 1) * 4 + warp, kv_lo);
      ks_next = p.kv_scales[(page * p.hkv + kvh) * 2];
      vs_next = p.kv_scales[(page * p.hkv + kvh) * 2 + 1];
    }
    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase))) { ok = false; break; }
    const int tok0 = b * kKvBlock + 16 * warp;
    if (tok0 < ctx) {
      const uint8_t* raw = stages + stage * kRawStage;
      expand_page(raw + warp * kRawPage, wk, lane, 32, p.kv_fmt);
      expand_page(raw + (4 + warp) * kRawPage, wv, lane, 32, p.kv_fmt);
      __syncwarp();
      float s[2][4];
      s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < kD / 16; ++kk) {
        const int mi = lane >> 3;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sk + kv_tile_off<kD>(8 * (mi >> 1) + (lane & 7), 16 * kk + 8 * (mi & 1)), b0, b1, b2, b3);
        mma_bf16_16816(s[0], qf[kk], b0, b1);
        mma_bf16_16816(s[1], qf[kk], b2, b3);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = tok0 + 8 * j + 2 * (lane & 3) + (e & 1);
          s[j][e] = (col < ctx && (col >= kv_lo || col < sink)) ? s[j][e] * ks : -INFINITY;
        }
      float pv[2][4];
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
          const float p0 = exp2f(s[j][2 * r] - m_use), p1 = exp2f(s[j][2 * r + 1] - m_use);
          sum += p0 + p1;
          pv[j][2 * r] = p0 * vs;        // V scale folded into the probabilities that meet V
          pv[j][2 * r + 1] = p1 * vs;
        }
        l_run[r] = l_run[r] * alpha + sum;
#pragma unroll
        for (int j = 0; j < kD / 8; ++j) { o[j][2 * r] *= alpha; o[j][2 * r + 1] *= alpha; }
      }
      uint32_t a[4];
      a[0] = pack_bf16(pv[0][0], pv[0][1]);
      a[1] = pack_bf16(pv[0][2], pv[0][3]);
      a[2] = pack_bf16(pv[1][0], pv[1][1]);
      a[3] = pack_bf16(pv[1][2], pv[1][3]);
#pragma unroll
      for (int jd = 0; jd < kD / 16; ++jd) {
        const int mi = lane >> 3;
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sv + kv_tile_off<kD>(8 * (mi & 1) + (lane & 7), 16 * jd + 8 * (mi >> 1)), b0, b1, b2, b3);
        mma_bf16_16816(o[2 * jd], a, b0, b1);
        mma_bf16_16816(o[2 * jd + 1], a, b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
    if (++stage == kDecStages) { stage = 0; phase ^= 1; }
  }
  if (!ok && lane == 0) atomicOr(p.status, kStatusWaitTimeout);

  compute_bar_sync();
  float* sm_o = reinterpret_cast<float*>(stages);   // [4][16][128] fp32 = 32 KB <= 48 KB of ring
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = (lane >> 2) + 8 * r;
    if ((lane & 3) == 0) { sm_ml[(warp * 16 + row) * 2] = m_run[r]; sm_ml[(warp * 16 + row) * 2 + 1] = l; }
#pragma unroll
    for (int j = 0; j < kD / 8; ++j) {
      float* dst = sm_o + static_cast<size_t>(warp * 16 + row) * kD + 8 * j + 2 * (lane & 3);
      dst[0] = o[j][2 * r];
      dst[1] = o[j][2 * r + 1];
    }
  }
  compute_bar_sync();
  for (int idx = threadIdx.x; idx < G * kD; idx += 128) {
    const int row = idx / kD, d = idx % kD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, sm_ml[(w * 16 + row) * 2]);
    const float m_use = (mx == -INFINITY) ? 0.f : mx;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = exp2f(sm_ml[(w * 16 + row) * 2] - m_use);
      acc += wgt * sm_o[static_cast<size_t>(w * 16 + row) * kD + d];
      l += wgt * sm_ml[(w * 16 + row) * 2 + 1];
    }
    const int head = kvh * G + row;
    if (p.num_splits == 1) {
      p.out[static_cast<size_t>(seq) * p.o_stride + head * kD + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
    } else {
      const size_t slot = (static_cast<size_t>(seq) * p.hq + head) * p.num_splits + split;
      p.part_o[slot * kD + d] = acc;
      if (d == 0) { p.part_ml[slot * 2] = mx; p.part_ml[slot * 2 + 1] = l; }
    }
  }
}

__global__ void paged_decode_fp8_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out, int hq,
                                              int num_splits, int o_stride) {
  const int seq = blockIdx.x, head = blockIdx.y;
  if (ctx_len[seq] <= 0) return;
  const size_t base = (static_cast<size_t>(seq) * hq + head) * num_splits;
  float mx = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mx = fmaxf(mx, part_ml[(base + s) * 2]);
  const float m_use = (mx == -INFINITY) ? 0.f : mx;
  for (int d = threadIdx.x; d < kD; d += blockDim.x) {
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float w = exp2f(part_ml[(base + s) * 2] - m_use);
      acc += w * part_o[(base + s) * kD + d];
      l += w * part_ml[(base + s) * 2 + 1];
    }
    out[static_cast<size_t>(seq) * o_stride + head * kD + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
  }
}

// ------------------------------------------------------------------------------------------
// decode, e4m3 pages fed to the tensor cores as they are (query group of at most 8 heads per KV head)
//
// The expanding kernel above pays a shared-memory round trip per page (raw bytes -> bf16 tile -> ldmatrix), and that
// round trip, not HBM, bounds it.  This kernel never expands: K and V bytes go from the TMA ring into
// mma.sync.m16n8k32 e4m3 fragments directly.
//   exactness  an e4m3 operand has 4 significant bits, a bf16 query (and a probability rounded the way the bf16 kernels
//              round it) has 8.  A decode tile has at most 8 real rows out of the MMA's 16, so rows 0..7 carry the top 4
//              bits of each value ("hi") and rows 8..15 the next 4 bits times 16 ("lo"); row g and row g + 8 of an
//              accumulator land in the same thread, which adds them as hi + lo / 16.  Queries are divided by a power of
//              two per row first (largest magnitude below 256), probabilities are multiplied by 256.
//   QK^T       B fragments are plain ldmatrix reads of the raw K page (8 token rows x 16 bytes per matrix).
//   PV         the k index of the MMA runs over tokens, which are 128 bytes apart in a V page: each thread loads 16
//              bytes of 4 token rows per page and transposes 4x4 byte blocks with byte permutes.  Which token sits at
//              which k, and which head dimension at which n, is then a fixed permutation that the P fragments and the
//              final store undo; no shared-memory staging.
//   scales     the K scale multiplies the scores of its page.  The V scale enters as log2(v_scale) added to the score
//              that feeds the probabilities (so the running maximum tracks probability x V scale and the e4m3
//              probabilities use their range whatever the page), and the row sum divides it out again per page.
// One stage holds 8 pages (128 keys): each of the four consumer warps owns two pages (one k = 32 step) of it.
// ------------------------------------------------------------------------------------------
constexpr int kMmaPages = 8;
constexpr int kMmaStage = kMmaPages * 2 * kRawPage;   // 32 KB
constexpr int kMmaStages = 3;
constexpr int kMmaKeys = kMmaPages * kPageTokens;     // 128
constexpr int kMmaSmem = kMmaStages * kMmaStage + 1024 + 1024;

OGB_DEVICE void mma_e4m3_16832(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// four floats -> four e4m3 bytes (v0 in the lowest byte), round to nearest, saturating
OGB_DEVICE uint32_t pack_e4m3x4(float v0, float v1, float v2, float v3) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v0, v1), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v2, v3), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
// x = hi + lo / 16 with hi holding the top 4 significant bits of x (exact in e4m3 for 2^-6 <= |x| <= 448)
OGB_DEVICE void split_hi_lo(float x, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xFFF00000u);
  lo = (x - hi) * 16.f;
}
OGB_DEVICE void pack_hi_lo(const float (&v)[4], uint32_t& hi, uint32_t& lo) {
  float h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) split_hi_lo(v[i], h[i], l[i]);
  hi = pack_e4m3x4(h[0], h[1], h[2], h[3]);
  lo = pack_e4m3x4(l[0], l[1], l[2], l[3]);
}
// rows r0..r3 each hold 4 bytes; out[j] byte i = r_i byte j
OGB_DEVICE void transpose_4x4_bytes(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t (&out)[4]) {
  const uint32_t a_lo = __byte_perm(r0, r1, 0x5140), a_hi = __byte_perm(r0, r1, 0x7362);
  const uint32_t b_lo = __byte_perm(r2, r3, 0x5140), b_hi = __byte_perm(r2, r3, 0x7362);
  out[0] = __byte_perm(a_lo, b_lo, 0x5410);
  out[1] = __byte_perm(a_lo, b_lo, 0x7632);
  out[2] = __byte_perm(a_hi, b_hi, 0x5410);
  out[3] = __byte_perm(a_hi, b_hi, 0x7632);
}

OGB_DEVICE void mbar_expect_tx_only(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Producer warp of the kernel below.  Lane i < 8 owns page i of each stage: it reads the page id, issues the page's two
// TMA boxes, then fetches the page's two scales and leaves them beside the stage, so the consumers never touch global
// memory inside their loop.  The byte count is announced before the loads, the barrier's one arrival comes after the
// scales are written.  Pages past the end of the context are not loaded, except that an odd tail is padded to a pair
// (a consumer warp reads both pages of its pair; masked probabilities must meet finite bytes).
OGB_DEVICE bool fp8_produce_wide(const CUtensorMap* kv_map, const AttnParams& p, uint8_t* stages, float* stage_scales,
                                 uint64_t* full_bar, uint64_t* empty_bar, int seq, int kvh, int ctx, int b_begin, int b_end,
                                 int kv_lo, int lane) {
  const int n_pages = (ctx + kPageTokens - 1) / kPageTokens;
  const int* table = p.page_table + static_cast<size_t>(seq) * p.max_pages;
  int stage = 0;
  uint32_t phase = 0;
  for (int b = b_begin; b < b_end; ++b) {
    const int n_load = min(kMmaPages, ((n_pages - b * kMmaPages + 1) >> 1) << 1);
    int64_t page = 0;
    if (lane < n_load) {
      const int pi = skip_gap_page(min(min(b * kMmaPages + lane, n_pages - 1), p.max_pages - 1), p.window, p.sink, kv_lo);
      page = table[pi];
      if (page < 0 || page >= p.num_pages) { atomicOr(p.status, kStatusIndexOutOfRange); page = 0; }
    }
    if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1))) return false;
    uint8_t* s = stages + stage * kMmaStage;
    if (lane == 0) mbar_expect_tx_only(&full_bar[stage], n_load * 2 * kRawPage);
    __syncwarp();
    if (lane < n_load) {
      const int row_k = static_cast<int>(((page * p.hkv + kvh) * 2) * kPageTokens);
      tma_load_2d(s + lane * kRawPage, kv_map, &full_bar[stage], 0, row_k);
      tma_load_2d(s + (kMmaPages + lane) * kRawPage, kv_map, &full_bar[stage], 0, row_k + kPageTokens);
      const float2 sc = *reinterpret_cast<const float2*>(p.kv_scales + (page * p.hkv + kvh) * 2);
      *reinterpret_cast<float2*>(stage_scales + (stage * kMmaPages + lane) * 2) = sc;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&full_bar[stage]);
    if (++stage == kMmaStages) { stage = 0; phase ^= 1; }
  }
  return true;
}

// 168 registers: two CTAs of five warps put three warps on one scheduler, whose 16384 registers must hold them.
__global__ void __maxnreg__(168) paged_decode_e4m3_mma_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                              const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kMmaStages * kMmaStage);
  uint64_t* empty_bar = full_bar + kMmaStages;
  float* sm_ml = reinterpret_cast<float*>(empty_bar + kMmaStages);   // [4 warps][8 rows][2]
  float* stage_scales = sm_ml + 4 * 8 * 2;                           // [stages][8 pages][K, V]

  const int seq = blockIdx.x / p.num_splits, split = blockIdx.x % p.num_splits, kvh = blockIdx.y;
  const int G = p.group;
  const int ctx = p.ctx_len[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int b_begin = 0, b_end = 0;
  const int kv_lo = (p.window > 0) ? max(0, ctx - p.window) : 0;
  const int sink = (p.window > 0) ? p.sink : 0;
  if (ctx > 0) {
    const int first = (sink > 0) ? 0 : kv_lo / kMmaKeys;
    const int last = (ctx + kMmaKeys - 1) / kMmaKeys;
    const int per = (last - first + p.num_splits - 1) / p.num_splits;
    b_begin = first + split * per;
    b_end = min(b_begin + per, last);
  }
  if (b_begin >= b_end) {
    if (p.num_splits > 1 && ctx > 0) {
      for (int idx = threadIdx.x; idx < G * kD; idx += blockDim.x) {
        const int r = idx / kD, d = idx % kD;
        const size_t slot = (static_cast<size_t>(seq) * p.hq + kvh * G + r) * p.num_splits + split;
        p.part_o[slot * kD + d] = 0.f;
        if (d == 0) { p.part_ml[slot * 2] = -INFINITY; p.part_ml[slot * 2 + 1] = 0.f; }
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < kMmaStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 4); }
    mbar_fence_init();
    tma_prefetch_desc(&kv_map);
  }
  __syncthreads();
  if (warp == 4) {
    if (!fp8_produce_wide(&kv_map, p, stages, stage_scales, full_bar, empty_bar, seq, kvh, ctx, b_begin, b_end, kv_lo, lane) && lane == 0)
      atomicOr(p.status, kStatusWaitTimeout);
    return;
  }
  const int g = lane >> 2, q = lane & 3;

  // query fragments: row g = hi part, row g + 8 = lo part of head kvh * G + g; k runs over the head dimension
  uint32_t qf[4][4];
  float q_scale;   // what one unit of the e4m3 query stands for, times the softmax scale
  {
    float qv[4][8];
    float amax = 0.f;
    const __nv_bfloat16* qsrc = p.q + static_cast<size_t>(seq) * p.q_stride + (kvh * G + g) * kD;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint2 raw = make_uint2(0, 0);
        if (g < G) raw = *reinterpret_cast<const uint2*>(qsrc + 32 * ks + 16 * h + 4 * q);
        const __nv_bfloat162 v01 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 v23 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        qv[ks][4 * h + 0] = __low2float(v01); qv[ks][4 * h + 1] = __high2float(v01);
        qv[ks][4 * h + 2] = __low2float(v23); qv[ks][4 * h + 3] = __high2float(v23);
#pragma unroll
        for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(qv[ks][4 * h + i]));
      }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int e = 0;
    if (amax > 0.f && amax < 3.0e38f) (void)frexpf(amax, &e);        // amax < 2^e
    e = max(min(e - 8, 100), -100);
    const float unit = ldexpf(1.f, e), inv_unit = ldexpf(1.f, -e);    // |q| / unit < 256
    q_scale = unit * p.scale_log2e;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float v[4] = {qv[ks][4 * h] * inv_unit, qv[ks][4 * h + 1] * inv_unit, qv[ks][4 * h + 2] * inv_unit,
                            qv[ks][4 * h + 3] * inv_unit};
        pack_hi_lo(v, qf[ks][2 * h], qf[ks][2 * h + 1]);
      }
  }

  // o[w * 4 + j]: head dimensions 16 * (2q) + 4w + j (c0 / c2) and 16 * (2q + 1) + 4w + j (c1 / c3); c2, c3 are the lo rows
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run = -INFINITY, l_run = 0.f;

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int b = b_begin; b < b_end; ++b) {
    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase))) { ok = false; break; }
    const int tok0 = b * kMmaKeys + 32 * warp;
    if (tok0 < ctx) {
      float kf[2], lv[2], inv_v[2];
      {
        const float4 sc4 = *reinterpret_cast<const float4*>(stage_scales + (stage * kMmaPages + 2 * warp) * 2);
        const float vs0 = fmaxf(sc4.y, 1e-30f), vs1 = fmaxf(sc4.w, 1e-30f);
        kf[0] = sc4.x * q_scale; kf[1] = sc4.z * q_scale;
        lv[0] = __log2f(vs0); lv[1] = __log2f(vs1);
        inv_v[0] = __fdividef(1.f, vs0); inv_v[1] = __fdividef(1.f, vs1);
      }
      const uint32_t k_u = smem_u32(stages + stage * kMmaStage + (2 * warp) * kRawPage);
      const uint8_t* v_p = stages + stage * kMmaStage + (kMmaPages + 2 * warp) * kRawPage;
      // scores: 4 groups of 8 tokens
      float sc[4][2];
#pragma unroll
      for (int ng = 0; ng < 4; ++ng) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        const int r = 8 * (ng & 1) + (lane & 7);
        const uint32_t row_u = k_u + (ng >> 1) * kRawPage + r * 128;
#pragma unroll
        for (int kp = 0; kp < 2; ++kp) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(row_u + ((((4 * kp + (lane >> 3)) ^ (r & 7))) << 4), b0, b1, b2, b3);
          mma_e4m3_16832(c, qf[2 * kp], b0, b1);
          mma_e4m3_16832(c, qf[2 * kp + 1], b2, b3);
        }
        const int pg = ng >> 1;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = tok0 + 8 * ng + 2 * q + e;
          const float s = (c[e] + c[2 + e] * 0.0625f) * kf[pg] + lv[pg];
          sc[ng][e] = (col < ctx && (col >= kv_lo || col < sink)) ? s : -INFINITY;
        }
      }
      float mx = fmaxf(fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1])),
                       fmaxf(fmaxf(sc[2][0], sc[2][1]), fmaxf(sc[3][0], sc[3][1])));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);
      m_run = m_new;
      float pe[4][2];
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int ng = 0; ng < 4; ++ng)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          pe[ng][e] = exp2f(sc[ng][e] - m_use);
          sum[ng >> 1] += pe[ng][e];
        }
      l_run = l_run * alpha + sum[0] * inv_v[0] + sum[1] * inv_v[1];
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int j = 0; j < 16; ++j) { o[j][0] *= alpha; o[j][1] *= alpha; o[j][2] *= alpha; o[j][3] *= alpha; }
      }
      // probabilities: k = 4q + i <-> token {2q, 2q + 1, 8 + 2q, 9 + 2q}[i] of the first page, k = 16 + ... of the second
      uint32_t a[4];
      {
        const float v0[4] = {pe[0][0] * 256.f, pe[0][1] * 256.f, pe[1][0] * 256.f, pe[1][1] * 256.f};
        const float v1[4] = {pe[2][0] * 256.f, pe[2][1] * 256.f, pe[3][0] * 256.f, pe[3][1] * 256.f};
        pack_hi_lo(v0, a[0], a[1]);
        pack_hi_lo(v1, a[2], a[3]);
      }
      uint4 va[4], vb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = 8 * (i >> 1) + 2 * q + (i & 1);
        const int off = t * 128 + ((g ^ (t & 7)) << 4);
        va[i] = *reinterpret_cast<const uint4*>(v_p + off);
        vb[i] = *reinterpret_cast<const uint4*>(v_p + kRawPage + off);
      }
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t ta[4], tb[4];
        const uint32_t* a0 = reinterpret_cast<const uint32_t*>(&va[0]);
        const uint32_t* b0 = reinterpret_cast<const uint32_t*>(&vb[0]);
        transpose_4x4_bytes(a0[w], a0[4 + w], a0[8 + w], a0[12 + w], ta);
        transpose_4x4_bytes(b0[w], b0[4 + w], b0[8 + w], b0[12 + w], tb);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_e4m3_16832(o[4 * w + j], a, ta[j], tb[j]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
    if (++stage == kMmaStages) { stage = 0; phase ^= 1; }
  }
  if (!ok && lane == 0) atomicOr(p.status, kStatusWaitTimeout);

  compute_bar_sync();
  float* sm_o = reinterpret_cast<float*>(stages);   // [4 warps][8 rows][128] fp32 = 16 KB of the ring
  {
    float l = l_run;
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (q == 0) { sm_ml[(warp * 8 + g) * 2] = m_run; sm_ml[(warp * 8 + g) * 2 + 1] = l; }
    float* dst = sm_o + static_cast<size_t>(warp * 8 + g) * kD;
#pragma unroll
    for (int w = 0; w < 4; ++w)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float* c = o[4 * w + j];
        dst[16 * (2 * q) + 4 * w + j] = (c[0] + c[2] * 0.0625f) * (1.f / 256.f);
        dst[16 * (2 * q + 1) + 4 * w + j] = (c[1] + c[3] * 0.0625f) * (1.f / 256.f);
      }
  }
  compute_bar_sync();
  for (int idx = threadIdx.x; idx < G * kD; idx += 128) {
    const int row = idx / kD, d = idx % kD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, sm_ml[(w * 8 + row) * 2]);
    const float m_use = (mx == -INFINITY) ? 0.f : mx;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = exp2f(sm_ml[(w * 8 + row) * 2] - m_use);
      acc += wgt * sm_o[static_cast<size_t>(w * 8 + row) * kD + d];
      l += wgt * sm_ml[(w * 8 + row) * 2 + 1];
    }
    const int head = kvh * G + row;
    if (p.num_splits == 1) {
      p.out[static_cast<size_t>(seq) * p.o_stride + head * kD + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
    } else {
      const size_t slot = (static_cast<size_t>(seq) * p.hq + head) * p.num_splits + split;
      p.part_o[slot * kD + d] = acc;
      if (d == 0) { p.part_ml[slot * 2] = mx; p.part_ml[slot * 2 + 1] = l; }
    }
  }
}

// ------------------------------------------------------------------------------------------
// prefill (chunked, causal): 64 query rows x one head per CTA; the four consumer warps expand each
// 64-key block together into one shared bf16 tile
// ------------------------------------------------------------------------------------------
constexpr int kPreStages = 2;
constexpr int kPreTile = kKvBlock * kD * 2;   // 16 KB bf16 K tile (and as much for V)
constexpr int kPreSmem = kPreStages * kRawStage + 2 * kPreTile + 64 * kD * 2 + 1024 + 1024;

__global__ void __launch_bounds__(kAttnThreads) paged_prefill_fp8_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                          const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* tile_k = smem + kPreStages * kRawStage;
  uint8_t* tile_v = tile_k + kPreTile;
  uint8_t* sq = tile_v + kPreTile;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sq + 64 * kD * 2);
  uint64_t* empty_bar = full_bar + kPreStages;
  float* sc_sh = reinterpret_cast<float*>(empty_bar + kPreStages);   // [4 pages][2]

  const int tile = blockIdx.x;
  if (tile >= p.num_tiles) return;
  const int head = blockIdx.y, kvh = head / p.group;
  const int seq = p.tile_seq[tile], q0 = p.tile_q0[tile];
  const int q_begin = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - q_begin;
  const int ctx = p.ctx_len[seq];
  const int rows = min(64, q_len - q0);
  const int pos0 = ctx - q_len + q0;
  if (rows <= 0 || ctx <= 0) return;
  const int kv_end = min(ctx, pos0 + rows);
  const int kv_lo = (p.window > 0) ? max(0, pos0 - p.window + 1) : 0;   // first key any row of the tile sees in its window
  const int b_end = (kv_end + kKvBlock - 1) / kKvBlock;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kPreStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 4); }
    mbar_fence_init();
    tma_prefetch_desc(&kv_map);
  }
  __syncthreads();
  if (warp == 4) {
    if (lane == 0 && !fp8_produce(&kv_map, p, stages, full_bar, empty_bar, kPreStages, seq, kvh, ctx, 0, b_end, kv_lo))
      atomicOr(p.status, kStatusWaitTimeout);
    return;
  }
  {
    const __nv_bfloat16* qsrc = p.q + static_cast<size_t>(q_begin + q0) * p.q_stride + head * kD;
    for (int idx = threadIdx.x; idx < 64 * (kD / 8); idx += 128) {
      const int row = idx / (kD / 8), ch = idx % (kD / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < rows) v = *reinterpret_cast<const uint4*>(qsrc + static_cast<size_t>(row) * p.q_stride + ch * 8);
      *reinterpret_cast<uint4*>(sq + q_tile_off<64>(row, ch * 8)) = v;
    }
  }
  compute_bar_sync();
  uint32_t qf[kD / 16][4];
  {
    const uint32_t sq_u = smem_u32(sq);
#pragma unroll
    for (int kk = 0; kk < kD / 16; ++kk)
      ldsm_x4(sq_u + q_tile_off<64>(16 * warp + (lane & 15), 16 * kk + 8 * (lane >> 4)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
  float o[kD / 8][4];
#pragma unroll
  for (int j = 0; j < kD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_a = 16 * warp + (lane >> 2);
  const int qpos_a = pos0 + row_a, qpos_b = pos0 + row_a + 8;
  const uint32_t sk = smem_u32(tile_k), sv = smem_u32(tile_v);

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int b = 0; b < b_end; ++b) {
    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase))) { ok = false; break; }
    const uint8_t* raw = stages + stage * kRawStage;
    // warp w expands page w of the block (K and V) into the shared bf16 tiles
    expand_page(raw + warp * kRawPage, tile_k + warp * kWorkPage, lane, 32, p.kv_fmt);
    expand_page(raw + (4 + warp) * kRawPage, tile_v + warp * kWorkPage, lane, 32, p.kv_fmt);
    if (lane < 2) {
      const int64_t page = page_of(p, seq, ctx, b * 4 + warp, kv_lo);
      sc_sh[warp * 2 + lane] = p.kv_scales[(page * p.hkv + kvh) * 2 + lane];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);   // the raw bytes are no longer needed
    compute_bar_sync();
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < kD / 16; ++kk) {
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        const int mi = lane >> 3;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sk + kv_tile_off<kD>(16 * jp + 8 * (mi >> 1) + (lane & 7), 16 * kk + 8 * (mi & 1)), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * jp], qf[kk], b0, b1);
        mma_bf16_16816(s[2 * jp + 1], qf[kk], b2, b3);
      }
    }
    const int kv_base = b * kKvBlock;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float ks = sc_sh[(j >> 1) * 2] * p.scale_log2e;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = kv_base + 8 * j + 2 * (lane & 3) + (e & 1);
        const int qpos = (e < 2) ? qpos_a : qpos_b;
        s[j][e] = key_visible(col, qpos, ctx, p.window, p.sink) ? s[j][e] * ks : -INFINITY;
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
        const float p0 = exp2f(s[j][2 * r] - m_use), p1 = exp2f(s[j][2 * r + 1] - m_use);
        sum += p0 + p1;
        const float vs = sc_sh[(j >> 1) * 2 + 1];
        s[j][2 * r] = p0 * vs;
        s[j][2 * r + 1] = p1 * vs;
      }
      l_run[r] = l_run[r] * alpha + sum;
#pragma unroll
      for (int j = 0; j < kD / 8; ++j) { o[j][2 * r] *= alpha; o[j][2 * r + 1] *= alpha; }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jd = 0; jd < kD / 16; ++jd) {
        const int mi = lane >> 3;
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sv + kv_tile_off<kD>(16 * kk + 8 * (mi & 1) + (lane & 7), 16 * jd + 8 * (mi >> 1)), b0, b1, b2, b3);
        mma_bf16_16816(o[2 * jd], a, b0, b1);
        mma_bf16_16816(o[2 * jd + 1], a, b2, b3);
      }
    }
    compute_bar_sync();   // everyone is done with the bf16 tiles before the next block is expanded
    if (++stage == kPreStages) { stage = 0; phase ^= 1; }
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
      __nv_bfloat16* dst = p.out + static_cast<size_t>(q_begin + q0 + row) * p.o_stride + head * kD + 2 * (lane & 3);
#pragma unroll
      for (int j = 0; j < kD / 8; ++j)
        *reinterpret_cast<uint32_t*>(dst + 8 * j) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
  }
}

static int get_fp8_tmap(const void* pool, int64_t num_pages, int hkv, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<const void*, std::pair<uint64_t, CUtensorMap>> cache;
  const uint64_t rows = static_cast<uint64_t>(num_pages) * hkv * 2 * kPageTokens;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(pool);
  if (it != cache.end() && it->second.first == rows) { *out = it->second.second; return 0; }
  CUtensorMap m;
  int rc = make_tmap_u8_2d(&m, pool, rows, kD, kD, kPageTokens, kD);
  if (rc != 0) return rc;
  cache[pool] = {rows, m};
  *out = m;
  return 0;
}

}  // namespace ogb

using namespace ogb;

static void fill_params(AttnParams& p, const void* q, void* out, const float* scales, const int* page_table, const int* ctx_len,
                        int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int q_stride, int o_stride, float scale,
                        int* status) {
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.page_table = page_table; p.ctx_len = ctx_len; p.num_seqs = num_seqs; p.max_pages = max_pages; p.num_pages = num_pages;
  p.hq = hq; p.hkv = hkv; p.group = hq / hkv; p.q_stride = q_stride; p.o_stride = o_stride;
  p.scale_log2e = scale * 1.4426950408889634f; p.status = status; p.kv_scales = scales; p.num_splits = 1;
}

// How decode reads e4m3 pages when a KV head serves at most 8 query heads: 2 = tcgen05 kernel (raw bytes as
// kind::f8f6f4 operands), 1 = mma.sync e4m3 kernel, 0 = expand pages to bf16 first.  -1: read OGB_E4M3_MMA once (default 2).
static int g_e4m3_mma = -1;
static int e4m3_mma_mode() {
  if (g_e4m3_mma < 0) {
    const char* e = getenv("OGB_E4M3_MMA");
    g_e4m3_mma = (e != nullptr && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 2;
  }
  return g_e4m3_mma;
}
extern "C" int ogb_attn_set_e4m3_mma(int mode) {
  const int old = e4m3_mma_mode();
  g_e4m3_mma = mode < 0 ? 0 : (mode > 2 ? 2 : mode);
  return old;
}

static int launch_decode_q(const void* q, void* out, const void* pool, const float* scales, int kv_fmt, const int* page_table,
                           const int* ctx_len, int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d,
                           int q_stride, int o_stride, float scale, int num_splits, float* part_o, float* part_ml,
                           int window, int sink, int* status, void* stream) {
  if (num_seqs <= 0) return 0;
  if (kv_fmt < 0 || kv_fmt > 2) return -3;
  if (d != kD || hkv <= 0 || hq % hkv != 0 || hq / hkv > 16 || (q_stride % 8) != 0 || scales == nullptr) return -3;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return -4;
  CUtensorMap map;
  int rc = get_fp8_tmap(pool, num_pages, hkv, &map);
  if (rc != 0) return rc;
  AttnParams p{};
  fill_params(p, q, out, scales, page_table, ctx_len, num_seqs, max_pages, num_pages, hq, hkv, q_stride, o_stride, scale, status);
  p.num_splits = num_splits; p.part_o = part_o; p.part_ml = part_ml; p.kv_fmt = kv_fmt;
  p.window = window; p.sink = window > 0 ? sink : 0;
  static bool attr_set = false;
  if (!attr_set) {
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_fp8_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    attr_set = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int mode = (kv_fmt == 0 && p.group <= 8) ? e4m3_mma_mode() : 0;
  if (mode == 2) {
    rc = launch_decode_e4m3_tc(p, pool, stream);
    if (rc != 0) return rc;
  } else if (mode == 1) {
    static bool mma_attr_set = false;
    if (!mma_attr_set) {
      OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_e4m3_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem));
      OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_e4m3_mma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
      mma_attr_set = true;
    }
    paged_decode_e4m3_mma_kernel<<<dim3(num_seqs * num_splits, hkv), kAttnThreads, kMmaSmem, st>>>(map, p);
  } else {
    paged_decode_fp8_kernel<<<dim3(num_seqs * num_splits, hkv), kAttnThreads, kDecSmem, st>>>(map, p);
  }
  rc = static_cast<int>(cudaGetLastError());
  if (rc == 0 && num_splits > 1) {
    paged_decode_fp8_merge_kernel<<<dim3(num_seqs, hq), kD, 0, st>>>(part_o, part_ml, ctx_len, p.out, hq, num_splits, o_stride);
    rc = static_cast<int>(cudaGetLastError());
  }
  return rc;
}

static int launch_prefill_q(const void* q, void* out, const void* pool, const float* scales, int kv_fmt, const int* page_table,
                            const int* ctx_len, const int* cu_q, const int* tile_seq, const int* tile_q0, int num_tiles,
                            int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride,
                            int o_stride, float scale, int window, int sink, int* status, void* stream) {
  if (num_tiles <= 0) return 0;
  if (kv_fmt < 0 || kv_fmt > 2) return -3;
  if (d != kD || hkv <= 0 || hq % hkv != 0 || (q_stride % 8) != 0 || (o_stride % 2) != 0 || scales == nullptr) return -3;
  CUtensorMap map;
  int rc = get_fp8_tmap(pool, num_pages, hkv, &map);
  if (rc != 0) return rc;
  AttnParams p{};
  fill_params(p, q, out, scales, page_table, ctx_len, num_seqs, max_pages, num_pages, hq, hkv, q_stride, o_stride, scale, status);
  p.cu_q = cu_q; p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.num_tiles = num_tiles; p.kv_fmt = kv_fmt;
  p.window = window; p.sink = window > 0 ? sink : 0;
  static bool attr_set = false;
  if (!attr_set) {
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_prefill_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPreSmem));
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_prefill_fp8_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    attr_set = true;
  }
  paged_prefill_fp8_kernel<<<dim3(num_tiles, hq), kAttnThreads, kPreSmem, static_cast<cudaStream_t>(stream)>>>(map, p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_paged_decode_fp8(const void* q, void* out, const void* pool, const float* scales, const int* page_table,
                                    const int* ctx_len, int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d,
                                    int q_stride, int o_stride, float scale, int num_splits, float* part_o, float* part_ml,
                                    int* status, void* stream) {
  return launch_decode_q(q, out, pool, scales, 0, page_table, ctx_len, num_seqs, max_pages, num_pages, hq, hkv, d, q_stride, o_stride,
                         scale, num_splits, part_o, part_ml, 0, 0, status, stream);
}
extern "C" int ogb_paged_prefill_fp8(const void* q, void* out, const void* pool, const float* scales, const int* page_table,
                                     const int* ctx_len, const int* cu_q, const int* tile_seq, const int* tile_q0, int num_tiles,
                                     int num_seqs, int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride,
                                     int o_stride, float scale, int* status, void* stream) {
  return launch_prefill_q(q, out, pool, scales, 0, page_table, ctx_len, cu_q, tile_seq, tile_q0, num_tiles, num_seqs, max_pages,
                          num_pages, hq, hkv, d, q_stride, o_stride, scale, 0, 0, status, stream);
}
// One-byte pages in any format: kv_format 0 = e4m3, 1 = int8 (symmetric), 2 = e5m2; same per-(page, head, K|V) scale layout.
extern "C" int ogb_paged_decode_q8(const void* q, void* out, const void* pool, const float* scales, int kv_format,
                                   const int* page_table, const int* ctx_len, int num_seqs, int max_pages, int64_t num_pages,
                                   int hq, int hkv, int d, int q_stride, int o_stride, float scale, int num_splits,
                                   float* part_o, float* part_ml, int window, int sink, int* status, void* stream) {
  return launch_decode_q(q, out, pool, scales, kv_format, page_table, ctx_len, num_seqs, max_pages, num_pages, hq, hkv, d, q_stride,
                         o_stride, scale, num_splits, part_o, part_ml, window, sink, status, stream);
}
extern "C" int ogb_paged_prefill_q8(const void* q, void* out, const void* pool, const float* scales, int kv_format,
                                    const int* page_table, const int* ctx_len, const int* cu_q, const int* tile_seq,
                                    const int* tile_q0, int num_tiles, int num_seqs, int max_pages, int64_t num_pages, int hq,
                                    int hkv, int d, int q_stride, int o_stride, float scale, int window, int sink, int* status,
                                    void* stream) {
  return launch_prefill_q(q, out, pool, scales, kv_format, page_table, ctx_len, cu_q, tile_seq, tile_q0, num_tiles, num_seqs,
                          max_pages, num_pages, hq, hkv, d, q_stride, o_stride, scale, window, sink, status, stream);
}
