// Split-KV GQA decode over e4m3 KV pages on the fifth-generation tensor cores (tcgen05, kind::f8f6f4).
//
// The reference never attends over quantised KV (its codec lives in host page storage,
// crates/onnx-genai-kv/src/fp8.rs:5-198; group_query_attention.rs:1140-1200 rejects quantised K/V).  Here the e4m3
// bytes are the tensor-core operands: no conversion instruction touches K or V.  (The legacy mma.sync path has no
// native e4m3 on this part: the compiler expands each such MMA into unpack arithmetic plus f16 MMAs, and that
// arithmetic, not HBM, bounded the register-level kernels in attention_fp8.cu.)
//
// One CTA = one (sequence, KV split, KV head); a stage = 8 pages = 128 keys, K and V, brought by TMA exactly as they
// lie in the pool (16 rows of 128 bytes per page side, 128-byte swizzle).  The problem is run transposed so that the
// 128-row MMA dimension is filled by keys (then by head dimensions), not by the handful of query heads:
//   S^T[128 keys x 16]  = K[128 keys x 128 d] . Qhl^T         A = K tile (K-major), B = Qhl (16 rows, K-major)
//   O^T[128 d    x 16] += V^T[128 d x 128 keys] . Phl^T        A = V tile read MN-major, B = Phl (16 rows, K-major)
// The 16 columns are the query heads of the KV head twice: an e4m3 operand has 4 significant bits, a bf16 query or a
// probability needs 8, so columns 0..7 carry the top 4 bits ("hi") and columns 8..15 the next 4 bits times 16 ("lo");
// hi + lo / 16 is formed where accumulators are read.  Needs at most 8 query heads per KV head and head_dim 128.
// Roles: warp 0 K producer, warp 6 V producer (also stages the page scales), warp 1 MMA issuer and TMEM owner, warps 2-5
// softmax: thread
// t owns key t of the stage (TMEM lane t of S^T) and later head dimension t (lane t of O^T).
// Softmax: the running reference m only moves when a block maximum exceeds it by more than 2^7 (probabilities then stay
// below e4m3's 448), so the O^T rescale through TMEM is rare.  The V scale of a page enters as log2 added to the score
// and is divided out of the row sum, as in the register-level kernel.  Every wait is bounded and aborts the CTA with a
// status bit; TMEM is freed on every path.
#include <cuda_fp8.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "attention_common.cuh"
#include "ogb_kernels.h"

namespace ogb {

constexpr int kTcD = 128;
constexpr int kTcPages = 8;
constexpr int kTcKeys = kTcPages * kPageTokens;          // 128
constexpr int kTcPageBytes = kPageTokens * kTcD;          // 2 KB per page side
constexpr int kTcSideBytes = kTcPages * kTcPageBytes;     // 16 KB: K tile, then V tile
constexpr int kTcStageBytes = 2 * kTcSideBytes;           // 32 KB
constexpr int kTcStages = 3;
constexpr int kTcThreads = 224;
constexpr int kTcSmallTile = 16 * 128;                    // Qhl / Phl: 16 rows x 128 bytes
constexpr int kTcTmemCols = 64;                           // S0 | S1 | O, 16 columns each
constexpr float kTcLag = 7.f;
constexpr int kTcSmem = kTcStages * kTcStageBytes + 3 * kTcSmallTile + 1024 /*barriers, scales, exchange*/ + 1024 /*align*/;

struct TcShared {                                         // lives after the tiles
  uint64_t k_full[kTcStages], k_empty[kTcStages], v_full[kTcStages], v_empty[kTcStages];
  uint64_t s_full[2], s_free[2], p_full[2], p_free[2];
  uint64_t o_done;
  uint32_t tmem_base;
  int abort_flag;
  float scales[kTcStages][kTcPages][2];
  float wmax[2][4][8];
  float q_unit[8];
  float lsum[4][8];
};
static_assert(sizeof(TcShared) <= 1024, "shared bookkeeping");

__host__ __device__ constexpr uint32_t make_idesc_e4m3(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4)                                   // D format: f32
         | (0u << 7) | (0u << 10)                    // A, B format: e4m3
         | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16)
         | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

OGB_DEVICE void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
OGB_DEVICE void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
OGB_DEVICE void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
OGB_DEVICE void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

OGB_DEVICE uint64_t tc_mn_major_desc(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((1024 >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
OGB_DEVICE void tc_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait that also gives up once another role of the CTA has raised the abort flag.
OGB_DEVICE bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_test(bar, parity)) {
    if (((++spins) & 0x3ff) == 0) {
      if (*abort_flag != 0 || global_timer_ns() - t0 > kWaitLimitNs) return false;
    }
  }
  return true;
}
// floats <-> integers with the same order (so that redux.sync can take a maximum of floats)
OGB_DEVICE int ordered_int(float v) {
  const int b = __float_as_int(v);
  return b ^ ((b >> 31) & 0x7fffffff);
}
OGB_DEVICE float ordered_float(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }
OGB_DEVICE float warp_max_redux(float v) {
  int r;
  asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(ordered_int(v)));
  return ordered_float(r);
}
// x = hi + lo / 16, hi = the top 4 significant bits of x
OGB_DEVICE void tc_split(float x, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xFFF00000u);
  lo = (x - hi) * 16.f;
}
OGB_DEVICE uint32_t tc_pack_e4m3x2(float v0, float v1) {   // v0 in the low byte
  return __nv_cvt_float2_to_fp8x2(make_float2(v0, v1), __NV_SATFINITE, __NV_E4M3);
}

// Optional stamps: with p.dbg set, CTA (dbg_tile, kv head 0) accumulates nanoseconds per phase.  Slots: 0 start, 1 end,
// 2 blocks; softmax (key 0): 3 wait S, 4 wait V + scales, 5 TMEM load, 6 maxima + exchange, 7 rescales, 8 wait P buffer,
// 9 exponentials + P store + fence; MMA thread: 10 wait K, 11 wait S buffer, 12 wait V + P; K producer 13 wait empty.
struct TcStamp {
  unsigned long long* d;
  uint64_t t;
  OGB_DEVICE void begin() { if (d) t = global_timer_ns(); }
  OGB_DEVICE void lap(int slot) { if (d) { const uint64_t n = global_timer_ns(); d[slot] += n - t; t = n; } }
};

__global__ void __launch_bounds__(kTcThreads) paged_decode_e4m3_tc_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                           const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* q_tile = smem + kTcStages * kTcStageBytes;
  uint8_t* p_tile = q_tile + kTcSmallTile;                 // two buffers
  TcShared& sh = *reinterpret_cast<TcShared*>(p_tile + 2 * kTcSmallTile);

  const int seq = blockIdx.x / p.num_splits, split = blockIdx.x % p.num_splits, kvh = blockIdx.y;
  const int G = p.group;
  const int ctx = p.ctx_len[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int b_begin = 0, b_end = 0;
  const int kv_lo = (p.window > 0) ? max(0, ctx - p.window) : 0;     // first key inside the window
  const int sink = (p.window > 0) ? p.sink : 0;
  if (ctx > 0) {
    const int first = (sink > 0) ? 0 : kv_lo / kTcKeys;             // with sinks the walk starts at key 0 (gap blocks are masked)
    const int last = (ctx + kTcKeys - 1) / kTcKeys;
    const int per = (last - first + p.num_splits - 1) / p.num_splits;
    b_begin = first + split * per;
    b_end = min(b_begin + per, last);
  }
  if (b_begin >= b_end) {
    if (p.num_splits > 1 && ctx > 0) {
      for (int idx = threadIdx.x; idx < G * kTcD; idx += blockDim.x) {
        const int r = idx / kTcD, d = idx % kTcD;
        const size_t slot = (static_cast<size_t>(seq) * p.hq + kvh * G + r) * p.num_splits + split;
        p.part_o[slot * kTcD + d] = 0.f;
        if (d == 0) { p.part_ml[slot * 2] = -INFINITY; p.part_ml[slot * 2 + 1] = 0.f; }
      }
    }
    return;
  }
  const int n_blocks = b_end - b_begin;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kTcStages; ++i) {
      mbar_init(&sh.k_full[i], 1); mbar_init(&sh.k_empty[i], 1);
      mbar_init(&sh.v_full[i], 1); mbar_init(&sh.v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.s_full[i], 1); mbar_init(&sh.s_free[i], 4);
      mbar_init(&sh.p_full[i], 4); mbar_init(&sh.p_free[i], 1);
    }
    mbar_init(&sh.o_done, 1);
    sh.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&kv_map);
  }
  if (warp == 1) { tmem_alloc(&sh.tmem_base, kTcTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_base;
  volatile int* abort_flag = &sh.abort_flag;
  const bool dbg_cta = p.dbg != nullptr && static_cast<int>(blockIdx.x) == p.dbg_tile && blockIdx.y == 0;
  TcStamp stamp{(dbg_cta && lane == 0 && (warp == 0 || warp == 1 || warp == 4)) ? p.dbg : nullptr, 0};
  if (dbg_cta && threadIdx.x == 0) { p.dbg[0] = global_timer_ns(); p.dbg[2] = n_blocks; }

  if (warp == 0 || warp == 6) {
    // ---- producers: warp 0 streams the K sides, warp 6 the V sides and the page scales; lane i < 8 owns page i of a stage.
    // K and V have their own barriers because a K tile is free as soon as its QK^T has run, a whole softmax earlier than V.
    const int side = (warp == 0) ? 0 : 1;
    uint64_t* full = side ? sh.v_full : sh.k_full;
    uint64_t* empty = side ? sh.v_empty : sh.k_empty;
    const int n_pages = (ctx + kPageTokens - 1) / kPageTokens;
    const int* table = p.page_table + static_cast<size_t>(seq) * p.max_pages;
    for (int i = 0; i < n_blocks; ++i) {
      const int b = b_begin + i, s = i % kTcStages;
      // K pages past the context are skipped (their keys are masked); V is always filled: masked probabilities are
      // zeros, and a zero must meet finite bytes.
      const int n_load = side ? kTcPages : min(kTcPages, n_pages - b * kTcPages);
      int64_t page = 0;
      if (lane < kTcPages) {
        const int pi = skip_gap_page(min(min(b * kTcPages + lane, n_pages - 1), p.max_pages - 1), p.window, p.sink, kv_lo);
        page = table[pi];
        if (page < 0 || page >= p.num_pages) { atomicOr(p.status, kStatusIndexOutOfRange); page = 0; }
      }
      bool ok = true;
      if (side == 0) stamp.begin();
      if (lane == 0) ok = tc_wait(&empty[s], ((i / kTcStages) & 1) ^ 1, abort_flag);
      if (side == 0) stamp.lap(13);
      if (!__shfl_sync(0xffffffffu, ok, 0)) {
        if (lane == 0) { sh.abort_flag = 1; atomicOr(p.status, kStatusWaitTimeout); }
        break;
      }
      uint8_t* st = stages + s * kTcStageBytes + side * kTcSideBytes;
      if (lane == 0) tc_expect_tx(&full[s], n_load * kTcPageBytes);
      __syncwarp();
      if (lane < n_load) {
        const int row = static_cast<int>(((page * p.hkv + kvh) * 2 + side) * kPageTokens);
        tma_load_2d(st + lane * kTcPageBytes, &kv_map, &full[s], 0, row);
      }
      if (side == 1 && lane < kTcPages) {
        const float2 sc = *reinterpret_cast<const float2*>(p.kv_scales + (page * p.hkv + kvh) * 2);
        sh.scales[s][lane][0] = sc.x;
        sh.scales[s][lane][1] = sc.y;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
    }
  } else if (warp == 1) {
    // ---- MMA issuer: QK(i) runs ahead of the softmax of block i - 1, PV(i - 1) follows as soon as its P tile is there
    asm volatile("bar.sync 2, 160;" ::: "memory");            // the Qhl tile is written
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_e4m3(128, 16, false, false);
      constexpr uint32_t idesc_o = make_idesc_e4m3(128, 16, true, false);
      const uint64_t dq = make_kmajor_sw128_desc(smem_u32(q_tile));
      bool ok = true;
      for (int i = 0; i <= n_blocks && ok; ++i) {
        if (i < n_blocks) {
          const int s = i % kTcStages, b = i & 1;
          stamp.begin();
          ok = tc_wait(&sh.k_full[s], (i / kTcStages) & 1, abort_flag);
          stamp.lap(10);
          if (ok && i >= 2) ok = tc_wait(&sh.s_free[b], ((i >> 1) - 1) & 1, abort_flag);
          stamp.lap(11);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dk = make_kmajor_sw128_desc(smem_u32(stages + s * kTcStageBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8(tmem + 16 * b, dk + 2 * k, dq + 2 * k, idesc_s, k > 0 ? 1u : 0u);
          umma_commit(&sh.s_full[b]);
          umma_commit(&sh.k_empty[s]);
        }
        if (i > 0) {
          const int j = i - 1, s = j % kTcStages, b = j & 1;
          stamp.begin();
          ok = tc_wait(&sh.v_full[s], (j / kTcStages) & 1, abort_flag) && tc_wait(&sh.p_full[b], (j >> 1) & 1, abort_flag);
          stamp.lap(12);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dv = tc_mn_major_desc(smem_u32(stages + s * kTcStageBytes + kTcSideBytes), kTcSideBytes);
          const uint64_t dp = make_kmajor_sw128_desc(smem_u32(p_tile + b * kTcSmallTile));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8(tmem + 32, dv + static_cast<uint64_t>(k) * (4096 >> 4), dp + 2 * k, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(&sh.p_free[b]);
          umma_commit(&sh.v_empty[s]);
          if (j == n_blocks - 1) umma_commit(&sh.o_done);
        }
      }
      if (!ok) { sh.abort_flag = 1; atomicOr(p.status, kStatusWaitTimeout); }
    }
    __syncwarp();
  } else {
    // ---- softmax warps: thread = key `t` of the stage, then head dimension `t` in the epilogue
    const int quarter = warp & 3;
    const int t = 32 * quarter + lane;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(32 * quarter) << 16);
    {
      // Qhl tile: thread (r, c) writes 16 bytes of row r (heads 0..7 hi, then lo), d = 16c .. 16c + 15
      const int st = (warp - 2) * 32 + lane;
      const int r = st >> 3, c = st & 7, g = r & 7;
      float v[16];
      uint4 raw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
      if (g < G) {
        const uint4* src = reinterpret_cast<const uint4*>(p.q + static_cast<size_t>(seq) * p.q_stride + (kvh * G + g) * kTcD + 16 * c);
        raw[0] = src[0];
        raw[1] = src[1];
      }
      float amax = 0.f;
      const uint32_t* w = reinterpret_cast<const uint32_t*>(raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = unpack_bf16(w[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      int e = 0;
      if (amax > 0.f && amax < 3.0e38f) (void)frexpf(amax, &e);      // amax < 2^e
      e = max(min(e - 8, 100), -100);
      const float inv_unit = ldexpf(1.f, -e);                         // |q| * inv_unit < 256
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float x[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float hi, lo;
          tc_split(v[4 * i + k] * inv_unit, hi, lo);
          x[k] = (r < 8) ? hi : lo;
        }
        o[i] = tc_pack_e4m3x2(x[0], x[1]) | (tc_pack_e4m3x2(x[2], x[3]) << 16);
      }
      *reinterpret_cast<uint4*>(q_tile + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
      if (r < 8 && c == 0) sh.q_unit[g] = ldexpf(1.f, e) * p.scale_log2e;
      fence_proxy_async_smem();
    }
    asm volatile("bar.sync 2, 160;" ::: "memory");
    float q_unit[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) q_unit[g] = sh.q_unit[g];
    float m_ref[8], l_run[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) { m_ref[g] = -INFINITY; l_run[g] = 0.f; }
    bool ok = true;
    for (int i = 0; i < n_blocks; ++i) {
      const int s = i % kTcStages, b = i & 1;
      stamp.begin();
      ok = tc_wait(&sh.s_full[b], (i >> 1) & 1, abort_flag);
      stamp.lap(3);
      ok = ok && tc_wait(&sh.v_full[s], (i / kTcStages) & 1, abort_flag);
      stamp.lap(4);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      tc_fence_after();
      uint32_t c[16];
      tmem_ld_32x16(lane_base + 16 * b, c);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.s_free[b]);
      stamp.lap(5);
      const float ks = sh.scales[s][t >> 4][0];
      const float vs = fmaxf(sh.scales[s][t >> 4][1], 1e-30f);
      const float lv = __log2f(vs), inv_v = __fdividef(1.f, vs);
      const int key = (b_begin + i) * kTcKeys + t;
      const bool valid = key < ctx && (key >= kv_lo || key < sink);
      float sc[8], blk[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float raw = __uint_as_float(c[g]) + __uint_as_float(c[8 + g]) * 0.0625f;
        sc[g] = valid ? raw * (ks * q_unit[g]) + lv : -INFINITY;
        blk[g] = warp_max_redux(sc[g]);
      }
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < 8; ++g) sh.wmax[b][quarter][g] = blk[g];
      }
      compute_bar_sync();
      bool grow = false;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        blk[g] = fmaxf(fmaxf(sh.wmax[b][0][g], sh.wmax[b][1][g]), fmaxf(sh.wmax[b][2][g], sh.wmax[b][3][g]));
        grow |= blk[g] > m_ref[g] + kTcLag;
      }
      stamp.lap(6);
      if (grow) {                                           // uniform over the four warps: same inputs everywhere
        float alpha[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float m_new = fmaxf(m_ref[g], blk[g]);
          alpha[g] = (m_new == -INFINITY) ? 1.f : exp2f(m_ref[g] - m_new);
          m_ref[g] = m_new;
          l_run[g] *= alpha[g];
        }
        if (i > 0) {                                        // O^T holds blocks 0 .. i - 1 once PV(i - 1) has retired
          ok = tc_wait(&sh.p_free[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag);
          if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
          tc_fence_after();
          uint32_t o[16];
          tmem_ld_32x16(lane_base + 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            o[g] = __float_as_uint(__uint_as_float(o[g]) * alpha[g]);
            o[8 + g] = __float_as_uint(__uint_as_float(o[8 + g]) * alpha[g]);
          }
          tmem_st_32x16(lane_base + 32, o);
          tc_st_wait();
          tc_fence_before();
        }
      }
      stamp.lap(7);
      float hi[8], lo[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float pr = exp2f(sc[g] - ((m_ref[g] == -INFINITY) ? 0.f : m_ref[g]));
        l_run[g] += pr * inv_v;
        tc_split(pr, hi[g], lo[g]);
      }
      if (i >= 2) {                                         // the P buffer is free once PV(i - 2) has retired
        ok = tc_wait(&sh.p_free[b], ((i >> 1) - 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      }
      stamp.lap(8);
      uint8_t* pt = p_tile + b * kTcSmallTile + (t & 15);
      const int chunk = t >> 4;
#pragma unroll
      for (int g = 0; g < 8; g += 2) {
        const uint32_t h2 = tc_pack_e4m3x2(hi[g], hi[g + 1]), l2 = tc_pack_e4m3x2(lo[g], lo[g + 1]);
        pt[g * 128 + ((chunk ^ g) << 4)] = static_cast<uint8_t>(h2);
        pt[(g + 1) * 128 + ((chunk ^ (g + 1)) << 4)] = static_cast<uint8_t>(h2 >> 8);
        pt[(8 + g) * 128 + ((chunk ^ g) << 4)] = static_cast<uint8_t>(l2);
        pt[(9 + g) * 128 + ((chunk ^ (g + 1)) << 4)] = static_cast<uint8_t>(l2 >> 8);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.p_full[b]);
      stamp.lap(9);
    }
    if (ok) ok = __all_sync(0xffffffffu, tc_wait(&sh.o_done, 0, abort_flag));
    if (!ok) {
      if (lane == 0) { sh.abort_flag = 1; atomicOr(p.status, kStatusWaitTimeout); }
    } else {
      tc_fence_after();
      uint32_t o[16];
      tmem_ld_32x16(lane_base + 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float l = warp_sum(l_run[g]);
        if (lane == 0) sh.lsum[quarter][g] = l;
      }
      compute_bar_sync();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        if (g < G) {
          const float l = sh.lsum[0][g] + sh.lsum[1][g] + sh.lsum[2][g] + sh.lsum[3][g];
          const float acc = __uint_as_float(o[g]) + __uint_as_float(o[8 + g]) * 0.0625f;
          const int head = kvh * G + g;
          if (p.num_splits == 1) {
            p.out[static_cast<size_t>(seq) * p.o_stride + head * kTcD + t] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
          } else {
            const size_t slot = (static_cast<size_t>(seq) * p.hq + head) * p.num_splits + split;
            p.part_o[slot * kTcD + t] = acc;
            if (t == 0) { p.part_ml[slot * 2] = m_ref[g]; p.part_ml[slot * 2 + 1] = l; }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (dbg_cta && threadIdx.x == 0) p.dbg[1] = global_timer_ns();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, kTcTmemCols); }
}

static int tc_tmap(const void* pool, int64_t num_pages, int hkv, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<const void*, std::pair<uint64_t, CUtensorMap>> cache;
  const uint64_t rows = static_cast<uint64_t>(num_pages) * hkv * 2 * kPageTokens;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(pool);
  if (it != cache.end() && it->second.first == rows) { *out = it->second.second; return 0; }
  CUtensorMap m;
  int rc = make_tmap_u8_2d(&m, pool, rows, kTcD, kTcD, kPageTokens, kTcD);
  if (rc != 0) return rc;
  cache[pool] = {rows, m};
  *out = m;
  return 0;
}

static unsigned long long* g_tc_dbg = nullptr;
static int g_tc_dbg_tile = 0;

// Launches the tcgen05 decode kernel; the caller runs the split merge.  `p` is fully filled (e4m3 pages, group <= 8).
int launch_decode_e4m3_tc(const AttnParams& p_in, const void* pool, void* stream) {
  AttnParams p = p_in;
  p.dbg = g_tc_dbg;
  p.dbg_tile = g_tc_dbg_tile;
  CUtensorMap map;
  int rc = tc_tmap(pool, p.num_pages, p.hkv, &map);
  if (rc != 0) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_e4m3_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem));
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_e4m3_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    attr_set = true;
  }
  paged_decode_e4m3_tc_kernel<<<dim3(p.num_seqs * p.num_splits, p.hkv), kTcThreads, kTcSmem, static_cast<cudaStream_t>(stream)>>>(map, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ogb

// Profiling aid: a device buffer of 16 zeroed 64-bit words receives the per-phase nanoseconds of one CTA (block index
// `tile` of the grid's x dimension, KV head 0) of the following launches; nullptr switches it off.
extern "C" void ogb_decode_tc_debug(void* buf16, int tile) {
  ogb::g_tc_dbg = static_cast<unsigned long long*>(buf16);
  ogb::g_tc_dbg_tile = tile;
}
