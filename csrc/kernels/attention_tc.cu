// Chunked causal prefill attention over paged KV on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// The reference's prefill attention is a wmma / SIMT flash-attention over a contiguous KV buffer
// (crates/onnx-runtime-ep-cuda/src/kernels/flash_attention.rs:280-345,352-363).  This kernel reads the
// KV pages in place through the page table and keeps both accumulators in tensor memory:
//
//   one CTA   = 128 query rows of one head (two of the scheduler's 64-row tiles) against the
//               sequence's keys, walked in blocks of BN = 128 tokens (8 pages)
//   warps 0,1 : TMA producers (warp 0: Q and K, warp 1: V).  Q comes from the packed qkv rows through a 2-D
//               tensor map; every K and V page half (16 tokens x 64 dims = 2 KB, 128-byte swizzled) is one
//               TMA box, landed so that a block is [dim half][token][64 dims]: K is then a K-major UMMA
//               operand and V an MN-major one (64-dim blocks BN*128 bytes apart, 8-token groups 1024 bytes apart)
//   warp 2    : one elected lane issues  S_j = Q K_j^T  (smem x smem -> TMEM, fp32) and
//               O_g += P_j V_j (TMEM x smem -> TMEM) in the order S_j, P_{j-1}V_{j-1}, S_{j+1}, ...
//   warps 3-6 : softmax group A, warps 7-10 : softmax group B.  Even key blocks belong to A, odd ones to B;
//               each group has its own score buffer, running maximum, running sum and accumulator O_g, so the
//               two groups never wait for each other: while one waits for its tensor-memory loads, stores and
//               barriers, the other one computes.  One thread owns one query row (a TMEM lane): tcgen05.ld of
//               the row of S in two passes (maximum, then exponentials), masking (causal, context end, sliding
//               window), P as packed bf16 written with tcgen05.st over the columns of S it came from.  The
//               running maximum is only raised when it grows by more than 2^24 (the accumulator is then
//               rescaled in TMEM); otherwise the stale maximum is kept, which leaves O / l exact, and blocks
//               that need no mask take a single pass.
//   epilogue  : the groups exchange their (m, l) and one half of their accumulators through shared memory;
//               each merges and stores one half of the output columns (bf16).
// Every wait is bounded and watches a CTA-wide abort flag; on expiry the status word gets
// kStatusWaitTimeout, the CTA drains, frees its TMEM and returns.  Page ids are bounds-checked.
#include <mutex>
#include <unordered_map>

#include "attention_common.cuh"
#include "ogb_kernels.h"

namespace ogb {

constexpr int kFaBM = 128;
constexpr int kFaFirstSoftmaxWarp = 3;                 // warp 0: K (and Q) producer, 1: V producer, 2: MMA issuer
constexpr int kFaSoftmaxWarps = 8;                     // two groups of four warps (one warp per TMEM lane quarter)
constexpr int kFaThreads = (kFaFirstSoftmaxWarp + kFaSoftmaxWarps) * 32;
// The running maximum of a row is re-centred only when a block's maximum exceeds it by more than this many
// powers of two.  Until then the stale maximum is used: probabilities are then at most 2^24, far inside the
// range of bf16 and of the fp32 sums, and the quotient O / l does not depend on the centre.
constexpr float kFaRecentre = 24.f;

template <int D, int BN>
struct FaCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kQBytes = kFaBM * D * 2;
  static constexpr int kKvBytes = BN * D * 2;          // one K or one V block
  static constexpr int kHalfStrideQ = kFaBM * 128;     // bytes between the 64-dim halves of Q
  static constexpr int kHalfStrideKv = BN * 128;       // bytes between the 64-dim halves of a K / V block
  static constexpr int kStages = 2;
  static constexpr int kSmemBytes = kQBytes + kStages * 2 * kKvBytes + 1024 /*alignment*/ + 512 /*barriers*/ +
                                    2 * kFaBM * 8 /*(m, l) of both groups*/;
  // TMEM columns: O_A | O_B | S0 (P0 over its first 64 columns) | S1 (P1)
  static constexpr int kColO = 0;
  static constexpr int kColS = 2 * D;
  static constexpr int kTmemCols = 512;
  static constexpr int kXPitch = (D / 2 + 4) * 4;      // bytes per row of the accumulator halves exchanged in the epilogue
  static_assert(2 * D + 2 * BN <= 512, "TMEM budget");
  static_assert(BN == 128, "a row of scores is processed as two 64-column chunks");
  static_assert(2 * kFaBM * kXPitch <= kStages * 2 * kKvBytes, "the exchange slab reuses the K/V rings");
};

OGB_DEVICE void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
OGB_DEVICE void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: A is 128 lanes x (K/2) 32-bit columns of packed bf16 pairs.
OGB_DEVICE void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory descriptor of an MN-major operand stored with the 128-byte swizzle: rows of 128 bytes hold
// 64 consecutive MN elements of one K index, eight K indices form a 1024-byte group (stride byte offset),
// and the next 64 MN elements start `lbo` bytes further (leading byte offset).
OGB_DEVICE uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((1024 >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Bounded wait that also gives up as soon as another role of the CTA has raised the abort flag.
OGB_DEVICE bool fa_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
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

// Optional stamps: when p.dbg is set, the CTA (dbg_tile, head 0) accumulates, per role, the nanoseconds spent
// in each kind of wait.  Slots: 0 start, 1 end, 2 setup done, 3 blocks; K producer 4 wait-empty, 5 issue;
// MMA 6 k_full, 8 p_full, 9 v_full; softmax (row 0 of group A) 10 s_full, 11 pv_done, 12 rescales, 13 math,
// 14 epilogue.
struct FaStamp {
  unsigned long long* d;
  uint64_t t;
  OGB_DEVICE void begin() { if (d) t = global_timer_ns(); }
  OGB_DEVICE void end(int slot) { if (d) d[slot] += global_timer_ns() - t; }
};

struct FaBars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_full[2], pv_done[2];
};

// exponentials of one 64-column chunk of a score row: load, mask, exp2((s - m) * scale) as packed bf16 pairs
// written over the chunk's first 32 columns' worth of the P area; returns the chunk's sum
template <int BN>
OGB_DEVICE float fa_exp_chunk(uint32_t s_addr, uint32_t p_addr, int hi, int lo, float scale, float neg_m) {
  uint32_t s[64];
  {
    uint32_t(&c0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
    uint32_t(&c1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
    tmem_ld_32x32(s_addr, c0);
    tmem_ld_32x32(s_addr + 32, c1);
  }
  tmem_ld_wait();
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    const float v0 = (2 * c <= hi && 2 * c >= lo) ? __uint_as_float(s[2 * c]) : -INFINITY;
    const float v1 = (2 * c + 1 <= hi && 2 * c + 1 >= lo) ? __uint_as_float(s[2 * c + 1]) : -INFINITY;
    const float e0 = exp2f(fmaf(v0, scale, neg_m));
    const float e1 = exp2f(fmaf(v1, scale, neg_m));
    sum[c & 3] += e0 + e1;
    s[c] = pack_bf16(e0, e1);          // pair c lands in word c <= 2c: in place
  }
  {
    uint32_t(&c0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
    tmem_st_32x32(p_addr, c0);
  }
  return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

// Fast pass over 32 columns that need no mask: exponentials against the current running maximum, packed into
// `pk` (16 words), the raw maximum folded into `mx`, the sum returned.  `cur` holds the columns; `nxt` (when
// non-null address) is loaded for the following call while this one computes.
OGB_DEVICE float fa_fast32(const uint32_t (&cur)[32], uint32_t (&pk)[16], float scale, float neg_m, float (&mx)[2]) {
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    const float v0 = __uint_as_float(cur[2 * c]), v1 = __uint_as_float(cur[2 * c + 1]);
    mx[0] = fmaxf(mx[0], v0);
    mx[1] = fmaxf(mx[1], v1);
    const float e0 = exp2f(fmaf(v0, scale, neg_m));
    const float e1 = exp2f(fmaf(v1, scale, neg_m));
    sum[c & 1] += e0 + e1;
    pk[c] = pack_bf16(e0, e1);
  }
  return sum[0] + sum[1];
}

OGB_DEVICE float fa_max_chunk(uint32_t s_addr, int hi, int lo) {
  uint32_t s[64];
  {
    uint32_t(&c0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
    uint32_t(&c1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
    tmem_ld_32x32(s_addr, c0);
    tmem_ld_32x32(s_addr + 32, c1);
  }
  tmem_ld_wait();
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < 64; ++c) {
    const float v = (c <= hi && c >= lo) ? __uint_as_float(s[c]) : -INFINITY;
    mx[c & 3] = fmaxf(mx[c & 3], v);
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

template <int D, int BN>
__global__ void __launch_bounds__(kFaThreads, 1)
paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                        const AttnParams p) {
  using Cfg = FaCfg<D, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kQBytes;                      // [stage][kKvBytes]
  uint8_t* sV = sK + Cfg::kStages * Cfg::kKvBytes;      // [stage][kKvBytes]
  FaBars* bars = reinterpret_cast<FaBars*>(sV + Cfg::kStages * Cfg::kKvBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float2* x_ml = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(bars) + 512);   // [group][row] (m, l)

  // ---- which rows ----
  const int tile = blockIdx.x;
  if (tile >= p.num_tiles) return;
  const int q0 = p.tile_q0[tile];
  if ((q0 & 127) != 0) return;                          // the odd 64-row tiles are served by their 128-row neighbours
  const int head = blockIdx.y;
  const int kvh = head / p.group;
  const int seq = p.tile_seq[tile];
  const int q_begin = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - q_begin;
  const int ctx = p.ctx_len[seq];
  const int rows = min(kFaBM, q_len - q0);
  const int pos0 = ctx - q_len + q0;                    // position of the tile's first query row
  if (rows <= 0 || ctx <= 0) return;
  const int kv_end = min(ctx, pos0 + rows);
  const int kv_lo = (p.window > 0) ? max(0, pos0 - p.window + 1) : 0;
  const int b_begin = kv_lo / BN;
  const int b_end = (kv_end + BN - 1) / BN;
  const int nblk = b_end - b_begin;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long* dbg = (p.dbg != nullptr && blockIdx.x == p.dbg_tile && blockIdx.y == 0) ? p.dbg : nullptr;
  if (dbg && threadIdx.x == 0) { dbg[0] = global_timer_ns(); dbg[3] = nblk; }
  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 4);
      mbar_init(&bars->pv_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&q_map);
    tma_prefetch_desc(&kv_map);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (dbg && threadIdx.x == 0) dbg[2] = global_timer_ns() - dbg[0];

  if (warp < 2) {
    // ------------------------------ TMA producers: warp 0 streams Q and K, warp 1 streams V ------------------------------
    if (lane == 0) {
      bool ok = true;
      FaStamp st{warp == 0 ? dbg : nullptr, 0};
      const bool is_v = (warp == 1);
      if (!is_v) {
        mbar_expect_tx(&bars->q_full, Cfg::kQBytes);
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h)
          tma_load_2d(sQ + h * Cfg::kHalfStrideQ, &q_map, &bars->q_full, head * D + h * 64, q_begin + q0);
      }
      const int n_pages = (ctx + kPageTokens - 1) / kPageTokens;
      const int* table = p.page_table + static_cast<size_t>(seq) * p.max_pages;
      uint64_t* full = is_v ? bars->v_full : bars->k_full;
      uint64_t* empty = is_v ? bars->v_empty : bars->k_empty;
      uint8_t* ring = is_v ? sV : sK;
      const int row_add = is_v ? kPageTokens : 0;
      for (int it = 0; it < nblk && ok; ++it) {
        const int b = b_begin + it;
        const int buf = it & 1;
        const uint32_t par = static_cast<uint32_t>((it >> 1) & 1);
        int row_of_page[BN / kPageTokens];
#pragma unroll
        for (int i = 0; i < BN / kPageTokens; ++i) {
          int pi = b * (BN / kPageTokens) + i;
          if (pi > n_pages - 1) pi = n_pages - 1;      // tail: re-read the last page, masked later
          if (pi > p.max_pages - 1) pi = p.max_pages - 1;
          pi = skip_gap_page(pi, p.window, 0, kv_lo);    // pages before the window may have been released
          int64_t page = table[pi];
          if (page < 0 || page >= p.num_pages) {
            atomicOr(p.status, kStatusIndexOutOfRange);
            page = 0;
          }
          row_of_page[i] = static_cast<int>(((page * p.hkv + kvh) * 2) * kPageTokens) + row_add;
        }
        st.begin();
        if (!fa_wait(&empty[buf], par ^ 1, abort_flag)) { ok = false; break; }
        st.end(4);
        st.begin();
        mbar_expect_tx(&full[buf], Cfg::kKvBytes);
        uint8_t* dst = ring + buf * Cfg::kKvBytes;
#pragma unroll
        for (int i = 0; i < BN / kPageTokens; ++i) {
#pragma unroll
          for (int h = 0; h < Cfg::kHalves; ++h)
            tma_load_2d(dst + h * Cfg::kHalfStrideKv + (i << 11), &kv_map, &full[buf], h * 64, row_of_page[i]);
        }
        st.end(5);
      }
      if (!ok) { atomicOr(p.status, kStatusWaitTimeout); *abort_flag = 1; }
    }
  } else if (warp == 2) {
    // ------------------------------ MMA issuer ------------------------------
    // tcgen05.mma instructions of one thread execute in issue order, so S_{j+2}, issued after P_j V_j, cannot
    // overwrite the columns of P_j (which live inside score buffer j & 1) before that product has read them.
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kFaBM, BN);
      constexpr uint32_t idesc_o = make_idesc_bf16(kFaBM, D) | (1u << 16);   // B (= V) is MN-major
      bool ok = fa_wait(&bars->q_full, 0, abort_flag);
      FaStamp st{dbg, 0};
      auto issue_pv = [&](int t) -> bool {
        const int buf = t & 1;
        const uint32_t par = static_cast<uint32_t>((t >> 1) & 1);
        st.begin();
        if (!fa_wait(&bars->p_full[buf], par, abort_flag)) return false;
        st.end(8);
        st.begin();
        if (!fa_wait(&bars->v_full[buf], par, abort_flag)) return false;
        st.end(9);
        tc_fence_after();
        const uint32_t sv = smem_u32(sV + buf * Cfg::kKvBytes);
        const uint32_t p_addr = tmem_base + Cfg::kColS + buf * BN;            // P_t: first BN/2 columns of score buffer t & 1
        const uint32_t o_addr = tmem_base + Cfg::kColO + buf * D;            // accumulator of the group that owns block t
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint64_t db = make_mnmajor_sw128_desc(sv + k * 2048, Cfg::kHalfStrideKv);
          umma_f16_ts(o_addr, p_addr + k * 8, db, idesc_o, (t >= 2 || k > 0) ? 1u : 0u);
        }
        umma_commit(&bars->v_empty[buf]);
        umma_commit(&bars->pv_done[buf]);
        return true;
      };
      for (int it = 0; it < nblk && ok; ++it) {
        const int buf = it & 1;
        const uint32_t par = static_cast<uint32_t>((it >> 1) & 1);
        st.begin();
        if (!fa_wait(&bars->k_full[buf], par, abort_flag)) { ok = false; break; }
        st.end(6);
        tc_fence_after();
        const uint32_t sq = smem_u32(sQ);
        const uint32_t sk = smem_u32(sK + buf * Cfg::kKvBytes);
        const uint32_t s_addr = tmem_base + Cfg::kColS + buf * BN;
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h) {
          const uint64_t da = make_kmajor_sw128_desc(sq + h * Cfg::kHalfStrideQ);
          const uint64_t db = make_kmajor_sw128_desc(sk + h * Cfg::kHalfStrideKv);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(s_addr, da + 2 * k, db + 2 * k, idesc_s, (h | k) != 0 ? 1u : 0u);
        }
        umma_commit(&bars->k_empty[buf]);
        umma_commit(&bars->s_full[buf]);
        if (it >= 1 && !issue_pv(it - 1)) { ok = false; break; }
      }
      if (ok && !issue_pv(nblk - 1)) ok = false;
      if (!ok) { atomicOr(p.status, kStatusWaitTimeout); *abort_flag = 1; }
    }
  } else {
    // ------------------------------ softmax groups / correction / epilogue ------------------------------
    const int q = warp & 3;                              // TMEM lane quarter this warp may touch
    const int g = (warp - kFaFirstSoftmaxWarp) >> 2;     // group: 0 takes the even key blocks, 1 the odd ones
    const int row = q * 32 + lane;                       // query row of this thread
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t s_addr = lane_base + Cfg::kColS + g * BN;
    const uint32_t o_addr = lane_base + Cfg::kColO + g * D;
    const int qpos = pos0 + row;
    const int hi_abs = min(qpos, ctx - 1);
    const int lo_abs = (p.window > 0) ? (qpos - p.window + 1) : 0;
    float m_run = -INFINITY, l_run = 0.f;                // running maximum in the scaled (log2) domain
    bool ok = true;
    FaStamp st{(row == 0 && g == 0) ? dbg : nullptr, 0};
    for (int it = g; it < nblk && ok; it += 2) {
      const uint32_t par = static_cast<uint32_t>((it >> 1) & 1);
      st.begin();
      ok = __all_sync(0xffffffffu, fa_wait(&bars->s_full[g], par, abort_flag));
      st.end(10);
      if (!ok) break;
      st.begin();
      tc_fence_after();
      const int col0 = (b_begin + it) * BN;
      bool done = false;
      // Fast path: every column of the block is visible to every row of the tile and the group already has a
      // running maximum.  One pass: exponentials against the running maximum, kept in registers until the
      // block's own maximum is known; they are stored unless some row's maximum grew past the re-centring
      // threshold, in which case the block takes the two-pass path below (the scores are still intact).
      const bool plain = (it >= 2) && (col0 + BN - 1 <= pos0) && (col0 + BN <= ctx) &&
                         (p.window <= 0 || col0 >= pos0 + kFaBM - p.window);
      if (plain) {
        const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
        uint32_t pk[BN / 2];
        float mx2[2] = {-INFINITY, -INFINITY};
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t a[32];
          tmem_ld_32x32(s_addr + 32 * c, a);
          tmem_ld_wait();
          sum += fa_fast32(a, *reinterpret_cast<uint32_t(*)[16]>(&pk[16 * c]), p.scale_log2e, neg_m, mx2);
        }
        const float mx = fmaxf(mx2[0], mx2[1]) * p.scale_log2e;
        const bool grew = (mx > m_run + kFaRecentre);
        if (!__any_sync(0xffffffffu, grew)) {
          l_run += sum;
          tmem_st_32x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
          tmem_st_32x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
          done = true;
        }
      }
      if (!done) {
        // pass 1: row maximum (columns outside [lo, hi] are masked; both bounds relative to the chunk)
        const float mx = fmaxf(fa_max_chunk(s_addr, hi_abs - col0, lo_abs - col0),
                               fa_max_chunk(s_addr + 64, hi_abs - col0 - 64, lo_abs - col0 - 64)) * p.scale_log2e;   // scale > 0
        const float m_new = fmaxf(m_run, mx);
        const bool raise = (m_new > m_run + kFaRecentre) || (m_run == -INFINITY && m_new > -INFINITY);
        if (it < 2) {
          m_run = m_new;
        } else if (__any_sync(0xffffffffu, raise)) {
          // the accumulator must hold every earlier block of this group before it is rescaled
          const int t = it - 2;
          st.end(13);
          st.begin();
          ok = __all_sync(0xffffffffu, fa_wait(&bars->pv_done[g], static_cast<uint32_t>((t >> 1) & 1), abort_flag));
          st.end(11);
          if (!ok) break;
          st.begin();
          tc_fence_after();
          if (st.d) st.d[12] += 1;
          float alpha = 1.f;
          if (raise) {
            alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
            m_run = m_new;
            l_run *= alpha;
          }
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(o_addr + 32 * c, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st_32x32(o_addr + 32 * c, o);
          }
          tmem_st_wait();
        }
        // pass 2: exponentials; P_it overwrites the first 64 columns of the score buffer, 32 at a time, each
        // chunk only after the scores it covers have been read
        const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
        l_run += fa_exp_chunk<BN>(s_addr, s_addr, hi_abs - col0, lo_abs - col0, p.scale_log2e, neg_m);
        l_run += fa_exp_chunk<BN>(s_addr + 64, s_addr + 32, hi_abs - col0 - 64, lo_abs - col0 - 64, p.scale_log2e, neg_m);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[g]);
      st.end(13);
    }
    // last block of this group: its product must have landed before the accumulator is read
    int last = nblk - 1;
    if ((last & 1) != g) --last;
    if (ok && last >= 0) {
      st.begin();
      ok = __all_sync(0xffffffffu, fa_wait(&bars->pv_done[g], static_cast<uint32_t>((last >> 1) & 1), abort_flag));
      st.end(11);
    }
    if (!ok && lane == 0) {
      atomicOr(p.status, kStatusWaitTimeout);
      *abort_flag = 1;
    }
    st.begin();
    // ---- merge the two groups: each finalises one half of the columns ----
    constexpr int OC = D / 2;
    uint8_t* xo = sK;                                    // [group][row][OC floats], pitch kXPitch; the rings are idle by now
    asm volatile("bar.sync 1, 256;" ::: "memory");       // every tensor-core read of the rings has completed
    const bool live = ok && last >= 0;                   // this group accumulated something
    if (live) {
      tc_fence_after();
      // the half of O_g that the other group finalises
      float* dst = reinterpret_cast<float*>(xo + (static_cast<size_t>(g) * kFaBM + row) * Cfg::kXPitch);
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(o_addr + (g ^ 1) * OC + 32 * c, o);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 8; ++v)
          *reinterpret_cast<uint4*>(dst + 32 * c + 4 * v) = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
      }
    }
    x_ml[g * kFaBM + row] = make_float2(live ? m_run : -INFINITY, live ? l_run : 0.f);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    {
      const float2 other = x_ml[(g ^ 1) * kFaBM + row];
      const float m_mine = live ? m_run : -INFINITY;
      const float m_all = fmaxf(m_mine, other.x);
      const float w_mine = (m_mine == -INFINITY) ? 0.f : exp2f(m_mine - m_all);
      const float w_other = (other.x == -INFINITY) ? 0.f : exp2f(other.x - m_all);
      const float l_tot = (live ? l_run : 0.f) * w_mine + other.y * w_other;
      const float inv = (l_tot > 0.f) ? 1.f / l_tot : 0.f;
      const float a = w_mine * inv, b = w_other * inv;
      const float* src = reinterpret_cast<const float*>(xo + (static_cast<size_t>(g ^ 1) * kFaBM + row) * Cfg::kXPitch);
      __nv_bfloat16* out = p.out + static_cast<size_t>(q_begin + q0 + row) * p.o_stride + head * D + g * OC;
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(o_addr + g * OC + 32 * c, o);
        tmem_ld_wait();
        if (row < rows) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float r[8];
            const uint4 x0 = *reinterpret_cast<const uint4*>(src + 32 * c + 8 * v);
            const uint4 x1 = *reinterpret_cast<const uint4*>(src + 32 * c + 8 * v + 4);
            const uint32_t xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              // a group without blocks holds an uninitialised accumulator: select, never multiply by zero
              const float mine = (a > 0.f) ? __uint_as_float(o[8 * v + j]) * a : 0.f;
              const float oth = (b > 0.f) ? __uint_as_float(xs[j]) * b : 0.f;
              r[j] = mine + oth;
            }
            uint4 w;
            w.x = pack_bf16(r[0], r[1]);
            w.y = pack_bf16(r[2], r[3]);
            w.z = pack_bf16(r[4], r[5]);
            w.w = pack_bf16(r[6], r[7]);
            *reinterpret_cast<uint4*>(out + 32 * c + 8 * v) = w;
          }
        }
      }
    }
    st.end(14);
  }

  tc_fence_before();
  __syncthreads();
  if (dbg && threadIdx.x == 0) dbg[1] = global_timer_ns() - dbg[0];
  if (*abort_flag != 0 && threadIdx.x == 0) {
    // A wait ran out: give copies that may still be in flight a bounded time to land.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------
struct FaMapKey {
  const void* base;
  uint64_t rows, cols, ld;
  bool operator==(const FaMapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld; }
};
struct FaMapKeyHash {
  size_t operator()(const FaMapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (std::hash<uint64_t>()(k.rows) * 1315423911u) ^
           (std::hash<uint64_t>()(k.cols) * 2654435761u) ^ std::hash<uint64_t>()(k.ld);
  }
};

// Tensor maps are pure functions of (address, shape, box); the step executor calls with a handful of
// distinct shapes, so they are encoded once and looked up afterwards.
static int cached_tmap(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<FaMapKey, CUtensorMap, FaMapKeyHash> cache;
  FaMapKey key{base, rows, cols, ld * 1024 + box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  if (cache.size() > 4096) cache.clear();
  CUtensorMap m;
  const int rc = make_tmap_bf16_2d(&m, base, rows, cols, ld, box_rows, 64);
  if (rc != 0) return rc;
  cache.emplace(key, m);
  *out = m;
  return 0;
}

template <int D>
static int launch_prefill_tc(const AttnParams& p, const void* pool, int q_rows, cudaStream_t stream) {
  constexpr int BN = 128;
  using Cfg = FaCfg<D, BN>;
  CUtensorMap q_map, kv_map;
  int rc = cached_tmap(p.q, static_cast<uint64_t>(q_rows), static_cast<uint64_t>(p.hq) * D, static_cast<uint64_t>(p.q_stride),
                       kFaBM, &q_map);
  if (rc != 0) return rc;
  rc = cached_tmap(pool, static_cast<uint64_t>(p.num_pages) * p.hkv * 2 * kPageTokens, D, D, kPageTokens, &kv_map);
  if (rc != 0) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    OGB_CUDA_CHECK(cudaFuncSetAttribute(paged_prefill_tc_kernel<D, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  dim3 grid(p.num_tiles, p.hq);
  paged_prefill_tc_kernel<D, BN><<<grid, kFaThreads, Cfg::kSmemBytes, stream>>>(q_map, kv_map, p);
  return static_cast<int>(cudaGetLastError());
}

static unsigned long long* g_fa_dbg = nullptr;
static int g_fa_dbg_tile = 0;
}  // namespace ogb

using namespace ogb;

// Profiling aid: a device buffer of 16 zeroed 64-bit words receives the per-role wait / work times of one CTA
// (tile index `tile`, head 0) of the following launches; nullptr switches it off.
extern "C" void ogb_prefill_tc_debug(void* buf16, int tile) {
  g_fa_dbg = static_cast<unsigned long long*>(buf16);
  g_fa_dbg_tile = tile;
}

// Same contract as ogb_paged_prefill_bf16 plus `q_rows`, the number of rows of the packed query buffer that
// may be read (the tensor map's bound): tiles are the scheduler's 64-row tiles in any order; each 128-row
// aligned pair is served by one CTA.
extern "C" int ogb_paged_prefill_tc_bf16(const void* q, void* out, const void* pool, const int* page_table, const int* ctx_len,
                                         const int* cu_q, const int* tile_seq, const int* tile_q0, int num_tiles, int num_seqs,
                                         int q_rows, int max_pages, int64_t num_pages, int hq, int hkv, int d, int q_stride,
                                         int o_stride, float scale, int window, int sink, int* status, void* stream) {
  if (num_tiles <= 0) return 0;
  if (window > 0 && sink > 0)   // attention sinks: the block walk with a gap lives in the mma.sync kernel
    return ogb_paged_prefill_bf16(q, out, pool, page_table, ctx_len, cu_q, tile_seq, tile_q0, num_tiles, num_seqs, max_pages,
                                  num_pages, hq, hkv, d, q_stride, o_stride, scale, window, sink, status, stream);
  if ((d != 64 && d != 128) || hkv <= 0 || hq % hkv != 0 || (q_stride % 8) != 0 || (o_stride % 8) != 0 || q_rows <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(pool)) & 15) return -4;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.page_table = page_table; p.ctx_len = ctx_len; p.cu_q = cu_q; p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.num_tiles = num_tiles; p.num_seqs = num_seqs; p.max_pages = max_pages; p.num_pages = num_pages;
  p.hq = hq; p.hkv = hkv; p.group = hq / hkv; p.q_stride = q_stride; p.o_stride = o_stride;
  p.scale_log2e = scale * 1.4426950408889634f; p.window = window; p.num_splits = 1; p.status = status;
  p.dbg = g_fa_dbg; p.dbg_tile = g_fa_dbg_tile;
  return d == 128 ? launch_prefill_tc<128>(p, pool, q_rows, static_cast<cudaStream_t>(stream))
                  : launch_prefill_tc<64>(p, pool, q_rows, static_cast<cudaStream_t>(stream));
}
