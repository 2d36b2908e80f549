// Dense bf16 GEMM for sm_100a:  C[M,N] = A[M,K] * W[N,K]^T  (+bias) (+residual) | SwiGLU.
//
// This is the projection GEMM of the decoder (qkv, o_proj, gate_up, down_proj, lm_head).  It
// takes the place of the library GEMMs the reference calls for MatMul / Gemm / FusedMatMulBias
// (crates/onnx-runtime-ep-cuda/src/blas.rs:305,430, kernels/matmul.rs:649) and of its dense
// GEMV (kernels/matmul.rs:732-748); the SwiGLU epilogue covers the silu_mul glue
// (kernels/elementwise.rs) and the residual epilogue covers the bias-slot residual add of
// optimizer.rs:42-60.
//
// Design (one CTA per SM, persistent over output tiles):
//   warp 0      : TMA producer.  One elected lane streams 128x64 (A) and BNx64 (W) bf16 tiles,
//                 128-byte swizzled, into a shared-memory ring and arms a "full" mbarrier.
//   warp 1      : allocates TMEM, then one elected lane issues tcgen05.mma (M=128, N=BN, K=16)
//                 four times per ring stage; tcgen05.commit releases the stage ("empty") and,
//                 at the end of a tile, publishes the accumulator ("tmem_full").
//   warps 2..5  : epilogue.  Each warp owns one 32-lane quarter of TMEM, reads the fp32
//                 accumulator with tcgen05.ld, applies the epilogue and writes bf16 rows.
//   TMEM holds two accumulators so the epilogue of tile i overlaps the main loop of tile i+1.
// Every wait is bounded; a wait that runs out sets kStatusWaitTimeout in *status, the CTA
// drains and frees its TMEM, and the kernel returns.
#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "ogb_kernels.h"
#include "tp_comm.cuh"

extern "C" int ogb_num_sms() {
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  return num_sms;
}

namespace ogb {

constexpr int kBM = 128;
constexpr int kBK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
constexpr int kGemmThreadsScatter = 224;  // + one warp that publishes finished tiles to peer GPUs

enum GemmEpilogue : int { kEpiNone = 0, kEpiResidual = 1, kEpiSwiGLU = 2, kEpiScatter = 3 };

constexpr int kStagingPitch = 272;                       // bytes per staged row: 128 bf16 + 16 bytes of padding
constexpr int kStagingWarpBytes = 32 * kStagingPitch;    // one epilogue warp: 32 rows

template <int BN>
struct GemmCfg {
  static constexpr int kStageA = kBM * kBK * 2;
  static constexpr int kStageB = BN * kBK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN >= 256) ? 4 : (BN >= 192 ? 4 : (BN >= 128 ? 6 : 8));
  static constexpr int kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));  // power of two
  static constexpr int kSmemBytes = kStages * kStage + 256 /*barriers*/ + 4 * kStagingWarpBytes /*epilogue staging*/;
};

// ----------------------------------------------------------------------------------------
// Work decomposition.  Data-parallel: output tiles are dealt round-robin to the persistent CTAs and a CTA runs the
// whole K loop of each of its tiles.  Stream-K: the (tile, k-block) iterations of all tiles are laid end to end and cut
// into one contiguous, equally long range per CTA, so every SM does the same amount of tensor-core work even when
// the tile count is not a multiple of the SM count.  A range may begin or end in the middle of a tile: the CTA whose
// range holds a tile's last k-block finishes the tile; CTAs that hold an earlier part of it leave their fp32
// accumulator in a workspace slot (one slot per CTA: a range ends inside at most one tile) and raise a flag; the
// finisher, which always has the higher block index, waits for those flags (bounded) and adds the partials before
// its epilogue.  Waiting only on lower-numbered CTAs keeps the scheme free of deadlock whatever the residency, and
// walking every range backwards (GemmWork::next) makes partials the first thing a CTA produces and fix-ups the last.
// ----------------------------------------------------------------------------------------
struct GemmSeg {
  int tile, kb0, kb1;
};

struct GemmWork {
  int k_blocks, num_tiles, stride, tile;   // data-parallel cursor
  long long it, it_end;                    // stream-K cursor over iterations
  bool sk;
  OGB_DEVICE static long long range_begin(long long total, int ctas, int b) {
    const long long base = total / ctas, rem = total % ctas;
    return b * base + (b < rem ? b : rem);
  }
  // the CTA whose range holds iteration i
  OGB_DEVICE static int owner(long long total, int ctas, long long i) {
    const long long base = total / ctas, rem = total % ctas;
    const long long cut = (base + 1) * rem;
    return i < cut ? static_cast<int>(i / (base + 1)) : static_cast<int>(rem + (i - cut) / base);
  }
  OGB_DEVICE GemmWork(bool stream_k, int tiles, int kblocks) : k_blocks(kblocks), num_tiles(tiles), sk(stream_k) {
    stride = gridDim.x;
    tile = blockIdx.x;
    const long long total = static_cast<long long>(tiles) * kblocks;
    it = stream_k ? range_begin(total, gridDim.x, blockIdx.x) : 0;
    it_end = stream_k ? range_begin(total, gridDim.x, blockIdx.x + 1) : 0;
  }
  OGB_DEVICE bool next(GemmSeg& s) {
    if (!sk) {
      if (tile >= num_tiles) return false;
      s.tile = tile; s.kb0 = 0; s.kb1 = k_blocks;
      tile += stride;
      return true;
    }
    // The range is walked from its end to its beginning.  The segment at the end of the range is the head of a tile
    // that a higher-numbered CTA finishes: it is produced first, so the finisher -- for which that tile's tail is the
    // *last* segment -- finds the partial waiting instead of stalling on a neighbour that has its whole range to go.
    if (it_end <= it) return false;
    s.tile = static_cast<int>((it_end - 1) / k_blocks);
    const long long tile_start = static_cast<long long>(s.tile) * k_blocks;
    const long long seg_begin = tile_start > it ? tile_start : it;
    s.kb0 = static_cast<int>(seg_begin - tile_start);
    s.kb1 = static_cast<int>(it_end - tile_start);
    it_end = seg_begin;
    return true;
  }
};

// fp32 partial accumulators of stream-K: slot = CTA, layout [BN / 32 column chunks][128 rows][32 floats], so a warp's
// 32 rows of one chunk are 4 KB contiguous.  flags[cta * 4 + quarter] holds the sequence number of the launch whose
// partial of that row quarter is complete.
template <int BN>
OGB_DEVICE float* sk_slot(float* ws, int cta, int chunk, int row) {
  return ws + ((static_cast<size_t>(cta) * (BN / 32) + chunk) * kBM + row) * 32;
}
OGB_DEVICE void sk_add32(uint32_t (&r)[32], const float* src) {
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    const float4 f = *reinterpret_cast<const float4*>(src + 4 * v);
    r[4 * v + 0] = __float_as_uint(__uint_as_float(r[4 * v + 0]) + f.x);
    r[4 * v + 1] = __float_as_uint(__uint_as_float(r[4 * v + 1]) + f.y);
    r[4 * v + 2] = __float_as_uint(__uint_as_float(r[4 * v + 2]) + f.z);
    r[4 * v + 3] = __float_as_uint(__uint_as_float(r[4 * v + 3]) + f.w);
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreadsScatter, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias,
                         const __nv_bfloat16* residual, float* __restrict__ C_f32, int M, int N, int K, int ldc, int ldr,
                         int* status, const TpScatter* __restrict__ sc, const int* __restrict__ group_tab,
                         const int* __restrict__ group_mtiles, uint32_t* a_ready, uint32_t* a_done, unsigned long long a_wait_ns,
                         float* sk_ws, uint32_t* sk_flags, uint32_t sk_seq) {
  using Cfg = GemmCfg<BN>;
  const bool stream_k = sk_ws != nullptr;
  if constexpr (EPI == kEpiScatter) pdl_trigger();   // the exchange kernel may start: it waits on the tile counters this kernel bumps
  // the kernel declares no static shared memory, so the dynamic window starts at the 1024-byte aligned
  // base the 128-byte swizzle needs
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStage);
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStage + 256;
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kStages;
  uint64_t* tmem_full = bars + 2 * Cfg::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* stored_cnt = tmem_slot + 2;  // [4] tiles stored so far by each epilogue warp (scatter epilogue only)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // grouped (MoE) mode: the m-tile list {expert, first row, end row} and its length live in device memory
  const int m_tiles = group_tab != nullptr ? *group_mtiles : (M + kBM - 1) / kBM;
  const int n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    *abort_flag = 0;
    stored_cnt[0] = stored_cnt[1] = stored_cnt[2] = stored_cnt[3] = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      unsigned long long seen_ready = 0ull;     // m-tiles (of the first 64) whose rows are known to have arrived
      GemmWork work(stream_k, num_tiles, k_blocks);
      GemmSeg seg;
      while (ok && work.next(seg)) {
        const int tile = seg.tile;
        const int mt = tile % m_tiles;
        const int n0 = (tile / m_tiles) * BN;
        const int m0 = group_tab != nullptr ? group_tab[4 * mt + 1] : mt * kBM;
        const int b_row = group_tab != nullptr ? group_tab[4 * mt] * N + n0 : n0;   // expert e's weights start at row e*N
        if (a_ready != nullptr && !(mt < 64 && ((seen_ready >> mt) & 1ull))) {
          // The rows of A are delivered by other GPUs (the all-gather half of a tensor-parallel exchange): every 8
          // rows that land bump the tile's counter.  Wait, bounded, until the whole tile is here; the loads below
          // go through the async proxy, so a proxy fence follows the acquire.
          const uint32_t want = static_cast<uint32_t>((min(kBM, M - m0) + 7) / 8);
          const uint64_t lim = a_wait_ns ? a_wait_ns : kWaitLimitNs;
          const uint64_t t0 = global_timer_ns();
          uint32_t spins = 0, got = 0;
          while (true) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(a_ready + mt) : "memory");
            if (got >= want) break;
            if (((++spins) & 0x3f) == 0 && global_timer_ns() - t0 > lim) { ok = false; break; }   // bounded by the timer
          }
          if (!ok) { atomicOr(status, kStatusPeerTimeout); break; }
          asm volatile("fence.proxy.async.global;" ::: "memory");
          if (mt < 64) seen_ready |= 1ull << mt;
        }
        for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStage;
          uint8_t* sb = sa + Cfg::kStageA;
          mbar_expect_tx(&full_bar[stage], Cfg::kStage);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * kBK, m0);
          tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBK, b_row);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { atomicOr(status, kStatusWaitTimeout); *abort_flag = 1; }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      GemmWork work(stream_k, num_tiles, k_blocks);
      GemmSeg seg;
      for (; ok && work.next(seg); ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_addr = tmem_base + acc * BN;
        for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStage);
          const uint32_t sb = sa + Cfg::kStageA;
          const uint64_t da = make_kmajor_sw128_desc(sa);
          const uint64_t db = make_kmajor_sw128_desc(sb);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // advance 16 bf16 = 32 bytes inside the swizzle row: +2 in the (>>4) address field
            umma_f16(d_addr, da + 2 * k, db + 2 * k, idesc, (kb > seg.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
      if (!ok) { atomicOr(status, kStatusWaitTimeout); *abort_flag = 1; }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    bool ok = true;
    int it = 0;
    GemmWork work(stream_k, num_tiles, k_blocks);
    GemmSeg seg;
    const long long sk_total = static_cast<long long>(num_tiles) * k_blocks;
    for (; ok && work.next(seg); ++it) {
      const int tile = seg.tile;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int mt = tile % m_tiles;
      const int m0 = group_tab != nullptr ? group_tab[4 * mt + 1] : mt * kBM;
      const int m_end = group_tab != nullptr ? group_tab[4 * mt + 2] : M;   // rows past m_end belong to the next expert
      const int n_tile = tile / m_tiles;
      const int n0 = n_tile * BN;
      // every lane polls (each needs the acquire); the vote keeps the warp converged for tcgen05.ld
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_phase))) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      // ---- stream-K: a partial segment leaves its accumulator in this CTA's workspace slot; the segment that
      // finishes a tile begun by other CTAs waits for their slots and adds them below ----
      int fix_lo = 0, fix_hi = 0;                      // CTAs [fix_lo, fix_hi) hold earlier parts of this tile
      if (stream_k) {
        if (seg.kb1 < k_blocks) {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c * 32, r);
            tmem_ld_wait();
            float* dst = sk_slot<BN>(sk_ws, blockIdx.x, c, q * 32 + lane);
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<float4*>(dst + 4 * v) = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                                  __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
          }
          __syncwarp();
          if (lane == 0) {
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(sk_flags + blockIdx.x * 4 + q), "r"(sk_seq) : "memory");
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
          continue;
        }
        if (seg.kb0 > 0) {
          fix_lo = GemmWork::owner(sk_total, gridDim.x, static_cast<long long>(tile) * k_blocks);
          fix_hi = blockIdx.x;
          for (int x = fix_lo; x < fix_hi && ok; ++x) {
            const uint64_t t0 = global_timer_ns();
            uint32_t spins = 0, got = 0;
            while (true) {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(got) : "l"(sk_flags + x * 4 + q) : "memory");
              if (got == sk_seq) break;
              if (((++spins) & 0x3f) == 0 && global_timer_ns() - t0 > kWaitLimitNs) { ok = false; break; }   // bounded by the timer
            }
          }
          if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        }
      }
      if (C_f32 != nullptr) {
        // fp32 output (diagnostics / fp32 logits): direct row-per-thread stores
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
          for (int x = fix_lo; x < fix_hi; ++x) sk_add32(r, sk_slot<BN>(sk_ws, x, c, q * 32 + lane));
          const int col = n0 + c * 32;
          if (row < m_end && col < N) {
            float* dst = C_f32 + static_cast<size_t>(row) * ldc + col;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < N) {
                float v = __uint_as_float(r[j]);
                if (bias != nullptr) v += __bfloat162float(bias[col + j]);
                if constexpr (EPI == kEpiResidual) v += __bfloat162float(residual[static_cast<size_t>(row) * ldr + col + j]);
                dst[j] = v;
              }
            }
          }
        }
      } else {
        // bf16 output.  Phase 1 (thread = row): TMEM -> registers -> epilogue math -> bf16 into this warp's
        // staging slab (32 rows x up to 128 columns, 272-byte pitch: conflict-free for 16-byte accesses).
        // Phase 2 (lanes along the row): 16-byte vectors are read back so that a warp instruction covers
        // whole 256-byte row segments; residual reads and output stores are therefore coalesced.
        constexpr int OUTW = (EPI == kEpiSwiGLU) ? BN / 2 : BN;      // output columns this tile produces
        const int out_cols = (EPI == kEpiSwiGLU) ? N / 2 : N;        // output matrix width
        const int out_col0 = (EPI == kEpiSwiGLU) ? n_tile * (BN / 2) : n0;
        uint8_t* stg = staging + (warp - 2) * kStagingWarpBytes;
#pragma unroll 1
        for (int cb = 0; cb < OUTW; cb += 128) {
          const int cw = (OUTW - cb < 128) ? OUTW - cb : 128;         // 128, 64 or 32
#pragma unroll 1
          for (int c = 0; c < cw / 32; ++c) {
            uint32_t o[16];
            if constexpr (EPI == kEpiSwiGLU) {
              uint32_t g[32], u[32];
              tmem_ld_32x32(t_row + cb + c * 32, g);
              tmem_ld_32x32(t_row + BN / 2 + cb + c * 32, u);
              tmem_ld_wait();
              for (int x = fix_lo; x < fix_hi; ++x) {
                sk_add32(g, sk_slot<BN>(sk_ws, x, (cb + c * 32) / 32, q * 32 + lane));
                sk_add32(u, sk_slot<BN>(sk_ws, x, (BN / 2 + cb + c * 32) / 32, q * 32 + lane));
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
                const float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
                o[j] = pack_bf16(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
              }
            } else {
              uint32_t r[32];
              tmem_ld_32x32(t_row + cb + c * 32, r);
              tmem_ld_wait();
              for (int x = fix_lo; x < fix_hi; ++x) sk_add32(r, sk_slot<BN>(sk_ws, x, (cb + c * 32) / 32, q * 32 + lane));
              const int col = n0 + cb + c * 32;
              if (bias != nullptr && col < N) {
                if (col + 32 <= N) {
#pragma unroll
                  for (int j4 = 0; j4 < 4; ++j4) {
                    const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + col) + j4);
                    float2 f;
                    f = unpack_bf16(bv.x); r[8 * j4 + 0] = __float_as_uint(__uint_as_float(r[8 * j4 + 0]) + f.x); r[8 * j4 + 1] = __float_as_uint(__uint_as_float(r[8 * j4 + 1]) + f.y);
                    f = unpack_bf16(bv.y); r[8 * j4 + 2] = __float_as_uint(__uint_as_float(r[8 * j4 + 2]) + f.x); r[8 * j4 + 3] = __float_as_uint(__uint_as_float(r[8 * j4 + 3]) + f.y);
                    f = unpack_bf16(bv.z); r[8 * j4 + 4] = __float_as_uint(__uint_as_float(r[8 * j4 + 4]) + f.x); r[8 * j4 + 5] = __float_as_uint(__uint_as_float(r[8 * j4 + 5]) + f.y);
                    f = unpack_bf16(bv.w); r[8 * j4 + 6] = __float_as_uint(__uint_as_float(r[8 * j4 + 6]) + f.x); r[8 * j4 + 7] = __float_as_uint(__uint_as_float(r[8 * j4 + 7]) + f.y);
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (col + j < N) r[j] = __float_as_uint(__uint_as_float(r[j]) + __bfloat162float(bias[col + j]));
                }
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) o[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            }
            uint4* srow = reinterpret_cast<uint4*>(stg + lane * kStagingPitch + c * 64);
#pragma unroll
            for (int v = 0; v < 4; ++v) srow[v] = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
          }
          __syncwarp();
          const int lanes_per_row = cw / 8;                 // 16, 8 or 4 sixteen-byte vectors per row segment
          const int rows_per_pass = 32 / lanes_per_row;
          const int ch = lane % lanes_per_row;
          const int gcol = out_col0 + cb + ch * 8;
          // the residual vectors of a batch of passes are requested together (memory-level parallelism:
          // one L2 round trip per batch instead of one per row) before any of them is consumed
          constexpr int kBatch = 8;
#pragma unroll 1
          for (int rb = 0; rb < 32; rb += rows_per_pass * kBatch) {
            uint4 resv[kBatch];
            if constexpr (EPI == kEpiResidual) {
#pragma unroll
              for (int t = 0; t < kBatch; ++t) {
                const int r_loc = rb + t * rows_per_pass + lane / lanes_per_row;
                const int grow = m0 + q * 32 + r_loc;
                resv[t] = make_uint4(0, 0, 0, 0);
                if (r_loc < 32 && grow < m_end && gcol + 8 <= out_cols)
                  resv[t] = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(grow) * ldr + gcol);
              }
            }
#pragma unroll
            for (int t = 0; t < kBatch; ++t) {
              const int r_loc = rb + t * rows_per_pass + lane / lanes_per_row;
              const int grow = m0 + q * 32 + r_loc;
              if (r_loc < 32 && grow < m_end && gcol < out_cols) {
                uint4 v = *reinterpret_cast<const uint4*>(stg + r_loc * kStagingPitch + ch * 16);
                __nv_bfloat16* dst;
                if constexpr (EPI == kEpiScatter) {
                  if (sc->push) {
                    // straight into the buffer of the rank that owns the row (a peer store over NVLink, or a local one):
                    // slab [this rank][row within the owner's chunk]; the stores drain under the next tile's main loop
                    const int owner = grow / sc->chunk;
                    dst = sc->staging[owner] + (static_cast<size_t>(sc->rank) * sc->chunk + (grow - owner * sc->chunk)) * N + gcol;
                  } else {
                    // the partial product stays in this rank's own buffer; the owner of the row pulls it
                    dst = sc->staging[sc->rank] + static_cast<size_t>(grow) * N + gcol;
                  }
                } else {
                  dst = C + static_cast<size_t>(grow) * ldc + gcol;
                }
                const bool full = (gcol + 8 <= out_cols);
                if constexpr (EPI == kEpiResidual) {
                  if (full) {
                    const uint4 rv = resv[t];
                    float2 a, b2;
                    a = unpack_bf16(v.x); b2 = unpack_bf16(rv.x); v.x = pack_bf16(a.x + b2.x, a.y + b2.y);
                    a = unpack_bf16(v.y); b2 = unpack_bf16(rv.y); v.y = pack_bf16(a.x + b2.x, a.y + b2.y);
                    a = unpack_bf16(v.z); b2 = unpack_bf16(rv.z); v.z = pack_bf16(a.x + b2.x, a.y + b2.y);
                    a = unpack_bf16(v.w); b2 = unpack_bf16(rv.w); v.w = pack_bf16(a.x + b2.x, a.y + b2.y);
                    *reinterpret_cast<uint4*>(dst) = v;
                  } else {
                    const __nv_bfloat16* rs = residual + static_cast<size_t>(grow) * ldr + gcol;
                    const __nv_bfloat16* pv = reinterpret_cast<const __nv_bfloat16*>(&v);
                    for (int j = 0; j < 8 && gcol + j < out_cols; ++j)
                      dst[j] = __float2bfloat16(__bfloat162float(pv[j]) + __bfloat162float(rs[j]));
                  }
                } else {
                  if (full) {
                    *reinterpret_cast<uint4*>(dst) = v;
                  } else {
                    const __nv_bfloat16* pv = reinterpret_cast<const __nv_bfloat16*>(&v);
                    for (int j = 0; j < 8 && gcol + j < out_cols; ++j) dst[j] = pv[j];
                  }
                }
              }
            }
          }
          __syncwarp();
        }
      }
      if constexpr (EPI == kEpiScatter) {
        // hand the finished warp tile to the signal warp: the warp barrier orders every lane's stores
        // before lane 0, whose CTA-scope release on the shared counter the signal lane acquires
        __syncwarp();
        if (lane == 0) asm volatile("red.release.cta.shared::cta.add.u32 [%0], 1;" ::"r"(smem_u32(&stored_cnt[q])) : "memory");
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
    if (!ok && lane == 0) { atomicOr(status, kStatusWaitTimeout); *abort_flag = 1; }
  } else {
    // ------------------------------ signal warp (scatter epilogue) ------------------------------
    // Lane q publishes the tiles of epilogue warp q: once that warp's stores are ordered (acquire on
    // its counter) a system-scope release bumps the arrival counter of the rank that owns the 32-row
    // group.  The tensor-core and epilogue warps never execute a system-scope fence.
    if constexpr (EPI == kEpiScatter) {
      if (lane < 4) {
        const int q = lane;  // row quarter of the tile = TMEM quarter of the epilogue warp that stores it
        uint32_t done = 0;
        bool ok = true;
        GemmWork work(stream_k, num_tiles, k_blocks);
        GemmSeg seg;
        while (ok && work.next(seg)) {
          if (seg.kb1 < k_blocks) continue;            // a partial segment stores nothing: its finisher signals the tile
          const int tile = seg.tile;
          const uint64_t t0 = global_timer_ns();
          uint32_t spins = 0;
          while (true) {
            uint32_t v;
            asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(&stored_cnt[q])) : "memory");
            if (v > done) break;
            if (*abort_flag != 0 || (((++spins) & 0x3ff) == 0 && global_timer_ns() - t0 > kWaitLimitNs)) { ok = false; break; }
          }
          if (!ok) break;
          const int m0 = (tile % m_tiles) * kBM;
          const int n0 = (tile / m_tiles) * BN;
          const int row0 = m0 + q * 32;
          if (row0 < M) {
            const int owner = row0 / sc->chunk;
            uint32_t* cnt = sc->tile_cnt[owner] + (row0 - owner * sc->chunk) / 32;
            // counted in 32-column units so the owner's expectation (N/32 per source rank) does not
            // depend on the tile width this launch picked
            const uint32_t units = static_cast<uint32_t>(min(BN, N - n0) / 32);
            asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(units) : "memory");
          }
          ++done;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    // A wait ran out: give copies that may still be in flight a bounded time to land.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (a_ready != nullptr && threadIdx.x == 0) {
    // The consumer clears what it consumed: the last CTA to finish zeroes the tiles' ready counters.  The next
    // arrivals on them belong to an exchange that needs this rank's next row-parallel GEMM, which is launched
    // after this kernel, so no arrival can be lost.
    __threadfence();
    if (atomicAdd(a_done, 1u) == gridDim.x - 1) {
      for (int i = 0; i < m_tiles; ++i) a_ready[i] = 0;
      *a_done = 0;
      __threadfence();
    }
  }
}

// ----------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

int encode_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                        uint32_t box_cols);

// Descriptors that were encoded before, per thread: a tensor map is a pure function of (address, extents, stride, box),
// the weights and the static activation buffers come back with the same values at every step, and a lookup costs a tenth
// of an encode.  The table is dropped when it grows past a bound (a process that keeps making new shapes).
struct TmapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && box_cols == o.box_cols;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.cols * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2));
    h ^= (k.ld + (static_cast<uint64_t>(k.box_rows) << 32) + k.box_cols + (h << 6) + (h >> 2));
    return static_cast<size_t>(h);
  }
};

// 2-D row-major bf16 matrix [rows, cols] with row stride `ld` elements; box = {64 cols, box_rows}.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols) {
  static thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const TmapKey key{base, rows, cols, ld, box_rows, box_cols};
  auto hit = cache.find(key);
  if (hit != cache.end()) {
    *out = hit->second;
    return 0;
  }
  const int rc = encode_tmap_bf16_2d(out, base, rows, cols, ld, box_rows, box_cols);
  if (rc == 0) {
    if (cache.size() > 16384) cache.clear();
    cache.emplace(key, *out);
  }
  return rc;
}

int encode_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                        uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}


// 2-D row-major byte matrix [rows, cols] (e4m3 KV pages); box = {box_cols bytes (<= 128), box_rows}.
int make_tmap_u8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

// Stream-K workspace: one fp32 slot of 128 x 256 per CTA plus four flag words per CTA, allocated once per
// (device, stream) at the first launch that wants it (outside any stream capture: a step is run eagerly before it
// is captured).  Launches on one stream are ordered, so they can share a workspace; the sequence number written
// into the flags distinguishes their partials without any reset.
struct SkWorkspace {
  float* ws = nullptr;
  uint32_t* flags = nullptr;
  uint32_t seq = 0;
  int ctas = 0;
};

static SkWorkspace* sk_workspace(cudaStream_t stream, int ctas) {
  static std::mutex mu;
  static std::unordered_map<uint64_t, SkWorkspace> table;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  const uint64_t key = (static_cast<uint64_t>(dev) << 56) ^ reinterpret_cast<uint64_t>(stream);
  std::lock_guard<std::mutex> lock(mu);
  SkWorkspace& w = table[key];
  if (w.ws == nullptr || w.ctas < ctas) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    if (w.ws != nullptr) { cudaFree(w.ws); cudaFree(w.flags); w.ws = nullptr; w.flags = nullptr; }
    const size_t bytes = static_cast<size_t>(ctas) * kBM * 256 * sizeof(float);
    if (cudaMalloc(&w.ws, bytes) != cudaSuccess) { w.ws = nullptr; return nullptr; }
    if (cudaMalloc(&w.flags, static_cast<size_t>(ctas) * 4 * sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(w.flags, 0, static_cast<size_t>(ctas) * 4 * sizeof(uint32_t)) != cudaSuccess) {
      cudaFree(w.ws);
      w.ws = nullptr;
      return nullptr;
    }
    w.ctas = ctas;
    w.seq = 0;
  }
  return &w;
}

static int g_stream_k = -1;     // -1: read OGB_STREAM_K once (default on); 0 / 1 set by ogb_gemm_set_stream_k

static bool stream_k_enabled() {
  if (g_stream_k < 0) {
    const char* e = getenv("OGB_STREAM_K");
    g_stream_k = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return g_stream_k == 1;
}
// Stream-K pays when round-robin tiles would leave a large part of the last wave idle and the fix-up is cheap next
// to a tile: every CTA boundary that falls inside a tile costs one fp32 partial written and read back and a flag wait
// in the finisher.  `fix` is that cost in k-blocks of tensor-core time.  Measured on the 7B shapes (tile widths 32 - 256
// with and without stream-K, M = 32 - 1472): about 40 for a plain epilogue -- with 13 the estimate chose wide stream-K
// tiles for K = 3584 projections that ran 1.3 - 1.5x slower than plain 128-wide tiles -- while the scatter epilogue of
// the tensor-parallel path, whose tiles end in stores to other GPUs, keeps the 13 it was tuned with.
constexpr float kSkFixPlain = 40.0f;
constexpr float kSkFixScatter = 13.0f;
static bool stream_k_applies(int tiles, int k_blocks, int sms, float fix) {
  if (!stream_k_enabled() || tiles % sms == 0 || static_cast<long long>(tiles) * k_blocks < 2LL * sms) return false;
  const float w = static_cast<float>(tiles) / static_cast<float>(sms);
  const float dp = static_cast<float>((tiles + sms - 1) / sms);
  const float sk = w + fix / static_cast<float>(k_blocks);
  return sk < 0.93f * dp;
}
// Relative duration of a launch with `tiles` tiles of relative cost `cost`: whole waves when tiles are dealt
// round-robin, the exact share plus the fix-up when stream-K spreads the k-blocks evenly.
static float launch_cost(int tiles, int k_blocks, int sms, float cost, float fix) {
  if (stream_k_applies(tiles, k_blocks, sms, fix))
    return (static_cast<float>(tiles) / static_cast<float>(sms) + fix / static_cast<float>(k_blocks)) * cost;
  return static_cast<float>((tiles + sms - 1) / sms) * cost;
}

template <int BN, int EPI>
static int launch_gemm(const void* A, const void* W, void* C, const void* bias, const void* residual, void* C_f32, int M,
                       int N, int K, int lda, int ldw, int ldc, int ldr, int* status, cudaStream_t stream,
                       const TpScatter* sc = nullptr, const int* group_tab = nullptr, const int* group_mtiles = nullptr,
                       int experts = 1, int max_mtiles = 0, uint32_t* a_ready = nullptr, uint32_t* a_done = nullptr,
                       unsigned long long a_wait_ns = 0) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap ta, tb;
  int rc = make_tmap_bf16_2d(&ta, A, M, K, lda, kBM, kBK);
  if (rc != 0) return rc;
  rc = make_tmap_bf16_2d(&tb, W, static_cast<uint64_t>(N) * experts, K, ldw, BN, kBK);
  if (rc != 0) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    OGB_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg::kSmemBytes));
    attr_set = true;
  }
  const int m_tiles = group_tab != nullptr ? max_mtiles : (M + kBM - 1) / kBM, n_tiles = (N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int sms = ogb_num_sms();
  int grid = tiles;
  if (grid > sms) grid = sms;
  // Stream-K when the tiles do not fill whole waves and there are few waves (with many, the idle tail is a small
  // share and the workspace traffic is not worth it); not for grouped (MoE) launches, whose tile table lives on the device.
  float* sk_ws = nullptr;
  uint32_t* sk_flags = nullptr;
  uint32_t sk_seq = 0;
  const int k_blocks = (K + kBK - 1) / kBK;
  if (group_tab == nullptr && stream_k_applies(tiles, k_blocks, sms, EPI == kEpiScatter ? kSkFixScatter : kSkFixPlain)) {
    SkWorkspace* w = sk_workspace(stream, sms);
    if (w != nullptr) {
      grid = sms;
      sk_ws = w->ws;
      sk_flags = w->flags;
      sk_seq = ++w->seq;
      if (sk_seq == 0) sk_seq = ++w->seq;     // the flags start at zero
    }
  }
  // A GEMM whose A rows arrive behind per-tile counters follows the exchange kernel that fills them: with PDL it starts
  // while that kernel is still running.
  const bool pdl = a_ready != nullptr && tp_pdl_enabled() != 0;
  return static_cast<int>(launch_kernel_pdl(
      gemm_bf16_tcgen05_kernel<BN, EPI>, dim3(grid), dim3(EPI == kEpiScatter ? kGemmThreadsScatter : kGemmThreads), Cfg::kSmemBytes, stream,
      pdl, ta, tb, static_cast<__nv_bfloat16*>(C), static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(residual),
      static_cast<float*>(C_f32), M, N, K, ldc, ldr, status, sc, group_tab, group_mtiles, a_ready, a_done,
      static_cast<unsigned long long>(a_wait_ns), sk_ws, sk_flags, sk_seq));
}

}  // namespace ogb

using namespace ogb;

#define OGB_GEMM_ARGS A, W, C, bias, residual, C_f32, M, N, K, lda, ldw, ldc, ldr, status, stream, nullptr, nullptr, nullptr, 1, 0, a_ready, a_done, a_wait_ns
#define OGB_GEMM_DISPATCH_BN(EPI)                              \
  switch (bn) {                                                \
    case 32: return launch_gemm<32, EPI>(OGB_GEMM_ARGS);       \
    case 64: return launch_gemm<64, EPI>(OGB_GEMM_ARGS);       \
    case 128: return launch_gemm<128, EPI>(OGB_GEMM_ARGS);     \
    case 192: return launch_gemm<192, EPI>(OGB_GEMM_ARGS);     \
    case 256: return launch_gemm<256, EPI>(OGB_GEMM_ARGS);     \
    default: return -2;                                        \
  }

// The GEMM whose A rows arrive from other GPUs: `a_ready` holds one counter per 128-row tile of A that grows by one
// for every 8 rows delivered (tp_exchange_norm_kernel); the TMA producer waits for a tile's counter, at most
// `a_wait_ns` nanoseconds (0 = the library default), before it loads the tile; the last CTA to finish zeroes the
// counters again (`a_done` is a zero-initialised word it counts finished CTAs in).  a_ready == nullptr: no wait.
extern "C" int ogb_gemm_bf16_wait(const void* A, const void* W, void* C, const void* bias, const void* residual, void* C_f32,
                                  int M, int N, int K, int lda, int ldw, int ldc, int ldr, int epilogue, int bn,
                                  uint32_t* a_ready, uint32_t* a_done, unsigned long long a_wait_ns, int* status, void* stream_);

// Switches the stream-K decomposition on (1) or off (0) for the GEMMs launched from now on; returns the old setting.
extern "C" int ogb_gemm_set_stream_k(int on) {
  const int old = g_stream_k < 0 ? 1 : g_stream_k;
  g_stream_k = on ? 1 : 0;
  return old;
}

extern "C" int ogb_gemm_bf16(const void* A, const void* W, void* C, const void* bias, const void* residual, void* C_f32,
                             int M, int N, int K, int lda, int ldw, int ldc, int ldr, int epilogue, int bn, int* status,
                             void* stream_) {
  return ogb_gemm_bf16_wait(A, W, C, bias, residual, C_f32, M, N, K, lda, ldw, ldc, ldr, epilogue, bn, nullptr, nullptr, 0, status, stream_);
}

extern "C" int ogb_gemm_bf16_wait(const void* A, const void* W, void* C, const void* bias, const void* residual, void* C_f32,
                                  int M, int N, int K, int lda, int ldw, int ldc, int ldr, int epilogue, int bn,
                                  uint32_t* a_ready, uint32_t* a_done, unsigned long long a_wait_ns, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a_ready != nullptr && a_done == nullptr) return -8;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) != 0 || (lda % 8) != 0 || (ldw % 8) != 0 || (ldc % 8) != 0) return -3;  // 16-byte TMA / vector rules
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(C)) & 15) return -4;
  if (epilogue == kEpiResidual && (residual == nullptr || (ldr % 8) != 0)) return -5;
  if (epilogue == kEpiSwiGLU && (bn < 64 || (N % bn) != 0 || C_f32 != nullptr)) return -6;
  if (bn == 0) {
    // Tiles are handed out round-robin to one persistent CTA per SM, so the kernel takes
    // ceil(tiles / SMs) "waves" of one tile time each.  Pick the tile width with the lowest
    // waves x relative-tile-cost (narrower tiles re-read A more often and amortise the epilogue
    // worse, hence the > bn/256 costs); ties go to the wider tile.
    const int m_tiles = (M + kBM - 1) / kBM;
    const int sms = ogb_num_sms();
    // Measured on B200: with one CTA per tile, a 128-wide tile is shared-memory-bandwidth bound
    // (A and B are re-read per MMA) and costs ~0.62 of a 256-wide one, not 0.5.
    const int cand[5] = {256, 192, 128, 64, 32};
    const float cost[5] = {1.0f, 0.78f, 0.62f, 0.40f, 0.28f};
    float best = 1e30f;
    bn = 256;
    for (int i = 0; i < 5; ++i) {
      if (cand[i] < 128 && m_tiles > 3) break;  // narrow tiles only pay off for decode-sized M
      const int tiles = m_tiles * ((N + cand[i] - 1) / cand[i]);
      const float t = launch_cost(tiles, (K + kBK - 1) / kBK, sms, cost[i], kSkFixPlain);
      if (t < best - 1e-6f) { best = t; bn = cand[i]; }
    }
  }
  if (epilogue == kEpiNone) { OGB_GEMM_DISPATCH_BN(kEpiNone) }
  if (epilogue == kEpiResidual) { OGB_GEMM_DISPATCH_BN(kEpiResidual) }
  if (epilogue == kEpiSwiGLU) {
    switch (bn) {
      case 64: return launch_gemm<64, kEpiSwiGLU>(OGB_GEMM_ARGS);
      case 128: return launch_gemm<128, kEpiSwiGLU>(OGB_GEMM_ARGS);
      case 256: return launch_gemm<256, kEpiSwiGLU>(OGB_GEMM_ARGS);
      default: return -2;
    }
  }
  return -7;
}

// Row-parallel GEMM of a tensor-parallel group: the partial product A[M,K_local] * W[N,K_local]^T of
// this rank is written tile by tile into this rank's peer-mapped partial buffer, and the arrival
// counter of the rank that owns each 32-row group is bumped as soon as the tile is stored.  `sc` is a device-resident TpScatter.
extern "C" int ogb_gemm_bf16_scatter(const void* A, const void* W, int M, int N, int K, int lda, int ldw, const void* sc,
                                     int bn, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0) return 0;
  if ((K % 8) != 0 || (lda % 8) != 0 || (ldw % 8) != 0 || (N % 32) != 0 || sc == nullptr) return -3;
  if (bn == 0) {      // OGB_TP_SCATTER_BN=128|192|256 fixes the tile width (an A/B switch for measurements)
    static int forced = -1;
    if (forced < 0) {
      const char* e = getenv("OGB_TP_SCATTER_BN");
      forced = e != nullptr ? atoi(e) : 0;
      if (forced != 128 && forced != 192 && forced != 256) forced = 0;
    }
    bn = forced;
  }
  if (bn == 0) {
    const int m_tiles = (M + kBM - 1) / kBM;
    const int sms = ogb_num_sms();
    const int cand[3] = {256, 192, 128};
    const float cost[3] = {1.0f, 0.78f, 0.62f};
    float best = 1e30f;
    bn = 256;
    for (int i = 0; i < 3; ++i) {
      const int tiles = m_tiles * ((N + cand[i] - 1) / cand[i]);
      const float t = launch_cost(tiles, (K + kBK - 1) / kBK, sms, cost[i], kSkFixScatter);
      if (t < best - 1e-6f) { best = t; bn = cand[i]; }
    }
  }
  const TpScatter* s = static_cast<const TpScatter*>(sc);
  void* dummy = const_cast<void*>(A);  // C is unused by the scatter epilogue but must be 16-byte aligned
  switch (bn) {
    case 128: return launch_gemm<128, kEpiScatter>(A, W, dummy, nullptr, nullptr, nullptr, M, N, K, lda, ldw, N, 0, status, stream, s);
    case 192: return launch_gemm<192, kEpiScatter>(A, W, dummy, nullptr, nullptr, nullptr, M, N, K, lda, ldw, N, 0, status, stream, s);
    case 256: return launch_gemm<256, kEpiScatter>(A, W, dummy, nullptr, nullptr, nullptr, M, N, K, lda, ldw, N, 0, status, stream, s);
    default: return -2;
  }
}

// Grouped GEMM over experts (MoE): rows of A are sorted by expert; `group_tab` holds one int4 per
// 128-row tile {expert, first row, end row, 0} and `group_mtiles` their count, both produced on the
// device by ogb_moe_permute, so no routing information crosses to the host.  W is [experts, N, K].
// epilogue 0 = plain, 2 = SwiGLU over per-expert packed gate|up weights (output width N/2).
extern "C" int ogb_grouped_gemm_bf16(const void* A, const void* W, void* C, const int* group_tab, const int* group_mtiles,
                                     int experts, int max_rows, int max_mtiles, int N, int K, int epilogue, int bn, int* status,
                                     void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (max_rows <= 0 || experts <= 0) return 0;
  if ((K % 8) != 0 || (N % bn) != 0) return -3;
  const int ldc = epilogue == kEpiSwiGLU ? N / 2 : N;
  if (epilogue == kEpiNone) {
    if (bn == 256) return launch_gemm<256, kEpiNone>(A, W, C, nullptr, nullptr, nullptr, max_rows, N, K, K, K, ldc, 0, status, stream, nullptr, group_tab, group_mtiles, experts, max_mtiles);
    if (bn == 128) return launch_gemm<128, kEpiNone>(A, W, C, nullptr, nullptr, nullptr, max_rows, N, K, K, K, ldc, 0, status, stream, nullptr, group_tab, group_mtiles, experts, max_mtiles);
  } else if (epilogue == kEpiSwiGLU) {
    if (bn == 256) return launch_gemm<256, kEpiSwiGLU>(A, W, C, nullptr, nullptr, nullptr, max_rows, N, K, K, K, ldc, 0, status, stream, nullptr, group_tab, group_mtiles, experts, max_mtiles);
    if (bn == 128) return launch_gemm<128, kEpiSwiGLU>(A, W, C, nullptr, nullptr, nullptr, max_rows, N, K, K, K, ldc, 0, status, stream, nullptr, group_tab, group_mtiles, experts, max_mtiles);
  }
  return -2;
}
