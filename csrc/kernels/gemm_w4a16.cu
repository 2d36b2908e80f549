// Weight-only int4 GEMM on the 5th-generation tensor cores: C[M, N] = A[M, K] (bf16) x dequant(W)[N, K]^T (+ bias), W in
// the MatMulNBits layout (block 32: 16 bytes of nibbles per block, one scale per block, optional packed 4-bit zero
// points).  The weights cross HBM as int4 and never exist in bf16 outside shared memory:
//
//   warp 0        TMA producer: the A tile(s) of each k-block (128-byte swizzle) into the stage ring
//   warp 1        MMA issuer and TMEM owner: tcgen05.mma kind::f16, fp32 accumulators in TMEM, double-buffered
//   warps 2..5    epilogue: tcgen05.ld -> (+ bias) -> bf16 -> staged in shared memory -> coalesced 16-byte stores
//   warps 6..13   dequantisers, two groups of four warps that take alternate k-blocks (a k-block's chain of loads ready ->
//                 nibbles to bf16 -> stores -> proxy fence -> arrival is latency-bound for one warp, so two run side by
//                 side on different ring slots).  A thread owns two 32-weight blocks of its group's k-block (128 rows x
//                 64 k): their 16 bytes of nibbles, scale and zero point sit in a register ring loaded four of the group's
//                 k-blocks ahead; nibble -> bf16 through the 0x4300 mantissa trick (128 + n, exact), minus (128 + zero
//                 point), times the scale as bf16x2, stored in the same swizzled K-major layout a TMA load of a bf16 tile
//                 would have produced, then a proxy fence and one arrival per warp on the slot's barrier
//
// (A variant that brought the packed nibbles in by TMA -- 128 rows x 32 bytes per k-block, unswizzled, into a ring of
// its own -- was 10 % faster and produced, in repeated runs, rare stale rows of B; the cause was not found, so the
// nibbles stay on plain loads.)
//
// A work item is MT 128-row tiles of A against one 128-column tile of W, so with MT = 2 (M > 128) one dequantised B
// tile feeds two accumulators and the ALU work per MMA halves.  It is the counterpart of the reference's Marlin-style kernel
// (crates/onnx-runtime-ep-cuda/src/kernels/marlin_gemm.rs: int4 tiles dequantised in registers in front of mma.sync).
#include <cuda.h>
#include <cuda_bf16.h>

#include "attention_common.cuh"
#include "common.cuh"
#include "ogb_kernels.h"

namespace ogb {

constexpr int kWTile = 128;                 // rows of an A tile, columns of a W tile
constexpr int kWBK = 64;                    // k per stage: one 128-byte swizzle row of bf16
constexpr int kWDequantWarps = 8;
constexpr int kWThreads = (2 + 4 + kWDequantWarps) * 32;
constexpr int kWGroups = 2;                 // dequantiser groups working on alternate k-blocks
constexpr int kWGroupWarps = kWDequantWarps / kWGroups;
constexpr int kWUnitRows = 64;              // rows of a W tile covered by one unit per thread of a group (128 threads x 2 halves of k)
constexpr int kWStagePitch = 272;           // epilogue staging: 128 bf16 + 16 bytes, conflict-free for 16-byte accesses
constexpr int kWStageWarpBytes = 32 * kWStagePitch;

// MT: A tiles (128 rows each) per W tile; TN: columns of a W tile (128, or 64 when 128-wide tiles would leave most SMs idle).
template <int MT, int TN>
struct W4Cfg {
  static constexpr int kStageA = MT * kWTile * kWBK * 2;
  static constexpr int kStageB = TN * kWBK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = MT == 2 ? 4 : 6;
  static constexpr int kAccCols = MT * TN;              // TMEM columns of one accumulator set
  static constexpr int kTmemCols = 2 * kAccCols;        // 128, 256 or 512: a power of two
  static constexpr int kBarOff = kStages * kStage;                      // barriers (512 bytes)
  static constexpr int kStagingOff = kBarOff + 512;
  static constexpr int kSmemBytes = kStagingOff + 4 * kWStageWarpBytes;
};

// 8 nibbles of `w` (k order: low nibble of byte 0 first) -> 4 bf16x2 words in k order, each (nibble - zero) * scale.
// prmt lines the nibbles up so that one mask yields the two neighbours of a pair in the two 16-bit halves.
OGB_DEVICE void dequant_word(uint32_t w, __nv_bfloat162 zz, __nv_bfloat162 ss, uint32_t (&out)[4]) {
  const uint32_t w4 = w >> 4;
  uint32_t x, y;
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(x) : "r"(w), "r"(w4));   // bytes (n0 n1) (n2 n3) | (n1 n2) (n3 n4)
  asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(y) : "r"(w), "r"(w4));   // bytes (n4 n5) (n6 n7) | (n5 n6) (n7 0)
  const uint32_t p[4] = {(x & 0x000F000Fu) | 0x43004300u, ((x >> 8) & 0x000F000Fu) | 0x43004300u,
                         (y & 0x000F000Fu) | 0x43004300u, ((y >> 8) & 0x000F000Fu) | 0x43004300u};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<const __nv_bfloat162*>(&p[i]), zz), ss);   // the subtraction is exact
    out[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
}

// What a dequantiser keeps per block between the load and its use.  The scale and the zero point stay as loaded (raw
// bits): converting them at load time would make the thread wait for the load right there and serialise the ring.
struct W4Unit {
  uint4 q;             // the block's 32 nibbles
  uint32_t s_raw;      // fp32 bits, or bf16 bits in the low half
  uint32_t z_raw;      // the byte that holds the zero-point nibble, or 0x88 (zero point 8)
  bool valid;          // false: a row past N or a block past K -- the loads went to a clamped address, the result is zero
};

template <int MT, bool SF32, int TN>
__global__ void __launch_bounds__(kWThreads, 1)
gemm_w4a16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const uint8_t* __restrict__ qw, const void* __restrict__ scales,
                          const uint8_t* __restrict__ zp, const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ C,
                          int M, int N, int K, int ldc, int* status) {
  using Cfg = W4Cfg<MT, TN>;
  constexpr int kUnits = TN / kWUnitRows;     // 32-weight blocks per dequantiser thread per k-block
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);
  uint8_t* staging = smem + Cfg::kStagingOff;
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kStages;
  uint64_t* tmem_full = bars + 2 * Cfg::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (M + MT * kWTile - 1) / (MT * kWTile);
  const int n_tiles = (N + TN - 1) / TN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + kWBK - 1) / kWBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&full_bar[i], 1 + kWGroupWarps);     // the producer's arrive.expect_tx + one arrival per warp of the group that fills it
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
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
    // ------------------------------ TMA producer (A) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * (MT * kWTile);
        const int mt_here = (MT == 2 && m0 + kWTile < M) ? 2 : 1;     // a second tile wholly past M is neither loaded nor multiplied
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStage;
          mbar_expect_tx(&full_bar[stage], static_cast<uint32_t>(mt_here * kWTile * kWBK * 2));
          for (int mi = 0; mi < mt_here; ++mi)
            tma_load_2d(sa + mi * (kWTile * kWBK * 2), &tmap_a, &full_bar[stage], kb * kWBK, m0 + mi * kWTile);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { atomicOr(status, kStatusWaitTimeout); *abort_flag = 1; }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kWTile, TN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
        const int m0 = (tile % m_tiles) * (MT * kWTile);
        const int mt_here = (MT == 2 && m0 + kWTile < M) ? 2 : 1;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_addr = tmem_base + acc * Cfg::kAccCols;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStage);
          const uint64_t db = make_kmajor_sw128_desc(sa + Cfg::kStageA);
          for (int mi = 0; mi < mt_here; ++mi) {
            const uint64_t da = make_kmajor_sw128_desc(sa + mi * (kWTile * kWBK * 2));
#pragma unroll
            for (int k = 0; k < kWBK / 16; ++k)
              umma_f16(d_addr + mi * TN, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
    uint8_t* stg = staging + (warp - 2) * kWStageWarpBytes;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int m0 = (tile % m_tiles) * (MT * kWTile);
      const int mt_here = (MT == 2 && m0 + kWTile < M) ? 2 : 1;
      const int n0 = (tile / m_tiles) * TN;
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_phase))) { ok = false; break; }
      tc_fence_after();
      for (int mi = 0; mi < mt_here; ++mi) {
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * Cfg::kAccCols + mi * TN;
        const int row0 = m0 + mi * kWTile + q * 32;
        // phase 1 (thread = row): TMEM -> registers -> + bias -> bf16 into this warp's staging slab
#pragma unroll 1
        for (int c = 0; c < TN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < N) r[j] = __float_as_uint(__uint_as_float(r[j]) + __bfloat162float(__ldg(bias + col + j)));
          }
          uint4* srow = reinterpret_cast<uint4*>(stg + lane * kWStagePitch + c * 64);
#pragma unroll
          for (int v = 0; v < 4; ++v)
            srow[v] = make_uint4(pack_bf16(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1])),
                                 pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                 pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                 pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
        }
        __syncwarp();
        // phase 2 (16 lanes along a row): two rows per pass, 256-byte row segments per warp instruction
        const int ch = lane & 15;
        const int gcol = n0 + ch * 8;
#pragma unroll 4
        for (int rb = 0; rb < 32; rb += 2) {
          const int r_loc = rb + (lane >> 4);
          const int grow = row0 + r_loc;
          if (grow < M && gcol < N && ch * 8 < TN) {
            const uint4 v = *reinterpret_cast<const uint4*>(stg + r_loc * kWStagePitch + ch * 16);
            __nv_bfloat16* dst = C + static_cast<size_t>(grow) * ldc + gcol;
            if (gcol + 8 <= N) {
              *reinterpret_cast<uint4*>(dst) = v;
            } else {
              const __nv_bfloat16* pv = reinterpret_cast<const __nv_bfloat16*>(&v);
              for (int j = 0; j < 8 && gcol + j < N; ++j) dst[j] = pv[j];
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
    if (!ok && lane == 0) { atomicOr(status, kStatusWaitTimeout); *abort_flag = 1; }
  } else {
    // ------------------------------ dequantisers (B) ------------------------------
    // Group g takes k-blocks g, g + 2, ...; a thread owns two 32-weight blocks of such a k-block: rows r and r + 64, the
    // same half.
    const int group = (warp - 6) / kWGroupWarps;
    const int t = ((warp - 6) % kWGroupWarps) * 32 + lane;   // 0..127 within the group
    const int half = t & 1;                                   // which 32-k block of the 64 k
    const int kb32 = (K + 31) / 32;
    const int zp_stride = (kb32 + 1) / 2;
    const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const long long iters = static_cast<long long>(my_tiles) * k_blocks;
    // The loads run kDepth of the group's k-blocks ahead of their use, in a register ring (each takes a trip to L2 or
    // DRAM): 128 threads x kDepth x 2 blocks x 16 bytes per group in flight.
    constexpr int kDepth = 4;                // a deeper ring (8) for the one-unit form measured no different
    struct Cursor {
      int tile, kb;
      size_t row_blk[kUnits];   // index of each row's first block
      size_t row_zp[kUnits];
      bool row_ok[kUnits];
    };
    auto seat = [&](Cursor& c) {               // derive the row data of c.tile
#pragma unroll
      for (int i = 0; i < kUnits; ++i) {
        const int n = c.tile < num_tiles ? (c.tile / m_tiles) * TN + (t >> 1) + i * kWUnitRows : N;
        c.row_ok[i] = n < N;
        c.row_blk[i] = static_cast<size_t>(c.row_ok[i] ? n : 0) * kb32;
        c.row_zp[i] = static_cast<size_t>(c.row_ok[i] ? n : 0) * zp_stride;
      }
    };
    auto fetch = [&](Cursor& c, W4Unit (&un)[kUnits]) {
      // The loads are unconditional (an out-of-range unit reads block 0, which always exists, and is zeroed through
      // its scale at use): a load under a data-dependent condition tends to become load + select, and the select
      // would wait for the load here instead of several iterations later.
      const int b = c.kb * 2 + half;
#pragma unroll
      for (int i = 0; i < kUnits; ++i) {
        un[i].valid = c.row_ok[i] && b < kb32;
        const size_t blk = un[i].valid ? c.row_blk[i] + b : 0;
        un[i].q = __ldg(reinterpret_cast<const uint4*>(qw) + blk);
        if constexpr (SF32) un[i].s_raw = __float_as_uint(__ldg(static_cast<const float*>(scales) + blk));
        else un[i].s_raw = __ldg(static_cast<const unsigned short*>(scales) + blk);
        un[i].z_raw = 0x88u;
        if (zp != nullptr) un[i].z_raw = __ldg(zp + (un[i].valid ? c.row_zp[i] + (b >> 1) : 0));
      }
      c.kb += kWGroups;                          // the group's next k-block
      while (c.kb >= k_blocks) {
        c.kb -= k_blocks;
        c.tile += gridDim.x;
        seat(c);
      }
    };
    Cursor cur{static_cast<int>(blockIdx.x), group, {}, {}, {}};
    while (cur.kb >= k_blocks) { cur.kb -= k_blocks; cur.tile += gridDim.x; }
    seat(cur);
    W4Unit ring[kDepth][kUnits];
#pragma unroll
    for (int d = 0; d < kDepth; ++d) fetch(cur, ring[d]);
    // ring positions of k-iteration j = group: the slots advance by kWGroups per step of this group
    int stage = group % Cfg::kStages;
    uint32_t phase = (group / Cfg::kStages) & 1;
    bool ok = true;
    for (long long j0 = group; ok && j0 < iters; j0 += kDepth * kWGroups) {
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        if (ok && j0 + d * kWGroups < iters) {
          if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1))) {
            ok = false;
          } else {
            tc_fence_after();              // the tensor core's reads of this slot are ordered before the stores below
#pragma unroll
            for (int i = 0; i < kUnits; ++i) {
              const int r_tile = (t >> 1) + i * kWUnitRows;
              uint8_t* sb = smem + stage * Cfg::kStage + Cfg::kStageA + static_cast<uint32_t>(r_tile) * 128u;
              const uint32_t sw = static_cast<uint32_t>(r_tile & 7);
              const W4Unit& un = ring[d][i];
              const uint32_t words[4] = {un.q.x, un.q.y, un.q.z, un.q.w};
              // this block is half `half` of its k-block: an odd block's zero point is the high nibble of its byte
              const uint32_t z = half ? (un.z_raw >> 4) & 0xFu : un.z_raw & 0xFu;
              const uint32_t zbits = 0x4300u | z;                       // bf16 128 + z, exact
              const uint32_t zz_u = zbits | (zbits << 16);
              uint32_t ss_u;
              if constexpr (SF32) {
                const __nv_bfloat162 tt = __float2bfloat162_rn(__uint_as_float(un.s_raw));
                ss_u = *reinterpret_cast<const uint32_t*>(&tt);
              } else {
                ss_u = un.s_raw | (un.s_raw << 16);
              }
              if (!un.valid) ss_u = 0u;
              const __nv_bfloat162 zz = *reinterpret_cast<const __nv_bfloat162*>(&zz_u);
              const __nv_bfloat162 ss = *reinterpret_cast<const __nv_bfloat162*>(&ss_u);
#pragma unroll
              for (int wi = 0; wi < 4; ++wi) {
                uint32_t o[4];
                dequant_word(words[wi], zz, ss, o);
                const uint32_t chunk = static_cast<uint32_t>(half * 4 + wi) ^ sw;       // 128-byte swizzle: 16-byte chunk index XOR row mod 8
                *reinterpret_cast<uint4*>(sb + chunk * 16) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
            fence_proxy_async_smem();      // the tensor core reads these bytes through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[stage]);
            fetch(cur, ring[d]);
            stage += kWGroups;
            if (stage >= Cfg::kStages) { stage -= Cfg::kStages; phase ^= 1; }
          }
        }
      }
    }
    if (!ok && lane == 0) { atomicOr(status, kStatusWaitTimeout); *abort_flag = 1; }
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
}

template <int MT, bool SF32, int TN>
static int launch_w4a16_gemm(const void* x, const void* qweight, const void* scales, const void* zp, const void* bias, void* out,
                             int M, int N, int K, int ldx, int ldc, int* status, cudaStream_t stream) {
  using Cfg = W4Cfg<MT, TN>;
  CUtensorMap ta;
  int rc = make_tmap_bf16_2d(&ta, x, M, K, ldx, kWTile, kWBK);
  if (rc != 0) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    OGB_CUDA_CHECK(cudaFuncSetAttribute(gemm_w4a16_tcgen05_kernel<MT, SF32, TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  const int tiles = ((M + MT * kWTile - 1) / (MT * kWTile)) * ((N + TN - 1) / TN);
  const int grid = tiles < ogb_num_sms() ? tiles : ogb_num_sms();
  gemm_w4a16_tcgen05_kernel<MT, SF32, TN><<<grid, kWThreads, Cfg::kSmemBytes, stream>>>(
      ta, static_cast<const uint8_t*>(qweight), scales, static_cast<const uint8_t*>(zp), static_cast<const __nv_bfloat16*>(bias),
      static_cast<__nv_bfloat16*>(out), M, N, K, ldc, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ogb

using namespace ogb;

// out[M, N] (bf16, row stride ldc) = x[M, K] (bf16, row stride ldx) * dequant(qweight)[N, K]^T (+ bias).  qweight is
// [N, K/32, 16] bytes, scales [N, K/32] fp32 (scales_f32 = 1) or bf16, zp packed nibbles [N, ceil(K/32 / 2)] or null
// (zero point 8).  K must be a multiple of 32; x and out 16-byte aligned with ldx, ldc multiples of 8.
extern "C" int ogb_w4a16_gemm(const void* x, const void* qweight, const void* scales, const void* zp, const void* bias, void* out,
                              int M, int N, int K, int ldx, int ldc, int scales_f32, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 32) != 0 || (ldx % 8) != 0 || (ldc % 8) != 0) return -3;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(qweight)) & 15) return -4;
  // 64-column W tiles when 128-column ones would occupy at most half of the SMs: the dequantisers of a CTA, not its
  // tensor core, set the pace, so twice the CTAs over half the rows each is close to twice as fast (down and o
  // projections at decode-sized M).
  const int mt = M > kWTile ? 2 : 1;
  const int tiles128 = ((M + mt * kWTile - 1) / (mt * kWTile)) * ((N + kWTile - 1) / kWTile);
  const bool narrow = 2 * tiles128 <= ogb_num_sms();
#define OGB_W4_LAUNCH(MT_, SF_, TN_) launch_w4a16_gemm<MT_, SF_, TN_>(x, qweight, scales, zp, bias, out, M, N, K, ldx, ldc, status, stream)
  if (mt == 2) {
    if (narrow) return scales_f32 ? OGB_W4_LAUNCH(2, true, 64) : OGB_W4_LAUNCH(2, false, 64);
    return scales_f32 ? OGB_W4_LAUNCH(2, true, 128) : OGB_W4_LAUNCH(2, false, 128);
  }
  if (narrow) return scales_f32 ? OGB_W4_LAUNCH(1, true, 64) : OGB_W4_LAUNCH(1, false, 64);
  return scales_f32 ? OGB_W4_LAUNCH(1, true, 128) : OGB_W4_LAUNCH(1, false, 128);
#undef OGB_W4_LAUNCH
}
