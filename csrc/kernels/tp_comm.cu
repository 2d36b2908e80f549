// Tensor-parallel communication over peer-mapped memory (NVLink 5 / NVSwitch), no NCCL inside.
//
// The reference has no multi-GPU execution at all: its comm crate is a trait plus an in-process
// host oracle (crates/onnx-runtime-comm/src/lib.rs:19-29, communicator.rs:32-160) and its TP
// notes are an analytic plan (docs/research/tensor-parallelism-feasibility.md:60-110).  This file
// is the product-side backend of that contract for row-parallel projections:
//
//   1. gemm_bf16_tcgen05<kEpiScatter> (gemm_tcgen05.cu) keeps its partial output in a peer-mapped
//      buffer of its own GPU and, tile by tile, bumps the arrival counter of the rank that owns
//      the rows (one remote reduction per warp tile; the tensor-core loop never waits on NVLink);
//   2. tp_reduce_bcast_kernel (here) waits per 32-row group for all sources, pulls their partial
//      rows with coalesced 512-byte peer loads (the reduce-scatter half), sums them in a fixed
//      rank order in fp32, adds the residual, and stores the new residual rows into every rank's
//      copy of the residual stream (the all-gather half), then waits until every other owner's
//      rows have landed locally.  Row groups are consumed as their counters fill, so the pull
//      overlaps the tail of slower peers' GEMMs.
// Every result row is produced by exactly one rank and copied bit-for-bit to the others, so all
// replicas stay identical.  Waits are bounded: on expiry the kernel ORs kStatusPeerTimeout into
// the status word and returns.  Counters are reset by the kernel that consumed them.
#include "common.cuh"
#include "ogb_kernels.h"
#include "tp_comm.cuh"

namespace ogb {

constexpr int kRbThreads = 256;

OGB_DEVICE uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded spin until *p >= want.  Returns false on timeout.
OGB_DEVICE bool wait_counter(const uint32_t* p, uint32_t want, uint64_t limit_ns = kWaitLimitNs) {
  if (ld_acquire_sys(p) >= want) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (ld_acquire_sys(p) < want) {
    if (((++spins) & 0xff) == 0 && global_timer_ns() - t0 > limit_ns) return false;
  }
  return true;
}

OGB_DEVICE void add_bf16x8(float (&acc)[8], const uint4& v) {
  float2 f;
  f = unpack_bf16(v.x); acc[0] += f.x; acc[1] += f.y;
  f = unpack_bf16(v.y); acc[2] += f.x; acc[3] += f.y;
  f = unpack_bf16(v.z); acc[4] += f.x; acc[5] += f.y;
  f = unpack_bf16(v.w); acc[6] += f.x; acc[7] += f.y;
}

// Tail shared by both exchange kernels: wait (bounded) until every owner's row blocks have landed in this
// rank's residual stream, then let the last CTA of the launch reset the counters it consumed.  That is
// safe: no rank can produce for the next use of this slot before it has received this rank's rows.
OGB_DEVICE void finish_reduce(const TpReduce& r, int groups, uint32_t expect_x, int* status) {
  if (threadIdx.x != 0) return;
  if (!wait_counter(r.x_cnt[r.rank], expect_x)) atomicOr(status, kStatusPeerTimeout);
  __threadfence();
  const uint32_t total_ctas = gridDim.x * gridDim.y;
  if (atomicAdd(r.done_cnt, 1u) == total_ctas - 1) {
    for (int i = 0; i < groups; ++i) r.tile_cnt[i] = 0;
    *r.x_cnt[r.rank] = 0;
    *r.done_cnt = 0;
    __threadfence_system();
  }
}

// grid = (min(owned row groups, SMs / column blocks), column blocks); CTAs stride over row groups.
// rows = total rows of the step (M); cols = columns per CTA.  TP is a template parameter so the
// loads of all sources for U vectors are issued back to back before the first add: with peer-load
// latencies of a few microseconds the kernel lives on memory-level parallelism.
template <int TP, int U>
__global__ void __launch_bounds__(kRbThreads) tp_reduce_bcast_kernel(const TpReduce* __restrict__ rp, int rows, int cols,
                                                                      uint32_t expect_x, int* status) {
  const TpReduce& r = *rp;
  const int groups = r.chunk / 32;
  const int col0 = blockIdx.y * cols;
  const int ncols = min(cols, r.n - col0);
  const int vec_per_row = ncols / 8;
  const int total = 32 * vec_per_row;
  __shared__ int ok_sh;
  const bool stamp = r.dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
  if (stamp) r.dbg[0] = global_timer_ns();
  for (int g = blockIdx.x; g < groups; g += gridDim.x) {   // g = owned 32-row group
    const int row_base = r.rank * r.chunk + g * 32;        // global row of the group
    if (row_base >= rows) break;
    __syncthreads();
    if (threadIdx.x == 0) {
      const bool ok = wait_counter(r.tile_cnt + g, static_cast<uint32_t>(r.n / 32) * TP);
      if (!ok) atomicOr(status, kStatusPeerTimeout);
      ok_sh = ok ? 1 : 0;
      if (stamp && g == 0) r.dbg[1] = global_timer_ns();
    }
    __syncthreads();
    if (ok_sh) {
      for (int i0 = threadIdx.x; i0 < total; i0 += kRbThreads * U) {
        uint4 xv[U];
        uint4 pv[U][TP];
        size_t off[U];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = i0 + u * kRbThreads;
          const int lr = i / vec_per_row, cv = i % vec_per_row;
          const int row = row_base + lr;
          live[u] = (i < total) && (row < rows);
          off[u] = static_cast<size_t>(row) * r.n + col0 + cv * 8;
          if (live[u]) {
            xv[u] = *reinterpret_cast<const uint4*>(r.x[r.rank] + off[u]);
#pragma unroll
            for (int src = 0; src < TP; ++src) pv[u][src] = *reinterpret_cast<const uint4*>(r.part[src] + off[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (!live[u]) continue;
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          add_bf16x8(acc, xv[u]);
#pragma unroll
          for (int src = 0; src < TP; ++src) add_bf16x8(acc, pv[u][src]);  // fixed order: independent of arrival order
          const uint4 o = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                                     pack_bf16(acc[6], acc[7]));
#pragma unroll
          for (int p = 0; p < TP; ++p)            // all-gather half: every replica receives the new row
            *reinterpret_cast<uint4*>(r.x[p] + off[u]) = o;
        }
      }
    }
    // publish: this block of rows is in place everywhere
    if (stamp && g == 0) r.dbg[4] = global_timer_ns();
    __syncthreads();
    if (threadIdx.x == 0) {
      if (stamp && g == 0) r.dbg[5] = global_timer_ns();
      __threadfence_system();
      if (stamp && g == 0) r.dbg[6] = global_timer_ns();
      // one fence orders the CTA's row stores before all the signals; a releasing reduction per peer would
      // each wait again for the SM's outstanding NVLink writes (measured: ~12 us apiece under load)
      for (int p = 0; p < TP; ++p) asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(r.x_cnt[p]) : "memory");
    }
  }
  if (stamp) r.dbg[2] = global_timer_ns();
  finish_reduce(r, groups, expect_x, status);
  if (stamp) r.dbg[3] = global_timer_ns();
}

// The same exchange through NVSwitch multicast (NVLS).  One multimem.ld_reduce returns the fp32-accumulated
// sum of all ranks' partial rows (the switch pulls each rank's copy: 1/TP of the bytes of TP peer loads
// arrive here), one multimem.st delivers the finished row to every rank's residual stream, and one
// multimem.red bumps every rank's delivery counter.  The owner still adds the residual and rounds once,
// so all replicas receive identical bits.
template <int U>
__global__ void __launch_bounds__(kRbThreads) tp_reduce_bcast_nvls_kernel(const TpReduce* __restrict__ rp, int rows, int cols,
                                                                           uint32_t expect_x, int* status) {
  const TpReduce& r = *rp;
  const int groups = r.chunk / 32;
  const int col0 = blockIdx.y * cols;
  const int ncols = min(cols, r.n - col0);
  const int vec_per_row = ncols / 8;
  const int total = 32 * vec_per_row;
  __shared__ int ok_sh;
  const bool stamp = r.dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
  if (stamp) r.dbg[0] = global_timer_ns();
  for (int g = blockIdx.x; g < groups; g += gridDim.x) {
    const int row_base = r.rank * r.chunk + g * 32;
    if (row_base >= rows) break;
    __syncthreads();
    if (threadIdx.x == 0) {
      const bool ok = wait_counter(r.tile_cnt + g, static_cast<uint32_t>(r.n / 32) * r.tp);
      if (!ok) atomicOr(status, kStatusPeerTimeout);
      ok_sh = ok ? 1 : 0;
      if (stamp && g == 0) r.dbg[1] = global_timer_ns();
    }
    __syncthreads();
    if (ok_sh) {
      for (int i0 = threadIdx.x; i0 < total; i0 += kRbThreads * U) {
        uint4 xv[U], sv[U];
        size_t off[U];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = i0 + u * kRbThreads;
          const int lr = i / vec_per_row, cv = i % vec_per_row;
          const int row = row_base + lr;
          live[u] = (i < total) && (row < rows);
          off[u] = static_cast<size_t>(row) * r.n + col0 + cv * 8;
          if (live[u]) {
            xv[u] = *reinterpret_cast<const uint4*>(r.x[r.rank] + off[u]);
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(sv[u].x), "=r"(sv[u].y), "=r"(sv[u].z), "=r"(sv[u].w)
                         : "l"(r.part_mc + off[u])
                         : "memory");
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (!live[u]) continue;
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          add_bf16x8(acc, xv[u]);
          add_bf16x8(acc, sv[u]);
          const uint32_t o0 = pack_bf16(acc[0], acc[1]), o1 = pack_bf16(acc[2], acc[3]), o2 = pack_bf16(acc[4], acc[5]),
                         o3 = pack_bf16(acc[6], acc[7]);
          asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(r.x_mc + off[u]),
                       "f"(__uint_as_float(o0)), "f"(__uint_as_float(o1)), "f"(__uint_as_float(o2)), "f"(__uint_as_float(o3))
                       : "memory");
        }
      }
    }
    if (stamp && g == 0) r.dbg[4] = global_timer_ns();
    __syncthreads();
    if (threadIdx.x == 0) {
      if (stamp && g == 0) r.dbg[5] = global_timer_ns();
      __threadfence_system();
      if (stamp && g == 0) r.dbg[6] = global_timer_ns();
      asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(r.x_cnt_mc), "r"(1u) : "memory");
    }
  }
  if (stamp) r.dbg[2] = global_timer_ns();
  finish_reduce(r, groups, expect_x, status);
  if (stamp) r.dbg[3] = global_timer_ns();
}

// ------------------------------------------------------------------------------------------------------
// Row-sharded residual: reduce-scatter + residual add + RMSNorm + all-gather of the normed rows, one kernel.
//
// One CTA pass = 8 owned rows, one warp per row (the whole row lives in the warp's registers, so the norm needs no
// shared memory).  Per row: the partial products of all ranks are summed (one multimem.ld_reduce per 16 bytes, or
// TP peer loads added in rank order), the owner's residual row is added and stored back locally (bf16), the
// statistics are taken from the rounded values exactly as the stand-alone RMSNorm does, and the normed row goes
// to every rank's h (multimem.st, or TP peer stores).  After a pass one thread fences and bumps the ready counter
// of the rows' 128-row tile on every rank; the next GEMM's TMA producer waits on that counter tile by tile, so
// nothing here waits for other owners and there is no stand-alone norm launch.
// Counters are cleared by whoever consumed them: tile_cnt[g] (arrivals from the scatter epilogues) by the last of
// the group's passes to get through its wait, the ready counters by the last CTA of the GEMM that waited on them.
// ------------------------------------------------------------------------------------------------------
// PUSHED: the partials were stored into this rank's buffer by their producers ([source][chunk][n], see TpScatter::push),
// so the reduction reads tp local slabs; otherwise it pulls (multimem.ld_reduce when NVLS, peer loads when not).
template <bool NVLS, int TP, int VPL, bool PUSHED>
__global__ void __launch_bounds__(kRbThreads) tp_exchange_norm_kernel(const TpReduce* __restrict__ rp,
                                                                       const __nv_bfloat16* __restrict__ norm_w, float eps,
                                                                       int rows, int* status) {
  const TpReduce& r = *rp;
  const uint64_t limit = r.wait_limit_ns ? r.wait_limit_ns : kWaitLimitNs;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = r.n;
  const int nvec = n / 8;
  const int own_rows = max(0, min(r.chunk, rows - r.rank * r.chunk));
  const int passes = (own_rows + kTpNormRows - 1) / kTpNormRows;
  __shared__ int ok_sh;
  const bool stamp = r.dbg != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
  if (stamp) r.dbg[0] = global_timer_ns();
  pdl_trigger();      // the GEMM that consumes h may start now: it waits per M-tile on the ready counters
  for (int ps = blockIdx.x; ps < passes; ps += gridDim.x) {
    const int local0 = ps * kTpNormRows;                  // first row of the pass, relative to the owned chunk
    const int row_base = r.rank * r.chunk + local0;
    const int g = local0 / 32;                            // 32-row group whose arrival counter covers these rows
    __syncthreads();
    if (threadIdx.x == 0) {
      const bool ok = wait_counter(r.tile_cnt + g, static_cast<uint32_t>(n / 32) * r.tp, limit);   // every rank's tiles of the group
      if (!ok) atomicOr(status, kStatusPeerTimeout);
      ok_sh = ok ? 1 : 0;
      if (ok) {
        // the last pass of the group to get here clears the arrival counter for the slot's next use
        const int group_rows = min(32, own_rows - g * 32);
        const uint32_t group_passes = static_cast<uint32_t>((group_rows + kTpNormRows - 1) / kTpNormRows);
        if (atomicAdd(r.group_done + g, 1u) == group_passes - 1) {
          r.group_done[g] = 0;
          r.tile_cnt[g] = 0;
        }
      }
      if (stamp && ps == 0) r.dbg[1] = global_timer_ns();
    }
    __syncthreads();
    const int row = row_base + warp;
    if (ok_sh && warp < kTpNormRows && local0 + warp < own_rows) {
      const size_t row_off = static_cast<size_t>(row) * n;
      uint4 xv[VPL], pv[VPL];
      if constexpr (NVLS && !PUSHED) {
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          const int v = lane + 32 * j;
          if (v < nvec) {
            xv[j] = *reinterpret_cast<const uint4*>(r.x_own + row_off + v * 8);
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(pv[j].x), "=r"(pv[j].y), "=r"(pv[j].z), "=r"(pv[j].w)
                         : "l"(r.part_mc + row_off + v * 8)
                         : "memory");
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          const int v = lane + 32 * j;
          if (v < nvec) xv[j] = *reinterpret_cast<const uint4*>(r.x_own + row_off + v * 8);
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int v = lane + 32 * j;
        if (v < nvec) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          add_bf16x8(acc, xv[j]);
          if constexpr (PUSHED) {
            // slab s = what rank s produced for this rank's rows, already in local memory
            const __nv_bfloat16* base = r.part[r.rank] + (static_cast<size_t>(local0 + warp)) * n + v * 8;
            uint4 src[TP];
#pragma unroll
            for (int s = 0; s < TP; ++s) src[s] = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(s) * r.chunk * n);
#pragma unroll
            for (int s = 0; s < TP; ++s) add_bf16x8(acc, src[s]);      // fixed order: independent of arrival order
          } else if constexpr (NVLS) {
            add_bf16x8(acc, pv[j]);
          } else {
            uint4 src[TP];
#pragma unroll
            for (int s = 0; s < TP; ++s) src[s] = *reinterpret_cast<const uint4*>(r.part[s] + row_off + v * 8);
#pragma unroll
            for (int s = 0; s < TP; ++s) add_bf16x8(acc, src[s]);      // fixed order: independent of arrival order
          }
          // the residual stream is stored in bf16: round first so the statistics see the stored value
          const uint4 o = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                                     pack_bf16(acc[6], acc[7]));
          *reinterpret_cast<uint4*>(r.x_own + row_off + v * 8) = o;
          xv[j] = o;
          float2 f;
          f = unpack_bf16(o.x); ss += f.x * f.x + f.y * f.y;
          f = unpack_bf16(o.y); ss += f.x * f.x + f.y * f.y;
          f = unpack_bf16(o.z); ss += f.x * f.x + f.y * f.y;
          f = unpack_bf16(o.w); ss += f.x * f.x + f.y * f.y;
        }
      }
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / static_cast<float>(n) + eps);
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int v = lane + 32 * j;
        if (v < nvec) {
          const uint4 wv = __ldg(reinterpret_cast<const uint4*>(norm_w) + v);
          float2 a, w;
          uint4 hv;
          a = unpack_bf16(xv[j].x); w = unpack_bf16(wv.x); hv.x = pack_bf16(a.x * inv * w.x, a.y * inv * w.y);
          a = unpack_bf16(xv[j].y); w = unpack_bf16(wv.y); hv.y = pack_bf16(a.x * inv * w.x, a.y * inv * w.y);
          a = unpack_bf16(xv[j].z); w = unpack_bf16(wv.z); hv.z = pack_bf16(a.x * inv * w.x, a.y * inv * w.y);
          a = unpack_bf16(xv[j].w); w = unpack_bf16(wv.w); hv.w = pack_bf16(a.x * inv * w.x, a.y * inv * w.y);
          if constexpr (NVLS) {
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(r.h_mc + row_off + v * 8),
                         "f"(__uint_as_float(hv.x)), "f"(__uint_as_float(hv.y)), "f"(__uint_as_float(hv.z)),
                         "f"(__uint_as_float(hv.w))
                         : "memory");
          } else {
#pragma unroll
            for (int p = 0; p < TP; ++p) *reinterpret_cast<uint4*>(r.h[p] + row_off + v * 8) = hv;
          }
        }
      }
    }
    if (stamp && ps == 0) r.dbg[4] = global_timer_ns();
    __syncthreads();
    if (threadIdx.x == 0 && ok_sh) {
      __threadfence_system();
      if (stamp && ps == 0) r.dbg[6] = global_timer_ns();
      const int tile = row_base / 128;
      if constexpr (NVLS) {
        asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(r.h_ready_mc + tile), "r"(1u) : "memory");
      } else {
#pragma unroll
        for (int p = 0; p < TP; ++p) asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(r.h_ready[p] + tile) : "memory");
      }
    }
  }
  if (stamp) r.dbg[3] = global_timer_ns();
}

// Waits (bounded) until every 128-row tile of the slot's normed activation has arrived on this rank: the kernels
// that follow on the stream and read h without a wait of their own (the gather of the rows that sample) are
// ordered after it.
__global__ void tp_wait_ready_kernel(const TpReduce* __restrict__ rp, int rows, int* status) {
  const TpReduce& r = *rp;
  const uint64_t limit = r.wait_limit_ns ? r.wait_limit_ns : kWaitLimitNs;
  const int tiles = (rows + 127) / 128;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const int valid = min(128, rows - t * 128);
    const uint32_t want = static_cast<uint32_t>((valid + kTpNormRows - 1) / kTpNormRows);
    if (!wait_counter(r.h_ready[r.rank] + t, want, limit)) atomicOr(status, kStatusPeerTimeout);
  }
  __syncthreads();
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) r.h_ready[r.rank][t] = 0;     // consumed: clear for the slot's next use
}

// Marks every 32-row group of this rank's staged partial product as complete on the rank that owns it.  Used
// when the partial was produced by kernels that do not signal themselves (the MoE combine): the kernel
// boundary has made the rows visible, one releasing reduction per group publishes them.
__global__ void tp_signal_rows_kernel(const TpScatter* __restrict__ scp, int rows) {
  const TpScatter& sc = *scp;
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  const int row0 = g * 32;
  if (row0 >= rows) return;
  const int owner = row0 / sc.chunk;
  uint32_t* cnt = sc.tile_cnt[owner] + (row0 - owner * sc.chunk) / 32;
  const uint32_t units = static_cast<uint32_t>(sc.n / 32);
  __threadfence_system();
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(units) : "memory");
}

// Copies rows [0, rows) of a local partial-sum matrix [rows, n] into the buffers of the ranks that own them (slab of
// this rank, see TpScatter::push) and bumps the owners' arrival counters.  One CTA per 32-row group, so the CTA's
// stores and its single releasing signal belong to one owner.
__global__ void __launch_bounds__(256) tp_push_rows_kernel(const TpScatter* __restrict__ scp, const __nv_bfloat16* __restrict__ src,
                                                           int rows) {
  const TpScatter& sc = *scp;
  const int row0 = blockIdx.x * 32;
  if (row0 >= rows) return;
  const int owner = row0 / sc.chunk;
  const int nvec = sc.n / 8;
  const int last = min(32, rows - row0);
  __nv_bfloat16* dst = sc.staging[owner] + (static_cast<size_t>(sc.rank) * sc.chunk + (row0 - owner * sc.chunk)) * sc.n;
  for (int i = threadIdx.x; i < last * nvec; i += blockDim.x) {
    const int rr = i / nvec, v = i % nvec;
    reinterpret_cast<uint4*>(dst + static_cast<size_t>(rr) * sc.n)[v] =
        reinterpret_cast<const uint4*>(src + static_cast<size_t>(row0 + rr) * sc.n)[v];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* cnt = sc.tile_cnt[owner] + (row0 - owner * sc.chunk) / 32;
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(static_cast<uint32_t>(sc.n / 32)) : "memory");
  }
}

}  // namespace ogb

using namespace ogb;

extern "C" int ogb_tp_push_rows(const void* sc, const void* src, int rows, void* stream) {
  if (rows <= 0) return 0;
  tp_push_rows_kernel<<<(rows + 31) / 32, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const TpScatter*>(sc), static_cast<const __nv_bfloat16*>(src), rows);
  return static_cast<int>(cudaGetLastError());
}

// Publishes rows [0, rows) of the local staging buffer described by `sc` (a device TpScatter) to their owners;
// ogb_tp_reduce_bcast on the same stream then folds all ranks' partials into the residual stream.
extern "C" int ogb_tp_signal_rows(const void* sc, int rows, void* stream) {
  if (rows <= 0) return 0;
  const int groups = (rows + 31) / 32;
  tp_signal_rows_kernel<<<(groups + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const TpScatter*>(sc), rows);
  return static_cast<int>(cudaGetLastError());
}

namespace {
// CTAs of `kernel` that fit on the device at once (every CTA of an exchange launch spins at the end, so
// the grid must be co-resident).  Queried once per kernel.
template <typename K>
int resident_ctas(K kernel, int* cache) {
  if (*cache == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kRbThreads, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    *cache = per_sm * ogb_num_sms();
  }
  return *cache;
}

template <typename K>
int launch_exchange(K kernel, int* occ_cache, const TpReduce* r, int rows, int n, int chunk, int cols, int* status,
                    cudaStream_t st) {
  const int groups = chunk / 32;
  const int col_blocks = (n + cols - 1) / cols;
  // blocks that will signal = row groups (over all ranks) that hold at least one valid row
  const int total_groups = (rows + 31) / 32;
  const uint32_t expect_x = static_cast<uint32_t>(total_groups) * col_blocks;
  int gx = resident_ctas(kernel, occ_cache) / col_blocks;
  if (gx < 1) return -4;
  if (gx > groups) gx = groups;
  kernel<<<dim3(gx, col_blocks), kRbThreads, 0, st>>>(r, rows, cols, expect_x, status);
  return static_cast<int>(cudaGetLastError());
}
}  // namespace

// x (every rank's residual stream) += sum over ranks of the staged partial tiles; `rp` is a
// device-resident TpReduce for the slot.  Must follow ogb_gemm_bf16_scatter on the same stream.
// nvls != 0 selects the NVSwitch-multicast kernel and requires the *_mc members of `rp` to be set.
extern "C" int ogb_tp_reduce_bcast(const void* rp, int rows, int n, int chunk, int tp, int nvls, int* status, void* stream) {
  if (rows <= 0) return 0;
  if (n % 8 || chunk % 32 || chunk / 32 > kTpMaxGroups) return -3;
  const TpReduce* r = static_cast<const TpReduce*>(rp);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Peer round trips cost microseconds, so the exchange is latency-bound: column blocks are sized so that
  // every thread issues all of its loads in one batch (256 threads x U vectors = 32 rows x cols) and the
  // grid covers all owned row groups at once whenever they fit on the device.
  static int occ[5] = {0, 0, 0, 0, 0};
  if (nvls) {
    if (tp == 8) return launch_exchange(tp_reduce_bcast_nvls_kernel<2>, &occ[0], r, rows, n, chunk, 128, status, st);
    if (tp == 2 || tp == 4) return launch_exchange(tp_reduce_bcast_nvls_kernel<4>, &occ[1], r, rows, n, chunk, 256, status, st);
    return -5;
  }
  switch (tp) {
    case 2: return launch_exchange(tp_reduce_bcast_kernel<2, 4>, &occ[2], r, rows, n, chunk, 256, status, st);
    case 4: return launch_exchange(tp_reduce_bcast_kernel<4, 4>, &occ[3], r, rows, n, chunk, 256, status, st);
    case 8: return launch_exchange(tp_reduce_bcast_kernel<8, 2>, &occ[4], r, rows, n, chunk, 128, status, st);
    default: return -5;
  }
}

// Row-sharded form of the exchange (see tp_exchange_norm_kernel): x_own[own rows] += sum over ranks of the staged
// partials, h[own rows] = RMSNorm(x_own) * norm_w on every rank, ready counters of the rows' tiles bumped everywhere.
// Must follow ogb_gemm_bf16_scatter (or ogb_tp_push_rows / ogb_tp_signal_rows) on the same stream.  pushed != 0: the
// producers stored their partials into the owners' buffers (TpScatter::push), so the sum reads local memory.
extern "C" int ogb_tp_exchange_norm(const void* rp, const void* norm_w, float eps, int rows, int n, int chunk, int tp, int nvls,
                                    int pushed, int* status, void* stream) {
  if (rows <= 0) return 0;
  if (n % 8 || n > 16 * 256 || chunk % 32 || chunk / 32 > kTpMaxGroups || rows > kTpMaxTiles * 128) return -3;
  const TpReduce* r = static_cast<const TpReduce*>(rp);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int passes = (chunk + kTpNormRows - 1) / kTpNormRows;     // upper bound: the kernel clips to the rows it owns
  int grid = passes < 1 ? 1 : passes;
  const int cap = 4 * ogb_num_sms();
  if (grid > cap) grid = cap;
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(norm_w);
  const int vpl = (n / 8 + 31) / 32;                              // 16-byte vectors per lane
#define OGB_EXCH(NV, TPN, PU)                                                                                          \
  do {                                                                                                             \
    /* with PDL the kernel starts while the scatter GEMM is still running and takes row groups as their tiles land */ \
    const bool pdl = tp_pdl_enabled() != 0;                                                                        \
    if (vpl <= 8) return static_cast<int>(launch_kernel_pdl(tp_exchange_norm_kernel<NV, TPN, 8, PU>, dim3(grid), dim3(kRbThreads), 0, st, pdl, r, w, eps, rows, status)); \
    return static_cast<int>(launch_kernel_pdl(tp_exchange_norm_kernel<NV, TPN, 16, PU>, dim3(grid), dim3(kRbThreads), 0, st, pdl, r, w, eps, rows, status)); \
  } while (0)
  if (pushed) {
    // partials already local: the template's TP is the number of slabs; NVLS only selects how h and the counters go out
    if (nvls) {
      switch (tp) {
        case 2: OGB_EXCH(true, 2, true);
        case 4: OGB_EXCH(true, 4, true);
        case 8: OGB_EXCH(true, 8, true);
        default: return -5;
      }
    }
    switch (tp) {
      case 2: OGB_EXCH(false, 2, true);
      case 4: OGB_EXCH(false, 4, true);
      case 8: OGB_EXCH(false, 8, true);
      default: return -5;
    }
  }
  if (nvls) {
    if (tp == 2 || tp == 4 || tp == 8) OGB_EXCH(true, 1, false);
    return -5;
  }
  switch (tp) {
    case 2: OGB_EXCH(false, 2, false);
    case 4: OGB_EXCH(false, 4, false);
    case 8: OGB_EXCH(false, 8, false);
    default: return -5;
  }
#undef OGB_EXCH
}

static int g_tp_pdl = -1;
int ogb::tp_pdl_enabled() {
  if (g_tp_pdl < 0) {
    const char* e = getenv("OGB_TP_PDL");
    g_tp_pdl = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return g_tp_pdl;
}
// Programmatic dependent launch between the scatter GEMM, the exchange kernel and the consuming GEMM: 1 / 0 sets it, the
// old value is returned.
extern "C" int ogb_tp_set_pdl(int on) {
  const int old = ogb::tp_pdl_enabled();
  g_tp_pdl = on ? 1 : 0;
  return old;
}

extern "C" int ogb_tp_wait_ready(const void* rp, int rows, int* status, void* stream) {
  if (rows <= 0) return 0;
  tp_wait_ready_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const TpReduce*>(rp), rows, status);
  return static_cast<int>(cudaGetLastError());
}

// ---- peer mapping helpers (CUDA IPC) ----
extern "C" int ogb_ipc_alloc(void** ptr, uint64_t bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*ptr, 0, bytes));
}
extern "C" int ogb_ipc_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }
extern "C" int ogb_ipc_get_handle(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int ogb_ipc_open_handle(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int ogb_ipc_close_handle(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }
extern "C" int ogb_tp_struct_sizes(int* scatter_bytes, int* reduce_bytes) {
  *scatter_bytes = static_cast<int>(sizeof(TpScatter));
  *reduce_bytes = static_cast<int>(sizeof(TpReduce));
  return 0;
}
