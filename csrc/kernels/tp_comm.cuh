// Device-visible description of a tensor-parallel group whose ranks have mapped each other's
// buffers (CUDA IPC over NVLink).  Shared by the GEMM scatter epilogue and the reduce+broadcast
// kernel.  All cross-GPU traffic is plain loads/stores and release/acquire counters on these
// mappings; nothing here issues TMA against peer memory.
#pragma once
#include <stdint.h>
#include <cuda_bf16.h>

namespace ogb {

constexpr int kMaxTp = 8;
constexpr int kTpSlots = 2;          // slot 0: o_proj, slot 1: down_proj (separate staging + counters)
constexpr int kTpMaxGroups = 256;    // 32-row groups one rank can own (8192 rows)

struct TpScatter {
  __nv_bfloat16* staging[kMaxTp];    // rank p's partial-product buffer for this slot
  uint32_t* tile_cnt[kMaxTp];        // rank p's arrival counters for this slot, one per owned 32-row group
  int rank, tp, chunk, n;            // chunk = rows owned per rank (multiple of 32)
  // push = 0: the partial stays in this rank's own buffer, indexed by global row ([rows][n]); the owner pulls it.
  // push = 1: the partial is stored straight into the OWNER's buffer over NVLink, laid out [source rank][chunk][n]
  //           (row = source * chunk + row within the owner's chunk); the owner then sums tp local slabs.
  int push, pad0, pad1, pad2;
};

struct TpReduce {
  const __nv_bfloat16* part[kMaxTp]; // every rank's partial-product buffer for the slot (peer-mapped, read here)
  uint32_t* tile_cnt;                // this rank's arrival counters for the slot
  __nv_bfloat16* x[kMaxTp];          // every rank's residual stream [rows, n]
  uint32_t* x_cnt[kMaxTp];           // every rank's "row blocks delivered" counter
  uint32_t* done_cnt;                // local: CTAs of this launch that have finished
  // NVSwitch multicast views of the same symmetric region (null when the region has no multicast
  // binding): a load through part_mc returns the sum over all ranks' buffers, a store through x_mc or
  // a reduction through x_cnt_mc lands in every rank's copy.
  const __nv_bfloat16* part_mc;
  __nv_bfloat16* x_mc;
  uint32_t* x_cnt_mc;
  unsigned long long* dbg;           // optional: 8 globaltimer stamps of CTA (0,0): start, group 0 ready, all rows signalled, end,
                                     // then for group 0: own stores issued, CTA stores issued, fence done
  int rank, tp, chunk, n;
  // ---- row-sharded residual (tp_exchange_norm_kernel) ----
  // The residual stream is owned by rows: rank r keeps rows [r*chunk, (r+1)*chunk) in x_own (a local buffer indexed
  // by global row) and nobody else reads them.  What is replicated is the *normed* activation h, the A operand of
  // the next column-parallel GEMM: the owner stores its normed rows into every rank's h and bumps, on every rank,
  // the ready counter of the 128-row tile they belong to (one arrival per 8 rows).
  __nv_bfloat16* x_own;              // local residual rows [rows, n]
  __nv_bfloat16* h[kMaxTp];          // every rank's normed-activation buffer [rows, n]
  __nv_bfloat16* h_mc;               // multicast view of the same (null without a multicast binding)
  uint32_t* h_ready[kMaxTp];         // every rank's per-128-row-tile ready counters of this slot
  uint32_t* h_ready_mc;              // multicast view
  uint32_t* group_done;              // local: per 32-row group, CTAs that have passed the arrival wait (the last one resets tile_cnt)
  unsigned long long wait_limit_ns;  // bound of every wait on a peer's signal; 0 = the library default
};

constexpr int kTpMaxTiles = 64;      // 128-row tiles of a step (8192 rows)
constexpr int kTpNormRows = 8;       // rows per CTA pass of the exchange = rows per arrival on a ready counter

}  // namespace ogb
