"""Fused tensor-parallel communicator: GEMM + reduce-scatter + all-gather over peer-mapped memory.

Every rank allocates one symmetric region (staging tiles for two projection slots, arrival
counters, the residual stream) with ``cudaMalloc``, exports it through CUDA IPC and maps every
peer's region.  A row-parallel projection is then two launches on each rank and no library
collective:

    ogb_gemm_bf16_scatter   tcgen05 GEMM whose epilogue keeps the partial tile in this rank's peer-mapped
                            buffer and bumps the owner rank's arrival counter over NVLink
    ogb_tp_reduce_bcast     owner pulls the sources' rows (peer loads), sums them in fixed rank order
                            + residual, stores the new rows into every rank's residual stream, waits
                            for the other owners

The decoder uses the row-sharded form of the exchange (:meth:`FusedComm.row_parallel_norm`): the residual stream is
owned by rows (rank r keeps rows ``[r*chunk, (r+1)*chunk)`` in a local buffer), and what every rank receives is the
*normed* activation ``h`` of the next column-parallel GEMM.  One kernel per projection boundary does
reduce-scatter + residual add + RMSNorm + all-gather, bumping a ready counter per 128-row tile of ``h`` on every
rank; the next GEMM's TMA producer waits on those counters tile by tile (``ops.gemm(..., a_ready=...)``), so there is
no stand-alone norm launch and no kernel that waits for the slowest owner.

When the region can be bound to an NVSwitch multicast object (the region is then allocated through
``torch.distributed._symmetric_memory``, which does the handle exchange and the binding), the second
launch uses ``multimem.ld_reduce`` / ``multimem.st`` / ``multimem.red`` instead of per-peer loads and
stores: the switch adds the partial rows and replicates the result (used from TP=4 up, where it moves
fewer bytes per GPU).  ``OGB_TP_NVLS=0`` keeps plain peer loads, ``OGB_TP_NVLS=1`` forces multicast at
TP=2; ``OGB_TP_SYMM=0`` keeps the CUDA-IPC region.

Collectives this class does not cover (broadcast of sampled tokens, barriers, scalar reductions)
go to the wrapped NCCL communicator.  The reference's counterpart is only a contract
(crates/onnx-runtime-comm/src/communicator.rs:32-160); its ordering rule -- every rank issues the
same collective in the same slot (ordering.rs:349-384) -- holds here by construction because every
rank runs the same step plan.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _native

MAX_TP = 8
SLOTS = 2
MAX_GROUPS = 256


class _Scatter(ctypes.Structure):
    _fields_ = [("staging", ctypes.c_uint64 * MAX_TP), ("tile_cnt", ctypes.c_uint64 * MAX_TP),
                ("rank", ctypes.c_int), ("tp", ctypes.c_int), ("chunk", ctypes.c_int), ("n", ctypes.c_int),
                ("push", ctypes.c_int), ("pad0", ctypes.c_int), ("pad1", ctypes.c_int), ("pad2", ctypes.c_int)]


class _Reduce(ctypes.Structure):
    _fields_ = [("part", ctypes.c_uint64 * MAX_TP), ("tile_cnt", ctypes.c_uint64), ("x", ctypes.c_uint64 * MAX_TP),
                ("x_cnt", ctypes.c_uint64 * MAX_TP), ("done_cnt", ctypes.c_uint64),
                ("part_mc", ctypes.c_uint64), ("x_mc", ctypes.c_uint64), ("x_cnt_mc", ctypes.c_uint64), ("dbg", ctypes.c_uint64),
                ("rank", ctypes.c_int), ("tp", ctypes.c_int), ("chunk", ctypes.c_int), ("n", ctypes.c_int),
                ("x_own", ctypes.c_uint64), ("h", ctypes.c_uint64 * MAX_TP), ("h_mc", ctypes.c_uint64),
                ("h_ready", ctypes.c_uint64 * MAX_TP), ("h_ready_mc", ctypes.c_uint64), ("group_done", ctypes.c_uint64),
                ("wait_limit_ns", ctypes.c_uint64)]


READY_WORDS = 80          # per slot: 64 per-tile ready counters, then the consumer GEMM's finished-CTA word


class _CudaArray:
    """Minimal __cuda_array_interface__ holder so torch can view IPC memory it did not allocate."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2}


def _lib():
    lib = _native.load()
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.ogb_ipc_alloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint64]
    lib.ogb_ipc_get_handle.argtypes = [P, P]
    lib.ogb_ipc_open_handle.argtypes = [P, ctypes.POINTER(ctypes.c_void_p)]
    lib.ogb_ipc_close_handle.argtypes = [P]
    lib.ogb_ipc_free.argtypes = [P]
    lib.ogb_tp_struct_sizes.argtypes = [ctypes.POINTER(I), ctypes.POINTER(I)]
    lib.ogb_gemm_bf16_scatter.argtypes = [P, P, I, I, I, I, I, P, I, P, P]
    lib.ogb_tp_reduce_bcast.argtypes = [P, I, I, I, I, I, P, P]
    lib.ogb_tp_signal_rows.argtypes = [P, I, P]
    lib.ogb_tp_signal_rows.restype = I
    lib.ogb_tp_exchange_norm.argtypes = [P, P, ctypes.c_float, I, I, I, I, I, I, P, P]
    lib.ogb_tp_push_rows.argtypes = [P, P, I, P]
    lib.ogb_tp_push_rows.restype = I
    lib.ogb_tp_exchange_norm.restype = I
    lib.ogb_tp_wait_ready.argtypes = [P, I, P, P]
    lib.ogb_tp_wait_ready.restype = I
    for f in ("ogb_ipc_alloc", "ogb_ipc_get_handle", "ogb_ipc_open_handle", "ogb_ipc_close_handle", "ogb_ipc_free",
              "ogb_tp_struct_sizes", "ogb_gemm_bf16_scatter", "ogb_tp_reduce_bcast"):
        getattr(lib, f).restype = I
    return lib


class FusedComm:
    backend_name = "fused-p2p"

    def __init__(self, base, device, hidden: int = 0, max_tokens: int = 0):
        self.base = base
        self.rank, self.world = base.rank, base.world
        self.device = torch.device(device)
        self.lib = _lib()
        self.ready = False
        self.failed: str | None = None     # set by poison(): why the region's counters can no longer be trusted
        self._last_slot = -1
        self.calls = 0
        if hidden and max_tokens:
            self.setup(hidden, max_tokens)

    # -- collectives delegated to the library backend ------------------------------------------
    def all_reduce(self, t):
        return self.base.all_reduce(t)

    def broadcast(self, t, src=0):
        return self.base.broadcast(t, src)

    def all_gather(self, out, t):
        return self.base.all_gather(out, t)

    def barrier(self):
        """All ranks meet with their streams drained up to here, so the next exchange may use either slot."""
        out = self.base.barrier()
        self._last_slot = -1
        return out

    def min_int(self, v):
        return self.base.min_int(v)

    def max_float(self, v):
        return self.base.max_float(v)

    # -- symmetric region ----------------------------------------------------------------------
    def _layout(self, hidden: int, max_tokens: int) -> int:
        """Offsets of the symmetric region's sections; returns its size in bytes."""
        tp = self.world
        self.hidden, self.max_tokens = hidden, max_tokens
        self.chunk_max = ((max_tokens + tp - 1) // tp + 31) // 32 * 32
        # one partial-product buffer per slot: [max_tokens, hidden] when owners pull, [tp][chunk][hidden] when producers
        # push (chunk is rounded up to 32 rows, so the pushed layout can need a little more)
        stage_bytes = max(max_tokens, tp * self.chunk_max) * hidden * 2
        align = lambda v: (v + 255) // 256 * 256
        self.off_stage = [0, align(stage_bytes)]
        self.off_x = self.off_stage[1] + align(stage_bytes)
        self.off_h = self.off_x + align(max_tokens * hidden * 2)
        self.off_cnt = self.off_h + align(max_tokens * hidden * 2)
        # counters: tile_cnt[SLOTS][MAX_GROUPS], x_cnt / done_cnt (64 words), h_ready[SLOTS][READY_WORDS],
        # group_done[SLOTS][MAX_GROUPS]
        self.cnt_words = SLOTS * MAX_GROUPS + 64 + SLOTS * READY_WORDS + SLOTS * MAX_GROUPS
        self.off_ready = self.off_cnt + (SLOTS * MAX_GROUPS + 64) * 4
        self.off_gdone = self.off_ready + SLOTS * READY_WORDS * 4
        self.wait_limit_ns = 0
        self.x_own_ptr = 0
        # OGB_TP_PUSH=0: the scatter epilogue keeps partials local and the owners pull them (multimem.ld_reduce / peer loads)
        self.push = os.environ.get("OGB_TP_PUSH", "1") != "0"
        self._partial_scratch = None
        return self.off_cnt + align(self.cnt_words * 4)

    @classmethod
    def loopback(cls, device, hidden: int, max_tokens: int, world: int = 2):
        """A group of ``world`` ranks whose regions all live on this one GPU (this process is rank 0; plain memory, no
        multicast).  Nothing real can be computed with it -- the "peers" never run -- which is its use: a launch on
        it waits for arrivals that cannot come, so the bounded waits of the exchange kernels can be exercised on one
        GPU without faulting or hanging anything (see :meth:`set_wait_limit`)."""
        self = cls.__new__(cls)

        n_ranks = world

        class _Solo:
            rank = 0
            world = n_ranks
            backend_name = "loopback"

            def barrier(self): return None
            def min_int(self, v): return v
            def max_float(self, v): return v

        self.base = _Solo()
        self.rank, self.world = 0, world
        self.device = torch.device(device)
        self.lib = _lib()
        self.failed, self._last_slot, self.calls = None, -1, 0
        total = self._layout(hidden, max_tokens)
        self.total_bytes = total
        self._region = torch.zeros(world * total, dtype=torch.uint8, device=self.device)
        self.local_ptr = self._region.data_ptr()
        self.peer_ptrs = [self.local_ptr + p * total for p in range(world)]
        self.mc_ptr, self.nvls, self._symm, self.dbg = 0, False, None, None
        self.backend_name = "loopback"
        self.x = self._region[self.off_x:self.off_x + max_tokens * hidden * 2].view(torch.bfloat16).view(max_tokens, hidden)
        self.h = self._region[self.off_h:self.off_h + max_tokens * hidden * 2].view(torch.bfloat16).view(max_tokens, hidden)
        self._structs = {}
        self.ready = True
        return self

    def reset_counters(self) -> None:
        """Zero every counter of this rank's region (after a wait ran out the counters are part-consumed)."""
        cnt = torch.as_tensor(_CudaArray(self.local_ptr + self.off_cnt, (self.cnt_words,), "<u4"), device=self.device)
        cnt.view(torch.int32).zero_()
        self._last_slot = -1

    def setup(self, hidden: int, max_tokens: int):
        """Allocate, export and map the symmetric region for a residual stream [max_tokens, hidden]."""
        sb, rb = ctypes.c_int(), ctypes.c_int()
        self.lib.ogb_tp_struct_sizes(ctypes.byref(sb), ctypes.byref(rb))
        assert sb.value == ctypes.sizeof(_Scatter) and rb.value == ctypes.sizeof(_Reduce), "struct layout mismatch"
        total = self._layout(hidden, max_tokens)
        self.total_bytes = total
        self.mc_ptr = 0
        self.nvls = False
        self._symm = None
        if os.environ.get("OGB_TP_SYMM", "1") != "0":
            try:
                self._setup_symmetric(total)
            except Exception as exc:       # no VMM handle exchange on this host: CUDA IPC still gives peer pointers
                self._symm = None
                self.symm_error = repr(exc)
        if not self.base.min_int(1 if self._symm is not None else 0):   # all ranks or none
            self._symm = None
            self.mc_ptr = 0
        if self._symm is None:
            self._setup_ipc(total)
        # Bytes per GPU and direction for a [rows, n] exchange: peer loads + stores move 2(tp-1)/tp of it, the
        # multicast path (tp+1)/tp (the switch also reads and writes the caller's own copy), so multicast pays
        # from tp = 4 up.  OGB_TP_NVLS=1 forces it at tp = 2, OGB_TP_NVLS=0 disables it.
        knob = os.environ.get("OGB_TP_NVLS", "auto")
        want_nvls = bool(self.mc_ptr) and knob != "0" and (self.world >= 4 or knob == "1")
        self.nvls = bool(self.base.min_int(1 if want_nvls else 0))
        if self.nvls:
            self.backend_name = "fused-nvls"
        self.dbg = torch.zeros(8, dtype=torch.int64, device=self.device) if os.environ.get("OGB_TP_STAMPS") else None
        self.x = torch.as_tensor(_CudaArray(self.local_ptr + self.off_x, (max_tokens, hidden), "<u2"),
                                 device=self.device).view(torch.bfloat16)
        self.h = torch.as_tensor(_CudaArray(self.local_ptr + self.off_h, (max_tokens, hidden), "<u2"),
                                 device=self.device).view(torch.bfloat16)
        self._structs: dict = {}
        torch.cuda.synchronize()
        self.base.barrier()
        self.ready = True

    def _setup_symmetric(self, total: int):
        import torch.distributed._symmetric_memory as symm_mem

        buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        hdl = symm_mem.rendezvous(buf, getattr(self.base, "group", None) or dist.group.WORLD)   # the ranks of this communicator only
        buf.zero_()
        self._symm = (buf, hdl)
        self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self.local_ptr = self.peer_ptrs[self.rank]
        assert self.local_ptr == buf.data_ptr()
        self.mc_ptr = int(hdl.multicast_ptr or 0)

    def _setup_ipc(self, total: int):
        tp = self.world
        ptr = ctypes.c_void_p()
        rc = self.lib.ogb_ipc_alloc(ctypes.byref(ptr), total)
        if rc != 0:
            raise RuntimeError(f"symmetric allocation of {total} bytes failed (cuda error {rc})")
        self.local_ptr = ptr.value
        handle = ctypes.create_string_buffer(64)
        rc = self.lib.ogb_ipc_get_handle(ptr, handle)
        if rc != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed ({rc})")
        handles = [None] * tp
        dist.all_gather_object(handles, bytes(handle.raw), group=getattr(self.base, "group", None))
        self.peer_ptrs = []
        for p in range(tp):
            if p == self.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            out = ctypes.c_void_p()
            buf = ctypes.create_string_buffer(handles[p], 64)
            rc = self.lib.ogb_ipc_open_handle(buf, ctypes.byref(out))
            if rc != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle for rank {p} failed ({rc})")
            self.peer_ptrs.append(out.value)

    def _tile_cnt(self, p, slot):
        return self.peer_ptrs[p] + self.off_cnt + slot * MAX_GROUPS * 4

    def _x_cnt(self, p):
        return self.peer_ptrs[p] + self.off_cnt + SLOTS * MAX_GROUPS * 4

    def _get_structs(self, slot: int, chunk: int, push: bool = False):
        key = (slot, chunk, bool(push))
        hit = self._structs.get(key)
        if hit is not None:
            return hit
        tp = self.world
        sc, rd = _Scatter(), _Reduce()
        for p in range(tp):
            sc.staging[p] = self.peer_ptrs[p] + self.off_stage[slot]
            sc.tile_cnt[p] = self._tile_cnt(p, slot)
            rd.part[p] = self.peer_ptrs[p] + self.off_stage[slot]
            rd.x[p] = self.peer_ptrs[p] + self.off_x
            rd.x_cnt[p] = self._x_cnt(p)
        sc.rank, sc.tp, sc.chunk, sc.n = self.rank, tp, chunk, self.hidden
        sc.push = 1 if push else 0
        rd.tile_cnt = self._tile_cnt(self.rank, slot)
        rd.done_cnt = self.local_ptr + self.off_cnt + (SLOTS * MAX_GROUPS + 8) * 4
        if self.nvls:
            rd.part_mc = self.mc_ptr + self.off_stage[slot]
            rd.x_mc = self.mc_ptr + self.off_x
            rd.x_cnt_mc = self.mc_ptr + self.off_cnt + SLOTS * MAX_GROUPS * 4
        rd.dbg = self.dbg.data_ptr() if self.dbg is not None else 0
        rd.rank, rd.tp, rd.chunk, rd.n = self.rank, tp, chunk, self.hidden
        rd.x_own = self.x_own_ptr
        for p in range(tp):
            rd.h[p] = self.peer_ptrs[p] + self.off_h
            rd.h_ready[p] = self.peer_ptrs[p] + self.off_ready + slot * READY_WORDS * 4
        if self.nvls:
            rd.h_mc = self.mc_ptr + self.off_h
            rd.h_ready_mc = self.mc_ptr + self.off_ready + slot * READY_WORDS * 4
        rd.group_done = self.local_ptr + self.off_gdone + slot * MAX_GROUPS * 4
        rd.wait_limit_ns = int(self.wait_limit_ns)
        mk = lambda st: torch.frombuffer(bytearray(bytes(st)), dtype=torch.uint8).to(self.device)
        hit = (mk(sc), mk(rd))
        self._structs[key] = hit
        return hit

    def poison(self, why: str) -> None:
        """Mark the group unusable after a device-side wait ran out.  The arrival counters of the exchange are then
        part-consumed (the kernel that gives up does not reset them), so a later exchange would count stale arrivals.
        This rank's counters are cleared so its memory is tidy, but the peers' state is unknown: every further fused
        call raises until the group is torn down and set up again."""
        self.failed = why
        self.ready = False
        try:
            cnt = torch.as_tensor(_CudaArray(self.local_ptr + self.off_cnt, (self.cnt_words,), "<u4"), device=self.device)
            cnt.view(torch.int32).zero_()
        except Exception:
            pass

    def _guard(self, rows: int, slot: int) -> None:
        if self.failed is not None:
            raise RuntimeError(f"fused tensor-parallel group is unusable ({self.failed}); rebuild the process group")
        if rows > self.max_tokens:
            raise ValueError(f"{rows} rows exceed the {self.max_tokens}-row symmetric region")
        # the consumer of a slot resets the slot's counters at its end, which is only safe because no rank can produce
        # into the same slot again before it has passed the other slot's exchange: uses must alternate
        if slot == self._last_slot:
            raise RuntimeError(f"slot {slot} used twice in a row: row-parallel exchanges must alternate between the two slots")
        self._last_slot = slot

    def chunk_for(self, rows: int) -> int:
        tp = self.world
        return max(32, ((rows + tp - 1) // tp + 31) // 32 * 32)

    # -- the fused row-parallel projection -----------------------------------------------------
    def row_parallel(self, a, w, rows: int, slot: int):
        """x[:rows] += sum over ranks of a @ w^T, on every rank (x = the symmetric residual stream)."""
        self._guard(rows, slot)
        chunk = self.chunk_for(rows)
        sc, rd = self._get_structs(slot, chunk)
        st = ops.status_word(self.device).data_ptr()
        stream = torch.cuda.current_stream().cuda_stream
        with ops.timed_region("gemm_scatter[K=%d]" % a.shape[1]):
            rc = self.lib.ogb_gemm_bf16_scatter(a.data_ptr(), w.data_ptr(), rows, self.hidden, a.shape[1], a.stride(0),
                                                w.stride(0), sc.data_ptr(), 0, st, stream)
        _native.check(rc, "ogb_gemm_bf16_scatter")
        with ops.timed_region("tp_reduce_bcast"):
            rc = self.lib.ogb_tp_reduce_bcast(rd.data_ptr(), rows, self.hidden, chunk, self.world, 1 if self.nvls else 0, st, stream)
        _native.check(rc, "ogb_tp_reduce_bcast")
        ops.launch_counts["gemm_bf16_scatter"] += 1
        ops.launch_counts["tp_reduce_bcast"] += 1
        self.calls += 1

    # -- row-sharded residual: reduce-scatter + residual + RMSNorm + all-gather in one kernel ---------------
    def bind_residual(self, x) -> None:
        """``x`` [max_tokens, hidden] is this rank's residual stream (plain local memory, indexed by global row); the
        exchange updates the rows this rank owns in place.  Structs built earlier are rebuilt with the new address."""
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == self.hidden
        self._residual = x
        self.x_own_ptr = x.data_ptr()
        self._structs.clear()

    def set_wait_limit(self, ns: int) -> None:
        """Bound, in nanoseconds, of every wait on another rank's signal in the exchange kernels and in the GEMMs that
        wait for ``h`` (0 = the library's default of two seconds).  A wait that runs out sets the peer-timeout bit of
        the device status word and the kernel returns."""
        self.wait_limit_ns = int(ns)
        self._structs.clear()

    def ready_ptrs(self, slot: int):
        """(ready counters, finished-CTA word) of ``slot`` on this rank, as ``ops.gemm(..., a_ready=...)`` takes them."""
        base = self.local_ptr + self.off_ready + slot * READY_WORDS * 4
        return base, base + 64 * 4, int(self.wait_limit_ns)

    def _exchange_norm(self, rd, norm_w, eps, rows, chunk, st, stream):
        with ops.timed_region("tp_exchange_norm"):
            rc = self.lib.ogb_tp_exchange_norm(rd.data_ptr(), norm_w.data_ptr(), float(eps), rows, self.hidden, chunk, self.world,
                                               1 if self.nvls else 0, 1 if self.push else 0, st, stream)
        _native.check(rc, "ogb_tp_exchange_norm")
        ops.launch_counts["tp_exchange_norm"] += 1
        self.calls += 1

    def row_parallel_norm(self, a, w, rows: int, slot: int, norm_w, eps: float):
        """residual[own rows] += sum over ranks of a @ w^T, then h[:rows] = RMSNorm(residual) * norm_w on every rank
        (delivered tile by tile: consumers wait on :meth:`ready_ptrs`)."""
        assert self.x_own_ptr, "bind_residual() first"
        self._guard(rows, slot)
        chunk = self.chunk_for(rows)
        sc, rd = self._get_structs(slot, chunk, self.push)
        st = ops.status_word(self.device).data_ptr()
        stream = torch.cuda.current_stream().cuda_stream
        with ops.timed_region("gemm_scatter[K=%d]" % a.shape[1]):
            rc = self.lib.ogb_gemm_bf16_scatter(a.data_ptr(), w.data_ptr(), rows, self.hidden, a.shape[1], a.stride(0),
                                                w.stride(0), sc.data_ptr(), 0, st, stream)
        _native.check(rc, "ogb_gemm_bf16_scatter")
        ops.launch_counts["gemm_bf16_scatter"] += 1
        self._exchange_norm(rd, norm_w, eps, rows, chunk, st, stream)

    def reduce_partial_norm(self, rows: int, slot: int, norm_w, eps: float):
        """Same exchange for a partial sum that other kernels left in :meth:`staging_view` (the MoE combine)."""
        assert self.x_own_ptr, "bind_residual() first"
        self._guard(rows, slot)
        chunk = self.chunk_for(rows)
        sc, rd = self._get_structs(slot, chunk, self.push)
        st = ops.status_word(self.device).data_ptr()
        stream = torch.cuda.current_stream().cuda_stream
        if self.push:      # the partial sits in local scratch: copy each 32-row group to its owner and signal it
            rc = self.lib.ogb_tp_push_rows(sc.data_ptr(), self._partial_scratch.data_ptr(), rows, stream)
            _native.check(rc, "ogb_tp_push_rows")
        else:
            rc = self.lib.ogb_tp_signal_rows(sc.data_ptr(), rows, stream)
            _native.check(rc, "ogb_tp_signal_rows")
        ops.launch_counts["tp_signal_rows"] += 1
        self._exchange_norm(rd, norm_w, eps, rows, chunk, st, stream)

    def wait_ready(self, slot: int, rows: int):
        """Order the stream after the arrival of every tile of ``h[:rows]`` of ``slot`` (and clear its counters)."""
        chunk = self.chunk_for(rows)
        _, rd = self._get_structs(slot, chunk)
        rc = self.lib.ogb_tp_wait_ready(rd.data_ptr(), rows, ops.status_word(self.device).data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "ogb_tp_wait_ready")
        ops.launch_counts["tp_wait_ready"] += 1

    # -- partial sums produced by other kernels (MoE combine) -------------------------------------
    def staging_view(self, slot: int, rows: int):
        """This rank's staging buffer of ``slot`` as a [rows, hidden] bf16 tensor: kernels that produce a partial
        sum of the residual stream write it here, then call :meth:`reduce_partial`."""
        if self.push and self.x_own_ptr:
            # producers push: kernels write their partial into local scratch, reduce_partial_norm() forwards the rows
            if self._partial_scratch is None:
                self._partial_scratch = torch.zeros(self.max_tokens, self.hidden, dtype=torch.bfloat16, device=self.device)
            return self._partial_scratch[:rows]
        t = torch.as_tensor(_CudaArray(self.local_ptr + self.off_stage[slot], (self.max_tokens, self.hidden), "<u2"),
                            device=self.device).view(torch.bfloat16)
        return t[:rows]

    def reduce_partial(self, rows: int, slot: int):
        """x[:rows] += sum over ranks of the staged partials (same exchange kernel as :meth:`row_parallel`)."""
        self._guard(rows, slot)
        chunk = self.chunk_for(rows)
        sc, rd = self._get_structs(slot, chunk)
        st = ops.status_word(self.device).data_ptr()
        stream = torch.cuda.current_stream().cuda_stream
        rc = self.lib.ogb_tp_signal_rows(sc.data_ptr(), rows, stream)
        _native.check(rc, "ogb_tp_signal_rows")
        with ops.timed_region("tp_reduce_bcast"):
            rc = self.lib.ogb_tp_reduce_bcast(rd.data_ptr(), rows, self.hidden, chunk, self.world, 1 if self.nvls else 0, st, stream)
        _native.check(rc, "ogb_tp_reduce_bcast")
        ops.launch_counts["tp_signal_rows"] += 1
        ops.launch_counts["tp_reduce_bcast"] += 1
        self.calls += 1
