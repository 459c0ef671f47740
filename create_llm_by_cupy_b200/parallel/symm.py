"""Symmetric-memory heap and the fused peer-memory collectives built on it.

``SymmetricHeap``: one ``cudaMalloc`` block per rank, exported with CUDA IPC and mapped by every
peer, so that the same byte offset names the same buffer on every GPU. A bump allocator hands out
torch tensors that alias the heap; all ranks allocate in the same order, hence symmetric offsets.
The first 64 KiB hold the signal flags the kernels use for their cross-GPU barriers.

``FusedCollectives`` is what a ZeRO manager takes as ``fused=``:
  * ``reduce_scatter_accumulate`` — one kernel: barrier, P2P pull of this rank's slice of every
    peer's gradient bucket, fp32 sum, store / accumulate (or AdamW), gradient statistics, barrier;
  * ``all_gather`` — every peer's parameter slice into the local unit buffer, by the copy engines
    (one ``cudaMemcpyAsync`` per peer slice, no SM involved; the default) or by the P2P pull kernel;
  * ``barrier`` — device-side barrier fencing the optimizer step.
The NCCL path of ``comm.py`` is the baseline these are measured against.

Every heap allocation sits between two 256-byte guard blocks filled with a known pattern;
``check_canaries()`` (also run by ``close()``) reports any allocation whose guards were overwritten —
the stand-in for a memory checker on buffers that other GPUs write and read through peer pointers.

Virtual ranks: ``LocalVirtualRanks`` builds W heaps on ONE device and drives the same kernels with
``gridDim.y = W`` (all ranks inside one launch), which is how the protocol is tested on a single
GPU; ranks that wait on one another are never emulated by separate launches on one device.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import native

# Budget of one cross-GPU wait (barrier flags): a peer that never arrives ends in an error status, not a
# hang. Ranks legitimately drift apart by far less than this (first-step lazy loading, a checkpoint write on
# one rank is fenced by a host barrier); the waits on local mbarriers inside the compute kernels use 2 s.
_DEFAULT_WAIT_NS = 10_000_000_000
_GUARD_BYTES = 256
_GUARD_BYTE = 0xA5
_DEFAULT_HEAP_BYTES = 8 << 30


class _RawCuda:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _wrap(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device)


def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(int(p)) for p in ptrs])


class SymmetricHeap:
    def __init__(self, comm, device, heap_bytes: int = 8 << 30):
        self.comm = comm
        self.device = torch.device(device)
        self.world_size = comm.world_size
        self.rank = comm.rank
        self.lib = native.lib()
        native.status_tensor(self.device)
        self.heap_bytes = int(heap_bytes)
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            native.check(self.lib.b200_symm_alloc(ctypes.c_ulonglong(self.heap_bytes), ctypes.byref(base)), "symm_alloc")
        self.base = int(base.value)
        self.pad_bytes = int(self.lib.b200_symm_pad_bytes())
        self.cursor = self.pad_bytes
        self.bytes_view = _wrap(self.base, self.heap_bytes, self.device)
        self.guards = []          # (byte offset of the data, data bytes) of every allocation
        self.peer_bases = [0] * self.world_size
        self.peer_bases[self.rank] = self.base
        self._imported = []
        if self.world_size > 1:
            handle = (ctypes.c_ubyte * 64)()
            native.check(self.lib.b200_symm_export(ctypes.c_void_p(self.base), handle), "symm_export")
            handles = comm.all_gather_object(bytes(handle))
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                out = ctypes.c_void_p()
                with torch.cuda.device(self.device):
                    native.check(self.lib.b200_symm_import(buf, ctypes.byref(out)), "symm_import")
                self.peer_bases[r] = int(out.value)
                self._imported.append(int(out.value))
            comm.barrier()
        self.table = _ptr_array(self.peer_bases)

    def alloc(self, n: int, dtype) -> torch.Tensor:
        """Zero-initialised tensor of ``n`` elements at the next 256-byte aligned heap offset, with a
        256-byte guard block on either side."""
        esz = torch.empty((), dtype=dtype).element_size()
        g0 = (self.cursor + 255) // 256 * 256
        off = g0 + _GUARD_BYTES
        nbytes = n * esz
        g1 = (off + nbytes + 255) // 256 * 256
        if g1 + _GUARD_BYTES > self.heap_bytes:
            raise MemoryError(f"symmetric heap exhausted: need {g1 + _GUARD_BYTES} of {self.heap_bytes} bytes")
        self.cursor = g1 + _GUARD_BYTES
        self.bytes_view[g0:off].fill_(_GUARD_BYTE)
        self.bytes_view[off + nbytes:g1 + _GUARD_BYTES].fill_(_GUARD_BYTE)
        self.guards.append((off, nbytes))
        return self.bytes_view[off:off + nbytes].view(dtype)

    def check_canaries(self) -> list:
        """Indices (allocation order) of the allocations whose guard blocks no longer hold the pattern,
        i.e. something wrote outside a neighbouring buffer. Synchronises the device."""
        bad = []
        for i, (off, nbytes) in enumerate(self.guards):
            end = (off + nbytes + 255) // 256 * 256 + _GUARD_BYTES
            lo = self.bytes_view[off - _GUARD_BYTES:off]
            hi = self.bytes_view[off + nbytes:end]
            if bool((lo != _GUARD_BYTE).any()) or bool((hi != _GUARD_BYTE).any()):
                bad.append(i)
        return bad

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off >= self.heap_bytes:
            raise ValueError("tensor does not live in the symmetric heap")
        return off

    def contains(self, t: torch.Tensor) -> bool:
        return 0 <= t.data_ptr() - self.base < self.heap_bytes

    def close(self):
        """Unmap the peers, free the heap; raises afterwards if a guard block was overwritten."""
        bad = []
        if self.base:
            torch.cuda.synchronize(self.device)
            bad = self.check_canaries()
        for p in self._imported:
            self.lib.b200_symm_unimport(ctypes.c_void_p(p))
        if self._imported and self.world_size > 1:
            self.comm.barrier()           # nobody frees a heap a peer still has mapped
        self._imported = []
        if self.base:
            self.bytes_view = None
            self.lib.b200_symm_free(ctypes.c_void_p(self.base))
            self.base = 0
        if bad:
            raise RuntimeError(f"symmetric heap: guard blocks of allocation(s) {bad} were overwritten "
                               f"(sizes {[self.guards[i][1] for i in bad]} bytes)")


class FusedCollectives:
    """Peer-memory collectives for one rank (one process per GPU)."""

    gather = True

    def __init__(self, comm, device, heap_bytes: int | None = None, rs_blocks: int = 64, ag_blocks: int = 64,
                 wait_ns: int = _DEFAULT_WAIT_NS, gather_mode: str = "copy", n_copy: int = 8,
                 copy_min_bytes: int = 1 << 20, reduce_mode: str = "copy", rs_local_blocks: int = 0):
        """``gather_mode`` selects how parameter units are gathered: ``"copy"`` (one ``cudaMemcpyAsync``
        per peer slice on the communication stream: the copy engines move the unit and no SM is taken
        from the GEMMs; slices below ``copy_min_bytes`` use the pull kernel), ``"pull"`` (the P2P pull
        kernel), ``"nccl"`` (ncclAllGather) or ``"gemm"`` (the first GEMM that consumes a
        transformer-block unit pulls its own weight while it runs; the rest of the unit and the other units go
        through the copy engines). ``reduce_mode`` selects how
        gradient buckets are reduced: ``"pull"`` (the fused kernel reads the peers' slices over NVLink while it
        sums) or ``"copy"`` (the default: the copy engines bring the peers' parts of this rank's slice into a local staging
        buffer between two barriers and the same kernel then sums local memory only: no SM ever waits on the
        link; parts below ``copy_min_bytes`` use the pull form). ``heap_bytes`` None: the heap is created on the first ``reserve`` /
        ``alloc`` (the ZeRO manager reserves what its layout needs)."""
        if gather_mode not in ("nccl", "pull", "gemm", "copy"):
            raise ValueError(f"unknown gather_mode {gather_mode!r}")
        if reduce_mode not in ("pull", "copy"):
            raise ValueError(f"unknown reduce_mode {reduce_mode!r}")
        self.comm = comm
        self.device = torch.device(device)
        self.world_size = comm.world_size
        self.rank = comm.rank
        self.lib = native.lib()
        self._heap = None
        if heap_bytes is not None:
            self._heap = SymmetricHeap(comm, device, heap_bytes)
        self.rs_blocks = rs_blocks
        self.ag_blocks = ag_blocks
        self.wait_ns = int(wait_ns)
        self.gather_mode = gather_mode
        self.gather = gather_mode != "nccl"
        self.gemm_fusion = gather_mode == "gemm"   # pull block units inside their first consuming GEMM
        self.copy_engine = gather_mode in ("copy", "gemm")     # "gemm": what the GEMM does not pull itself
        self.copy_min_bytes = int(copy_min_bytes)
        self.n_copy = n_copy                # CTAs of that GEMM that copy instead of multiply
        self.reduce_mode = reduce_mode
        if not rs_local_blocks:
            rs_local_blocks = (2 * torch.cuda.get_device_properties(self.device).multi_processor_count
                               if self.device.type == "cuda" else 8)
        self.rs_local_blocks = int(rs_local_blocks)
        self._stage = None                  # staging buffer of the copy-engine reduce-scatter (local memory)
        self.rs_epoch = 0
        self.stage_epoch = 0
        self.barrier_epochs = {}            # channel -> barriers issued on it so far
        self.launches = 0                   # kernels of this module launched so far
        self.copies = 0                     # copy-engine transfers issued so far

    @property
    def heap(self) -> SymmetricHeap:
        if self._heap is None:
            self._heap = SymmetricHeap(self.comm, self.device, _DEFAULT_HEAP_BYTES)
        return self._heap

    def reserve(self, nbytes: int):
        """Create the heap with room for ``nbytes`` of allocations (plus signal pad and guards) if it
        does not exist yet. Every rank must ask for the same size."""
        if self._heap is None:
            total = int(nbytes) + (64 << 20)
            self._heap = SymmetricHeap(self.comm, self.device, (total + (1 << 21) - 1) >> 21 << 21)
        return self._heap

    def alloc(self, n: int, dtype) -> torch.Tensor:
        return self.heap.alloc(n, dtype)

    def reserve_stage(self, part_elems: int):
        """Make the staging buffer of the copy-engine reduce-scatter hold W - 1 parts of ``part_elems`` bf16
        elements (the largest share of one launch that falls into a rank's slice). Called before the first
        collective so that no device allocation happens while peers wait in a kernel."""
        part = (int(part_elems) + 7) // 8 * 8
        need = part * max(self.world_size - 1, 1)
        if self._stage is None or self._stage.numel() < need:
            self._stage = torch.empty(need, dtype=torch.bfloat16, device=self.device)
        return self._stage

    def reduce_scatter_accumulate(self, dst: torch.Tensor, bucket: torch.Tensor, accumulate: bool, stream=None,
                                  stats: torch.Tensor | None = None, do_stats: bool = False, adam: dict | None = None,
                                  elem_range: tuple | None = None):
        """dst[n] (<- or +=) sum over ranks of their bucket[rank * n : (rank + 1) * n]; bucket is a
        bf16 heap tensor at the same offset on every rank. With ``adam`` (tensors m, v, master,
        param and the scalar hyper-parameters) the reduced gradient goes straight into AdamW.
        ``elem_range`` = (lo, hi), multiples of 8: only those elements of the bucket are reduced (a
        sub-bucket that is complete before the rest); each rank handles what falls into its slice."""
        n = dst.numel()
        assert bucket.numel() == n * self.world_size and bucket.dtype == torch.bfloat16 and n % 8 == 0
        lo, hi = elem_range if elem_range is not None else (0, bucket.numel())
        assert 0 <= lo <= hi <= bucket.numel() and lo % 8 == 0 and hi % 8 == 0
        self.rs_epoch += 1
        mode = 2 if adam is not None else (1 if accumulate else 0)
        if mode == 1:
            assert dst.dtype == torch.float32
        adam_ptrs = None
        adam_f = None
        if adam is not None:
            adam_ptrs = _ptr_array([adam["m"].data_ptr(), adam["v"].data_ptr(), adam["master"].data_ptr(),
                                    adam["param"].data_ptr()])
            adam_f = (ctypes.c_float * 8)(adam["lr"], adam["beta1"], adam["beta2"], adam["eps"], adam["weight_decay"],
                                          adam["m_corr"], adam["v_corr"], adam["grad_scale"])
        s = native.stream_ptr() if stream is None else ctypes.c_void_p(stream.cuda_stream)
        # the rank's share of this launch; every rank computes every rank's share, so all take the same branch
        shares = [max(0, min(hi, (r + 1) * n) - max(lo, r * n)) for r in range(self.world_size)]
        if self.reduce_mode == "copy" and self.world_size > 1 and max(shares) * 2 >= self.copy_min_bytes:
            part = (max(shares) + 7) // 8 * 8
            stage = self.reserve_stage(part)
            self.stage_epoch += 1
            rc = self.lib.b200_symm_reduce_scatter_staged(
                self.heap.table, self.world_size, self.rank, ctypes.c_ulonglong(self.heap.offset_of(bucket)),
                ctypes.c_longlong(n), ctypes.c_longlong(lo), ctypes.c_longlong(hi), ctypes.c_void_p(dst.data_ptr()),
                int(dst.dtype == torch.float32), mode, ctypes.c_void_p(stats.data_ptr() if stats is not None else 0),
                int(do_stats), adam_ptrs, adam_f, ctypes.c_void_p(stage.data_ptr()), ctypes.c_longlong(part), 1, 2,
                ctypes.c_uint(self.stage_epoch), ctypes.c_ulonglong(self.wait_ns), self.rs_local_blocks, s)
            native.check(rc, "symm_reduce_scatter_staged")
            native.bump(3 if shares[self.rank] > 0 else 2)
            self.launches += 3 if shares[self.rank] > 0 else 2
            if shares[self.rank] > 0:
                self.copies += self.world_size - 1
            return
        rc = self.lib.b200_symm_reduce_scatter_range(
            self.heap.table, self.world_size, self.rank, 1, ctypes.c_ulonglong(self.heap.offset_of(bucket)),
            ctypes.c_longlong(n), ctypes.c_longlong(lo), ctypes.c_longlong(hi), _ptr_array([dst.data_ptr()]),
            int(dst.dtype == torch.float32), mode,
            _ptr_array([stats.data_ptr() if stats is not None else 0]), int(do_stats), adam_ptrs, adam_f,
            ctypes.c_uint(self.rs_epoch), ctypes.c_ulonglong(self.wait_ns), self.rs_blocks, s)
        native.check(rc, "symm_reduce_scatter")
        native.bump()
        self.launches += 1

    def all_gather(self, out: torch.Tensor, shard_slice: torch.Tensor, stream=None, skip=None, only=None):
        """out[W * n] <- every rank's shard_slice[n] (shard_slice is a heap tensor). ``skip`` /
        ``only`` = (lo, hi) byte range of ``out`` to leave out / to restrict the copy to."""
        n = shard_slice.numel()
        assert out.numel() == n * self.world_size and n % 8 == 0 and shard_slice.element_size() == 2
        s = native.stream_ptr() if stream is None else ctypes.c_void_p(stream.cuda_stream)
        if self.copy_engine and skip is None and only is None and n * 2 >= self.copy_min_bytes:
            rc = self.lib.b200_symm_all_gather_copy(self.heap.table, self.world_size, self.rank,
                                                    ctypes.c_ulonglong(self.heap.offset_of(shard_slice)),
                                                    ctypes.c_longlong(n), 2, ctypes.c_void_p(out.data_ptr()), s)
            native.check(rc, "symm_all_gather_copy")
            self.copies += self.world_size - 1
            return
        if self.copy_engine and skip is not None and only is None and n * 2 >= self.copy_min_bytes:
            rc = self.lib.b200_symm_all_gather_copy_skip(
                self.heap.table, self.world_size, self.rank, ctypes.c_ulonglong(self.heap.offset_of(shard_slice)),
                ctypes.c_longlong(n), 2, ctypes.c_void_p(out.data_ptr()), ctypes.c_ulonglong(skip[0]),
                ctypes.c_ulonglong(skip[1]), s)
            native.check(rc, "symm_all_gather_copy_skip")
            self.copies += self.world_size - 1
            return
        if skip is None and only is None:
            rc = self.lib.b200_symm_all_gather(self.heap.table, self.world_size, self.rank, 1,
                                               ctypes.c_ulonglong(self.heap.offset_of(shard_slice)), ctypes.c_longlong(n),
                                               _ptr_array([out.data_ptr()]), self.ag_blocks, s)
        else:
            lo, hi = skip if skip is not None else only
            rc = self.lib.b200_symm_all_gather_range(
                self.heap.table, self.world_size, self.rank, 1, ctypes.c_ulonglong(self.heap.offset_of(shard_slice)),
                ctypes.c_longlong(n), _ptr_array([out.data_ptr()]), self.ag_blocks, ctypes.c_ulonglong(lo),
                ctypes.c_ulonglong(hi), 1 if skip is not None else 2, s)
        native.check(rc, "symm_all_gather")
        native.bump()
        self.launches += 1

    def barrier(self, stream=None, channel: int = 1):
        """Cross-GPU barrier kernel on ``stream``. A channel has its own flags and its own epoch count, and all
        barriers of one channel must be issued on ONE stream: two barrier kernels of a channel in flight at once
        can overwrite each other's epochs in a peer's flag word (the later one then waits until its time-out).
        Channel 1: the optimizer's stream (per-unit "slice updated"); channel 2: the communication stream (the
        copy-engine reduce-scatter); channel 3: the compute stream (whole-step fences)."""
        self.barrier_epochs[channel] = self.barrier_epochs.get(channel, 0) + 1
        s = native.stream_ptr() if stream is None else ctypes.c_void_p(stream.cuda_stream)
        rc = self.lib.b200_symm_barrier(self.heap.table, self.world_size, self.rank, 1, channel,
                                        ctypes.c_uint(self.barrier_epochs[channel]), ctypes.c_ulonglong(self.wait_ns), s)
        native.check(rc, "symm_barrier")
        native.bump()
        self.launches += 1

    def check_canaries(self) -> list:
        return self._heap.check_canaries() if self._heap is not None else []

    def close(self):
        if self._heap is not None:
            self._heap.close()


class LocalVirtualRanks:
    """W heaps on one device; every collective is ONE launch whose gridDim.y enumerates the ranks."""

    def __init__(self, world_size: int, device="cuda", heap_bytes: int = 64 << 20, wait_ns: int = 2_000_000_000):
        self.world_size = world_size
        self.device = torch.device(device)
        self.lib = native.lib()
        native.status_tensor(self.device)
        self.heap_bytes = heap_bytes
        self.bases = []
        for _ in range(world_size):
            b = ctypes.c_void_p()
            native.check(self.lib.b200_symm_alloc(ctypes.c_ulonglong(heap_bytes), ctypes.byref(b)), "symm_alloc")
            self.bases.append(int(b.value))
        self.views = [_wrap(b, heap_bytes, self.device) for b in self.bases]
        self.cursor = int(self.lib.b200_symm_pad_bytes())
        self.wait_ns = wait_ns
        self.rs_epoch = 0
        self.barrier_epoch = 0
        # every virtual rank sees the same mapping (all heaps are local)
        self.tables = _ptr_array([b for _ in range(world_size) for b in self.bases])

    def alloc(self, n: int, dtype):
        """The same offset in every heap: returns one tensor per rank."""
        esz = torch.empty((), dtype=dtype).element_size()
        off = (self.cursor + 255) // 256 * 256
        self.cursor = off + n * esz
        assert self.cursor <= self.heap_bytes
        return off, [v[off:off + n * esz].view(dtype) for v in self.views]

    def reduce_scatter(self, bucket_off: int, n_slice: int, dsts, accumulate=False, stats=None, do_stats=False,
                       adam=None, blocks: int = 4, elem_range: tuple | None = None):
        self.rs_epoch += 1
        W = self.world_size
        lo, hi = elem_range if elem_range is not None else (0, W * n_slice)
        mode = 2 if adam is not None else (1 if accumulate else 0)
        adam_ptrs = adam_f = None
        if adam is not None:
            flat = []
            for r in range(W):
                flat += [adam["m"][r].data_ptr(), adam["v"][r].data_ptr(), adam["master"][r].data_ptr(),
                         adam["param"][r].data_ptr()]
            adam_ptrs = _ptr_array(flat)
            adam_f = (ctypes.c_float * 8)(adam["lr"], adam["beta1"], adam["beta2"], adam["eps"], adam["weight_decay"],
                                          adam["m_corr"], adam["v_corr"], adam["grad_scale"])
        rc = self.lib.b200_symm_reduce_scatter_range(
            self.tables, W, 0, W, ctypes.c_ulonglong(bucket_off), ctypes.c_longlong(n_slice), ctypes.c_longlong(lo),
            ctypes.c_longlong(hi), _ptr_array([d.data_ptr() for d in dsts]), int(dsts[0].dtype == torch.float32), mode,
            _ptr_array([s.data_ptr() for s in stats] if stats is not None else [0] * W), int(do_stats), adam_ptrs, adam_f,
            ctypes.c_uint(self.rs_epoch), ctypes.c_ulonglong(self.wait_ns), blocks, native.stream_ptr())
        native.check(rc, "symm_reduce_scatter")

    def reduce_scatter_staged(self, bucket_off: int, n_slice: int, dsts, accumulate=False, stats=None, do_stats=False,
                              blocks: int = 8, elem_range: tuple | None = None, ranks=None, stage=None):
        """The copy-engine form of the reduce-scatter, the ranks one after the other on this device: per rank the
        W - 1 staging copies and the local summing kernel, without the cross-rank barriers (nothing runs
        concurrently here, and kernels that wait on one another may not be separate launches on one GPU).
        ``ranks``: only these ranks (default all); ``stage``: a staging buffer to reuse (timing loops)."""
        W = self.world_size
        lo, hi = elem_range if elem_range is not None else (0, W * n_slice)
        part = max(max(0, min(hi, (r + 1) * n_slice) - max(lo, r * n_slice)) for r in range(W))
        part = max((part + 7) // 8 * 8, 8)
        own_stage = stage is None
        if own_stage:
            stage = torch.empty(part * max(W - 1, 1), dtype=torch.bfloat16, device=self.device)
        assert stage.numel() >= part * max(W - 1, 1)
        for r in (range(W) if ranks is None else ranks):
            rc = self.lib.b200_symm_reduce_scatter_staged(
                _ptr_array(self.bases), W, r, ctypes.c_ulonglong(bucket_off), ctypes.c_longlong(n_slice),
                ctypes.c_longlong(lo), ctypes.c_longlong(hi), ctypes.c_void_p(dsts[r].data_ptr()),
                int(dsts[r].dtype == torch.float32), 1 if accumulate else 0,
                ctypes.c_void_p(stats[r].data_ptr() if stats is not None else 0), int(do_stats), None, None,
                ctypes.c_void_p(stage.data_ptr()), ctypes.c_longlong(part), 0, 2, ctypes.c_uint(1),
                ctypes.c_ulonglong(self.wait_ns), blocks, native.stream_ptr())
            native.check(rc, "symm_reduce_scatter_staged")
        if own_stage:
            torch.cuda.synchronize(self.device)      # the staging buffer is freed on return

    def all_gather(self, shard_off: int, n_slice: int, outs, blocks: int = 4):
        rc = self.lib.b200_symm_all_gather(self.tables, self.world_size, 0, self.world_size,
                                           ctypes.c_ulonglong(shard_off), ctypes.c_longlong(n_slice),
                                           _ptr_array([o.data_ptr() for o in outs]), blocks, native.stream_ptr())
        native.check(rc, "symm_all_gather")

    def gemm_allgather(self, a, shard_off: int, n_slice: int, unit_buf, b_offset: int, b_shape, *, trans_b: bool,
                       only_b: bool = False, n_copy: int = 4, add=None):
        """The GEMM with the all-gather fused in, as ONE rank sees it, with every "peer" slice on this
        device: ``unit_buf`` (W * n_slice bf16, local) is filled from the W heaps' slices at ``shard_off``
        by the copy CTAs of the same launch that multiplies ``a`` with the weight stored at element
        ``b_offset`` of ``unit_buf``. With ``only_b`` the kernel copies just the chunks that hold that
        weight and the rest of the unit is gathered here by the pull kernel (range mode), as the ZeRO
        manager does on its communication stream. Returns the product."""
        from ..ops.gemm import ag_region, gemm_allgather
        W = self.world_size
        assert unit_buf.numel() == W * n_slice and unit_buf.dtype == torch.bfloat16
        peer = [b + shard_off for b in self.bases]
        seg = torch.zeros((unit_buf.numel() * 2 + (1 << 20) - 1) >> 20, dtype=torch.int64, device=self.device)
        if only_b:
            n_b = 1
            for d in b_shape:
                n_b *= int(d)
            lo, hi = ag_region(n_slice * 2, W, b_offset * 2, n_b * 2)
            rc = self.lib.b200_symm_all_gather_range(
                _ptr_array(self.bases), W, 0, 1, ctypes.c_ulonglong(shard_off), ctypes.c_longlong(n_slice),
                _ptr_array([unit_buf.data_ptr()]), 4, ctypes.c_ulonglong(lo), ctypes.c_ulonglong(hi), 1,
                native.stream_ptr())
            native.check(rc, "symm_all_gather_range")
        return gemm_allgather(a, unit_buf, b_offset, tuple(b_shape), trans_b=trans_b, peer_slices=peer, seg=seg,
                              epoch=1, n_copy=n_copy, add=add, only_b=only_b)

    def barrier(self, channel: int = 1):
        self.barrier_epoch += 1
        rc = self.lib.b200_symm_barrier(self.tables, self.world_size, 0, self.world_size, channel,
                                        ctypes.c_uint(self.barrier_epoch), ctypes.c_ulonglong(self.wait_ns),
                                        native.stream_ptr())
        native.check(rc, "symm_barrier")

    def close(self):
        torch.cuda.synchronize(self.device)
        for b in self.bases:
            self.lib.b200_symm_free(ctypes.c_void_p(b))
        self.bases = []
