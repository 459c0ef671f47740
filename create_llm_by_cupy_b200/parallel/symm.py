"""Symmetric-memory heap and the fused peer-memory collectives built on it.

``SymmetricHeap``: one ``cudaMalloc`` block per rank, exported with CUDA IPC and mapped by every
peer, so that the same byte offset names the same buffer on every GPU. A bump allocator hands out
torch tensors that alias the heap; all ranks allocate in the same order, hence symmetric offsets.
The first 64 KiB hold the signal flags the kernels use for their cross-GPU barriers.

``FusedCollectives`` is what a ZeRO manager takes as ``fused=``:
  * ``reduce_scatter_accumulate`` — one kernel: barrier, P2P pull of this rank's slice of every
    peer's gradient bucket, fp32 sum, store / accumulate (or AdamW), gradient statistics, barrier;
  * ``all_gather`` — P2P pull of every peer's parameter slice into the local unit buffer;
  * ``barrier`` — device-side barrier fencing the optimizer step.
The NCCL path of ``comm.py`` is the baseline these are measured against.

Virtual ranks: ``LocalVirtualRanks`` builds W heaps on ONE device and drives the same kernels with
``gridDim.y = W`` (all ranks inside one launch), which is how the protocol is tested on a single
GPU; ranks that wait on one another are never emulated by separate launches on one device.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import native

_DEFAULT_WAIT_NS = 20_000_000_000   # 20 s: a peer that never arrives ends in an error status, not a hang


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
        """Zero-initialised tensor of ``n`` elements at the next 256-byte aligned heap offset."""
        esz = torch.empty((), dtype=dtype).element_size()
        off = (self.cursor + 255) // 256 * 256
        nbytes = n * esz
        if off + nbytes > self.heap_bytes:
            raise MemoryError(f"symmetric heap exhausted: need {off + nbytes} of {self.heap_bytes} bytes")
        self.cursor = off + nbytes
        return self.bytes_view[off:off + nbytes].view(dtype)

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off >= self.heap_bytes:
            raise ValueError("tensor does not live in the symmetric heap")
        return off

    def contains(self, t: torch.Tensor) -> bool:
        return 0 <= t.data_ptr() - self.base < self.heap_bytes

    def close(self):
        for p in self._imported:
            self.lib.b200_symm_unimport(ctypes.c_void_p(p))
        self._imported = []
        if self.base:
            torch.cuda.synchronize(self.device)
            self.lib.b200_symm_free(ctypes.c_void_p(self.base))
            self.base = 0


class FusedCollectives:
    """Peer-memory collectives for one rank (one process per GPU)."""

    gather = True

    def __init__(self, comm, device, heap_bytes: int = 8 << 30, rs_blocks: int = 64, ag_blocks: int = 64,
                 wait_ns: int = _DEFAULT_WAIT_NS, gather_mode: str = "pull", n_copy: int = 8):
        """``gather_mode`` selects how parameter units are gathered: ``"nccl"`` (ncclAllGather on the
        communication stream), ``"pull"`` (the P2P pull kernel on the communication stream) or
        ``"gemm"`` (transformer-block units are pulled inside the first GEMM that consumes them;
        the other units use the pull kernel). Gradient reduction always uses the fused kernel."""
        if gather_mode not in ("nccl", "pull", "gemm"):
            raise ValueError(f"unknown gather_mode {gather_mode!r}")
        self.heap = SymmetricHeap(comm, device, heap_bytes)
        self.comm = comm
        self.device = self.heap.device
        self.world_size = comm.world_size
        self.rank = comm.rank
        self.lib = self.heap.lib
        self.rs_blocks = rs_blocks
        self.ag_blocks = ag_blocks
        self.wait_ns = int(wait_ns)
        self.gather_mode = gather_mode
        self.gather = gather_mode != "nccl"
        self.gemm_fusion = gather_mode == "gemm"   # pull block units inside their first consuming GEMM
        self.n_copy = n_copy                # CTAs of that GEMM that copy instead of multiply
        self.rs_epoch = 0
        self.barrier_epoch = 0
        self.launches = 0

    def alloc(self, n: int, dtype) -> torch.Tensor:
        return self.heap.alloc(n, dtype)

    def reduce_scatter_accumulate(self, dst: torch.Tensor, bucket: torch.Tensor, accumulate: bool, stream=None,
                                  stats: torch.Tensor | None = None, do_stats: bool = False, adam: dict | None = None):
        """dst[n] (<- or +=) sum over ranks of their bucket[rank * n : (rank + 1) * n]; bucket is a
        bf16 heap tensor at the same offset on every rank. With ``adam`` (tensors m, v, master,
        param and the scalar hyper-parameters) the reduced gradient goes straight into AdamW."""
        n = dst.numel()
        assert bucket.numel() == n * self.world_size and bucket.dtype == torch.bfloat16 and n % 8 == 0
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
        rc = self.lib.b200_symm_reduce_scatter(
            self.heap.table, self.world_size, self.rank, 1, ctypes.c_ulonglong(self.heap.offset_of(bucket)),
            ctypes.c_longlong(n), _ptr_array([dst.data_ptr()]), int(dst.dtype == torch.float32), mode,
            _ptr_array([stats.data_ptr() if stats is not None else 0]), int(do_stats), adam_ptrs, adam_f,
            ctypes.c_uint(self.rs_epoch), ctypes.c_ulonglong(self.wait_ns), self.rs_blocks, s)
        native.check(rc, "symm_reduce_scatter")
        native.bump()

    def all_gather(self, out: torch.Tensor, shard_slice: torch.Tensor, stream=None, skip=None, only=None):
        """out[W * n] <- every rank's shard_slice[n] (shard_slice is a heap tensor). ``skip`` /
        ``only`` = (lo, hi) byte range of ``out`` to leave out / to restrict the copy to."""
        n = shard_slice.numel()
        assert out.numel() == n * self.world_size and n % 8 == 0 and shard_slice.element_size() == 2
        s = native.stream_ptr() if stream is None else ctypes.c_void_p(stream.cuda_stream)
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

    def barrier(self, stream=None, channel: int = 1):
        self.barrier_epoch += 1
        s = native.stream_ptr() if stream is None else ctypes.c_void_p(stream.cuda_stream)
        rc = self.lib.b200_symm_barrier(self.heap.table, self.world_size, self.rank, 1, channel,
                                        ctypes.c_uint(self.barrier_epoch), ctypes.c_ulonglong(self.wait_ns), s)
        native.check(rc, "symm_barrier")
        native.bump()

    def close(self):
        self.heap.close()


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
                       adam=None, blocks: int = 4):
        self.rs_epoch += 1
        W = self.world_size
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
        rc = self.lib.b200_symm_reduce_scatter(
            self.tables, W, 0, W, ctypes.c_ulonglong(bucket_off), ctypes.c_longlong(n_slice),
            _ptr_array([d.data_ptr() for d in dsts]), int(dsts[0].dtype == torch.float32), mode,
            _ptr_array([s.data_ptr() for s in stats] if stats is not None else [0] * W), int(do_stats), adam_ptrs, adam_f,
            ctypes.c_uint(self.rs_epoch), ctypes.c_ulonglong(self.wait_ns), blocks, native.stream_ptr())
        native.check(rc, "symm_reduce_scatter")

    def all_gather(self, shard_off: int, n_slice: int, outs, blocks: int = 4):
        rc = self.lib.b200_symm_all_gather(self.tables, self.world_size, 0, self.world_size,
                                           ctypes.c_ulonglong(shard_off), ctypes.c_longlong(n_slice),
                                           _ptr_array([o.data_ptr() for o in outs]), blocks, native.stream_ptr())
        native.check(rc, "symm_all_gather")

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
