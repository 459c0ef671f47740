"""ZeRO runtime: ``MemoryZeRO3Manager`` (parameters, gradients and optimizer state sharded) and
``MemoryZeRO2_5Manager`` (a chosen fraction of the parameters replicated, the rest ZeRO-3; the
replicas' gradients and optimizer state still sharded).

They keep the manager protocol the model calls between layers (reference: model/ZeRO3.py:798-1707,
model/ZeRO2_5.py:788-1363) — gather/prefetch/wait/release of module parameters, gradient buckets
flushed asynchronously, embedding handling, step-boundary statistics — on top of a different
data layout: every unit (one transformer block, the embedding, ...) is sharded evenly across
ranks (see ``layout.py``), so a gather is ONE balanced all-gather into a pooled unit buffer whose
slices become the layer parameters (views, no copies), and a gradient flush is ONE balanced
reduce-scatter of the unit's flat gradient buffer that the GEMMs wrote in place. Communication
runs on a side stream ordered with events; the host never blocks in the steady state.

Fused mode (``fused=True`` with a symmetric-memory heap): the reduce-scatter is replaced by a
kernel that pulls the peers' bucket slices over NVLink, sums them in fp32, scales and either
accumulates into the fp32 gradient shard or applies AdamW directly, and the all-gather by a pull
kernel that writes tile-ready flags the consuming GEMM waits on; NCCL remains the baseline.
"""
from __future__ import annotations

import collections
import time

import torch

from ..ops import functional as F
from .layout import FlatLayout, select_replicated_params


class _Buf:
    __slots__ = ("t", "free_event", "ready_event", "uid", "seg", "epoch", "flushed")

    def __init__(self, t):
        self.t = t
        self.free_event = None
        self.ready_event = None
        self.uid = -1
        self.seg = None
        self.epoch = 0
        self.flushed = []        # element ranges of a gradient bucket that were reduced ahead of the rest


class _PendingGather:
    """A unit whose all-gather has not run yet because it is going to be fused into the first GEMM
    that reads one of its weights. ``gemm`` launches that fused kernel; ``flush`` falls back to the
    stand-alone pull when something else touches the unit first."""

    def __init__(self, mgr, uid: int, buf, param_index=None, region=None, rest_ready=None):
        self.mgr, self.uid, self.buf = mgr, uid, buf
        self.done = False
        # The weight the fused GEMM is expected to read, the byte range of the unit buffer that GEMM
        # will fill itself, and the event after which the rest of the unit (pulled on the
        # communication stream when the gather was requested) is in place.
        self.param_index, self.region, self.rest_ready = param_index, region, rest_ready

    def _peer_slices(self):
        m = self.mgr
        lo, _ = m.layout.unit_shard_range(self.uid)
        off = m.fused.heap.offset_of(m.param_shard_f16) + lo * m.param_shard_f16.element_size()
        return [b + off for b in m.fused.heap.peer_bases]

    def gemm(self, a, param_index: int, *, trans_b: bool, add=None, out=None):
        from ..ops.gemm import gemm_allgather
        m = self.mgr
        s = m.layout.slots[param_index]
        assert s.unit == self.uid and not self.done
        if self.region is not None and param_index != self.param_index:
            self.flush()                      # another weight came first: finish the gather the plain way
            from ..ops import functional as F
            return F.gemm(a, m.model.params[param_index], trans_b=trans_b, add=add, out=out)
        b = self.buf
        if getattr(b, "seg", None) is None:
            b.seg = torch.zeros((b.t.numel() * 2 + (1 << 20) - 1) >> 20, dtype=torch.int64, device=m.device)
            b.epoch = 0
        only_b = self.region is not None
        if only_b:
            b.seg.zero_()                     # the copied range differs from use to use
            b.epoch = 1
        else:
            b.epoch += 1
        self.done = True
        res = gemm_allgather(a, b.t, s.offset, tuple(s.shape), trans_b=trans_b, peer_slices=self._peer_slices(),
                             seg=b.seg, epoch=b.epoch, n_copy=m.fused.n_copy, add=add, out=out, only_b=only_b)
        if only_b:
            m._wait(m.compute_stream, self.rest_ready)     # the other weights of the unit are needed next
        else:
            m.bytes_gathered += (b.t.numel() - b.t.numel() // m.world_size) * 2
        return res

    def flush(self):
        if self.done:
            return
        m = self.mgr
        lo, hi = m.layout.unit_shard_range(self.uid)
        if self.region is not None:
            m.fused.all_gather(self.buf.t, m.param_shard_f16[lo:hi], m.compute_stream, only=self.region)
            m._wait(m.compute_stream, self.rest_ready)
        else:
            m.fused.all_gather(self.buf.t, m.param_shard_f16[lo:hi], m.compute_stream)
            m.bytes_gathered += (self.buf.t.numel() - self.buf.t.numel() // m.world_size) * 2
        self.done = True


class _Pool:
    """Reusable flat buffers keyed by size; zero-filled once so alignment gaps stay zero.

    ``rotate`` > 1 keeps that many buffers per size in rotation (first in, first out): a buffer
    handed back while a collective is still reading it is then not the next one to be written, so
    the producer of the next unit does not wait for that collective. The choice depends only on the
    call sequence, never on timing, so every rank allocates the same buffers in the same order
    (they live at equal offsets of the symmetric heap)."""

    def __init__(self, dtype, device, alloc=None, rotate: int = 1):
        self.dtype, self.device = dtype, device
        self.free = collections.defaultdict(list)
        self.alloc = alloc
        self.total_bytes = 0
        self.rotate = max(int(rotate), 1)
        self.made = collections.defaultdict(int)

    def get(self, n: int) -> _Buf:
        lst = self.free[n]
        if lst and self.made[n] >= self.rotate:
            return lst.pop(0) if self.rotate > 1 else lst.pop()
        self.made[n] += 1
        t = self.alloc(n, self.dtype) if self.alloc is not None else torch.zeros(n, dtype=self.dtype, device=self.device)
        self.total_bytes += t.numel() * t.element_size()
        b = _Buf(t)
        if t.is_cuda:
            # The block may have been handed back by a tensor of the allocating stream whose kernels are still
            # queued, and the zero fill itself runs on that stream: whoever uses the buffer first on ANOTHER
            # stream (the communication stream gathers into it) has to wait for this point, exactly as for a
            # buffer that comes back from a release.
            b.free_event = torch.cuda.Event()
            b.free_event.record(torch.cuda.current_stream(t.device))
        return b

    def put(self, b: _Buf):
        self.free[b.t.numel()].append(b)


class MemoryZeRO3Manager:
    enable_grad_bucket = True
    enable_param_prefetch = True
    enable_forward_param_prefetch = True
    enable_backward_param_prefetch = True

    def __init__(self, model, world_size: int, comm, rank: int, stream=None, *, accum_steps: int = 1,
                 replica_ratio: float = 0.0, replica_policy: str = "largest_first", fused=None,
                 profile_comm: bool = False):
        self.model = model
        self.world_size = int(world_size)
        self.comm = comm
        self.rank = int(rank)
        self.device = model.device
        self.dtype = model.dtype
        self.cuda = self.device.type == "cuda"
        self.accum_steps = int(accum_steps)
        self.replica_ratio = float(replica_ratio)
        self.replica_policy = replica_policy
        self.fused = fused
        self.profile_comm = profile_comm
        self.sync_after_each_microbatch = bool(getattr(model, "zero3_sync_after_each_microbatch", False))
        self.max_pending_reduces = int(getattr(model, "zero3_max_pending_reduces", 8))
        self.sync_gather = bool(getattr(model, "zero3_sync_gather", False))
        pf = bool(getattr(model, "zero3_param_prefetch", True)) and self.world_size > 1
        self.enable_param_prefetch = pf
        self.enable_forward_param_prefetch = pf and bool(getattr(model, "zero3_forward_param_prefetch", True))
        self.enable_backward_param_prefetch = pf and bool(getattr(model, "zero3_backward_param_prefetch", True))
        self.enable_grad_bucket = bool(getattr(model, "zero3_grad_bucket", True))
        # Largest number of elements one reduce-scatter launch takes (fused mode): a unit's gradient bucket that
        # is larger is reduced in parts of at most this size, and the part that is complete first (the MLP
        # weights of a block) goes out before the block's backward has finished.
        self.grad_bucket_elems = int(getattr(model, "grad_bucket_elems", 0) or 0)
        # Reduce the MLP part of a block's bucket as soon as its weight gradients are complete, i.e. while the
        # attention half of the block is still in backward. Off by default: the reduce-scatter CTAs then run
        # beside the attention-backward CTAs, whose registers leave no room for them on the same SM, and the
        # 1.3 B step at 2 GPUs measured 1.1 ms slower than with the whole bucket reduced at the block's end
        # (where the reduce-scatter overlaps the next block's MLP GEMMs, which do share their SMs).
        self.early_bucket_flush = bool(getattr(model, "zero3_early_bucket_flush", False))

        if self.cuda:
            self.compute_stream = stream if stream is not None else torch.cuda.current_stream(self.device)
            self.comm_stream = torch.cuda.Stream(device=self.device) if self.world_size > 1 else self.compute_stream
            # Parameter gathers that do not go through NCCL get a stream of their own: a prefetch then never
            # queues behind a gradient reduction (they touch different buffers and the gathers have no barrier
            # kernel). NCCL collectives stay on one stream: a communicator wants one issue order on every rank.
            own = (self.world_size > 1 and fused is not None and fused.gather
                   and bool(getattr(model, "zero3_gather_stream", True)))
            self.gather_stream = torch.cuda.Stream(device=self.device) if own else self.comm_stream
        else:
            self.compute_stream = self.comm_stream = self.gather_stream = None

        self._tag_model_param_indices()
        self._build_layout()
        if self.cuda and self.world_size > 1 and getattr(model, "keep_params_until_backward", False):
            # One multi-GPU run with this option never finished and its cause was not established; until it
            # is, the option is accepted on CPU ranks (where it is tested) and on a single GPU only.
            raise ValueError("keep_params_until_backward is not available on multi-GPU runs")
        if fused is not None:
            fused.reserve(self._heap_bytes_needed())
        # Gradients accumulate in fp32 across micro-batches (the reference accumulates in fp16,
        # model/ZeRO3.py:1396); with a single micro-batch the reduced bf16 gradient is used as is.
        self.grad_dtype = self.dtype if (self.accum_steps == 1) else torch.float32
        self.direct_grad = self.accum_steps == 1      # reduced gradients land in the shard as they are
        if fused is not None:      # peers pull parameter slices straight out of this buffer
            self.param_shard_f16 = fused.alloc(max(self.shard_size, 8), self.dtype)[:self.shard_size]
        else:
            self.param_shard_f16 = torch.zeros(max(self.shard_size, 1), dtype=self.dtype, device=self.device)[:self.shard_size]
        self.grad_shard_f16 = torch.zeros(max(self.shard_size, 1), dtype=self.grad_dtype, device=self.device)[:self.shard_size]
        self.live_param_to_idx = {}     # data_ptr of a live parameter view -> index in model.params
        self._replica_tmp = {}
        self._init_replica_buffers()
        self._initialize_param_shard_from_rank0()

        alloc = fused.alloc if fused is not None else None
        self.gather_pool = _Pool(self.dtype, self.device, None)
        self._params_ready_event = None   # recorded after the optimizer step; gathers wait on it
        self.unit_ready = {}              # uid -> event: this unit's shard slice has been updated (pipelined optimizer)
        self.grad_pool = _Pool(self.dtype, self.device, alloc, rotate=2 if world_size > 1 else 1)
        self.live = {}              # uid -> _Buf holding gathered parameters
        self.pending_gather = {}    # uid -> _Buf with an all-gather in flight
        self.deferred = {}          # uid -> _PendingGather (gather fused into the consuming GEMM)
        self.phase = "fwd"          # set by the model: which pass is asking for parameters
        self.fused_adam = None      # set per step by the trainer: {"opt", "lr", "grad_scale"}
        self.cur_grad = {}          # uid -> _Buf being written by backward
        self.pending_reduce_handles = collections.deque()
        self.exposed_pairs = []     # (event before wait, event after wait) on the compute stream
        self.bytes_gathered = 0
        self.bytes_reduced = 0
        self.micro_index = 0        # micro-batch inside the current optimizer step
        self._stats = torch.zeros(2, dtype=torch.float32, device=self.device)
        if self.cuda and self.world_size > 1:
            self._prewarm_pools()

    def _heap_bytes_needed(self) -> int:
        """Bytes of symmetric heap this manager allocates: the parameter shard, two gradient buckets per
        distinct unit size (see ``_Pool.rotate``), the replicated parameters and their gradient bucket
        (ZeRO-2.5), each with its guard blocks."""
        esz = 2
        sizes = sorted({u.padded for u in self.layout.units if not u.empty})
        total = max(self.shard_size, 8) * esz + sum(2 * n * esz for n in sizes)
        total += 2 * self.layout.replica_padded_total * esz
        return total + 1024 * (2 * len(sizes) + 4)

    def _prewarm_pools(self):
        """Create the pooled buffers the steady state needs before the first collective runs, so that no
        device allocation (a ``cudaMalloc`` inside the caching allocator, which can serialise with kernels
        that wait for a peer) happens while such kernels are in flight: per distinct unit size two gradient
        buckets (the rotation) and as many gather buffers as are live at once (two where several units
        share the size: the unit in use and the prefetched one)."""
        if self.fused is not None and getattr(self.fused, "reduce_mode", "pull") == "copy":
            # staging buffer of the copy-engine reduce-scatter: the largest share of one launch in a rank's slice
            W = self.world_size
            part = max([u.padded // W for u in self.layout.units if not u.empty] + [8])
            if self.grad_bucket_elems > 0 and self.early_bucket_flush:
                part = min(part, self.grad_bucket_elems // 8 * 8)
            part = max(part, self.layout.replica_padded_total // W)
            self.fused.reserve_stage(part)
        count = collections.Counter(u.padded for u in self.layout.units if not u.empty)
        for n in sorted(count):
            bufs = [self.grad_pool.get(n) for _ in range(self.grad_pool.rotate)]
            for b in bufs:
                self.grad_pool.put(b)
            bufs = [self.gather_pool.get(n) for _ in range(2 if count[n] > 1 else 1)]
            for b in bufs:
                self.gather_pool.put(b)

    # ------------------------------------------------------------------ layout
    def _tag_model_param_indices(self):
        self.unit_modules = self.model.unit_modules()
        self.unit_names = [n for n, _ in self.model.unit_defs()]
        self.uid_of_name = {n: i for i, n in enumerate(self.unit_names)}
        self.uid_of_module = {}
        for name, ent in self.unit_modules.items():
            uid = self.uid_of_name[name]
            for mod, j, idx in ent:
                if mod is self.model:
                    continue
                self.uid_of_module[id(mod)] = uid
                lst = getattr(mod, "_zero3_param_indices", None)
                if lst is None or len(lst) != len(mod.params):
                    mod._zero3_param_indices = [None] * len(mod.params)
                mod._zero3_param_indices[j] = idx

    def _build_layout(self):
        shapes = [tuple(p.shape) for p in self.model.params]
        sizes = [int(p.numel()) for p in self.model.params]
        emb_idx = [idx for (_, _, idx) in self.unit_modules["embedding"]]
        rep = select_replicated_params(sizes, emb_idx, self.replica_ratio, self.replica_policy)
        self.layout = FlatLayout.build(shapes, self.model.unit_defs(), self.world_size, rep)
        self.shard_size = self.layout.shard_size
        self.padded_total = self.layout.padded_total
        d = self.layout.describe()
        self.param_offsets, self.param_shapes, self.param_sizes = d["param_offsets"], d["param_shapes"], d["param_sizes"]
        self.replicated_param_indices = list(rep)
        self.replica_total = self.layout.replica_total
        self.replica_padded_total = self.layout.replica_padded_total
        self.replica_opt_shard_size = self.layout.replica_opt_shard_size

    def _init_replica_buffers(self):
        n = self.replica_padded_total
        gdt = torch.float32 if self.accum_steps > 1 else self.dtype
        self._replica_bucket = None         # bf16 heap copy of an fp32 replica gradient (fused reduce-scatter input)
        self._replica_shard_buf = None      # reduced slice the replica optimizer reads (allocated once)
        self._replica_stats_fused = False
        if n and self.fused is not None and self.world_size > 1:
            # peers pull the updated slices / the gradient slices straight out of these buffers
            self.replica_param_f16 = self.fused.alloc(n, self.dtype)
            bucket = self.fused.alloc(n, self.dtype)
            if gdt == self.dtype:
                self.replica_grad_f16 = bucket
            else:
                self.replica_grad_f16 = torch.zeros(n, dtype=gdt, device=self.device)
                self._replica_bucket = bucket
        else:
            self.replica_param_f16 = torch.zeros(n, dtype=self.dtype, device=self.device) if n else None
            self.replica_grad_f16 = torch.zeros(n, dtype=gdt, device=self.device) if n else None
        self.replica_grad_shard = None
        self.replica_views = {}
        self.replica_grad_views = {}
        for i in self.replicated_param_indices:
            s = self.layout.slots[i]
            self.replica_views[i] = self.replica_param_f16[s.offset:s.offset + s.size].view(s.shape)
            self.replica_grad_views[i] = self.replica_grad_f16[s.offset:s.offset + s.size].view(s.shape)
            self.live_param_to_idx[self.replica_views[i].data_ptr()] = i

    def _initialize_param_shard_from_rank0(self):
        """Pack the model's freshly built parameters unit by unit, take rank 0's values
        (model/ZeRO3.py:1674-1707 does this one parameter and one host sync at a time), keep this
        rank's slice, then detach the full parameters from the model."""
        params = self.model.params
        W = self.world_size
        for uid, unit in enumerate(self.layout.units):
            if unit.empty:
                continue
            buf = torch.zeros(unit.padded, dtype=self.dtype, device=self.device)
            for i in unit.param_indices:
                s = self.layout.slots[i]
                if s.unit == uid:
                    buf[s.offset:s.offset + s.size].copy_(params[i].reshape(-1))
            if W > 1:
                self.comm.broadcast(buf, src=0)
            lo, hi = self.layout.unit_shard_range(uid)
            sl = unit.padded // W
            self.param_shard_f16[lo:hi].copy_(buf[self.rank * sl:(self.rank + 1) * sl])
            del buf
        if self.replica_param_f16 is not None:
            for i in self.replicated_param_indices:
                self.replica_views[i].copy_(params[i])
            if W > 1:
                self.comm.broadcast(self.replica_param_f16, src=0)
        new = [self.replica_views.get(i) for i in range(len(params))]
        self.model.link_params(new)
        if self.cuda:
            torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ stream helpers
    def _record(self, stream, timing: bool = False):
        if not self.cuda:
            return None
        ev = torch.cuda.Event(enable_timing=timing)
        ev.record(stream)
        return ev

    def _wait(self, stream, ev):
        if self.cuda and ev is not None:
            stream.wait_event(ev)

    def _comm_ctx(self):
        if self.cuda and self.comm_stream is not self.compute_stream:
            return torch.cuda.stream(self.comm_stream)
        return _NullCtx()

    def _gather_ctx(self):
        if self.cuda and self.gather_stream is not self.compute_stream:
            return torch.cuda.stream(self.gather_stream)
        return _NullCtx()

    # ------------------------------------------------------------------ parameter gather
    def _unit_ids(self, modules):
        seen, out = set(), []
        for m in modules:
            uid = self.uid_of_module[id(m)]
            if uid not in seen:
                seen.add(uid)
                out.append(uid)
        return out

    def _start_gather(self, uid: int, tag=None):
        if uid in self.live or uid in self.pending_gather:
            return
        unit = self.layout.units[uid]
        if unit.empty:
            return
        lo, hi = self.layout.unit_shard_range(uid)
        if self.world_size == 1:
            b = _Buf(self.param_shard_f16[lo:hi])
            b.uid = uid
            b.ready_event = self.unit_ready.get(uid)     # set while the optimizer of the last step is still running
            self.pending_gather[uid] = b
            return
        b = self.gather_pool.get(unit.padded)
        b.uid = uid
        if self._fuse_gather_into_gemm(uid):
            # The first GEMM that consumes the unit pulls the chunks that hold ITS weight while it runs;
            # everything else of the unit is pulled now, on the communication stream.
            from ..ops.gemm import ag_region
            ready = self.unit_ready.get(uid, self._params_ready_event)
            self._wait(self.compute_stream, b.free_event)
            self._wait(self.compute_stream, ready)
            pidx = self._first_weight_index(uid)
            region = rest_ready = None
            if pidx is not None:
                slot = self.layout.slots[pidx]
                esz = b.t.element_size()
                region = ag_region((unit.padded // self.world_size) * esz, self.world_size, slot.offset * esz,
                                   slot.size * esz)
                with self._gather_ctx():
                    self._wait(self.gather_stream, b.free_event)
                    self._wait(self.gather_stream, ready)
                    self.fused.all_gather(b.t, self.param_shard_f16[lo:hi], self.gather_stream, skip=region)
                    rest_ready = self._record(self.gather_stream)
                self.bytes_gathered += (unit.padded - unit.padded // self.world_size) * esz
            b.ready_event = None
            self.pending_gather[uid] = b
            self.deferred[uid] = _PendingGather(self, uid, b, pidx, region, rest_ready)
            return
        with self._gather_ctx():
            self._wait(self.gather_stream, b.free_event)
            self._wait(self.gather_stream, self.unit_ready.get(uid, self._params_ready_event))
            if self.fused is not None and self.fused.gather:
                self.fused.all_gather(b.t, self.param_shard_f16[lo:hi], self.gather_stream)
            else:
                self.comm.all_gather_into(b.t, self.param_shard_f16[lo:hi])
            b.ready_event = self._record(self.gather_stream)
        self.bytes_gathered += (unit.padded - unit.padded // self.world_size) * b.t.element_size()
        self.pending_gather[uid] = b
        if self.sync_gather and self.cuda:
            self.gather_stream.synchronize()

    def _finish_gather(self, uid: int):
        if uid in self.live:
            return self.live[uid]
        b = self.pending_gather.pop(uid, None)
        if b is None:
            self._start_gather(uid)
            b = self.pending_gather.pop(uid, None)
            if b is None:          # unit with no sharded parameters (all replicated)
                return None
        if b.ready_event is not None:
            if self.profile_comm:
                e0 = self._record(self.compute_stream, True)
                self._wait(self.compute_stream, b.ready_event)
                self.exposed_pairs.append((e0, self._record(self.compute_stream, True)))
            else:
                self._wait(self.compute_stream, b.ready_event)
        self.live[uid] = b
        self._attach(uid, b.t)
        pg = self.deferred.get(uid)
        if pg is not None:
            consumer = self._first_consumer(uid)
            if consumer is None:
                pg.flush()
                del self.deferred[uid]
            else:
                consumer.pending_gather = pg
        return b

    def _attach(self, uid: int, buf: torch.Tensor):
        name = self.unit_names[uid]
        for mod, j, idx in self.unit_modules[name]:
            s = self.layout.slots[idx]
            if s.unit != uid:
                continue
            view = buf[s.offset:s.offset + s.size].view(s.shape)
            if mod is self.model:
                getattr(self.model, j)[0] = view
            else:
                mod.params[j] = view
            self.model.params[idx] = view
            self.live_param_to_idx[view.data_ptr()] = idx

    def _detach(self, uid: int):
        name = self.unit_names[uid]
        for mod, j, idx in self.unit_modules[name]:
            if self.layout.slots[idx].unit != uid:
                continue
            old = self.model.params[idx]
            if old is not None:
                self.live_param_to_idx.pop(old.data_ptr(), None)
            if mod is self.model:
                getattr(self.model, j)[0] = None
            else:
                mod.params[j] = None
            self.model.params[idx] = None

    def _fuse_gather_into_gemm(self, uid: int) -> bool:
        return (self.fused is not None and self.fused.gather and getattr(self.fused, "gemm_fusion", False)
                and self.world_size > 1 and self.unit_names[uid].startswith("block"))

    def _first_consumer(self, uid: int):
        """The layer whose first GEMM reads this unit: the attention projection in forward, the MLP
        (its down-projection dgrad) in backward."""
        mods = [m for (m, _, _) in self.unit_modules[self.unit_names[uid]]]
        want = "SwiGLU" if self.phase == "bwd" else "GroupedQueryAttention"
        for m in mods:
            if type(m).__name__ == want:
                return m
        return None

    def _first_weight_index(self, uid: int):
        """Global parameter index of the weight that the first GEMM on this unit reads: W_KQV of the
        attention in the forward pass, the down projection of the MLP in the backward pass."""
        consumer = self._first_consumer(uid)
        if consumer is None:
            return None
        want = 1 if self.phase == "bwd" else 0
        for mod, j, idx in self.unit_modules[self.unit_names[uid]]:
            if mod is consumer and j == want and self.layout.slots[idx].unit == uid:
                return idx
        return None

    def ensure_gathered(self, module):
        """Called by a layer that is about to read its parameters outside the fused GEMM."""
        pg = getattr(module, "pending_gather", None)
        if pg is not None:
            pg.flush()
            module.pending_gather = None
            self.deferred.pop(pg.uid, None)

    def _release_unit(self, uid: int):
        b = self.live.pop(uid, None)
        if b is None:
            return
        pg = self.deferred.pop(uid, None)
        if pg is not None and not pg.done:
            raise RuntimeError(f"unit {self.unit_names[uid]} was released before its fused gather ran")
        self._detach(uid)
        if self.world_size > 1:
            b.free_event = self._record(self.compute_stream)
            b.ready_event = None
            self.gather_pool.put(b)

    def prefetch_modules(self, modules, tag=None):
        for uid in self._unit_ids(modules):
            self._start_gather(uid, tag)

    def wait_modules(self, modules):
        for uid in self._unit_ids(modules):
            self._finish_gather(uid)

    def gather_modules(self, modules):
        self.prefetch_modules(modules)
        self.wait_modules(modules)

    def gather_module(self, module):
        self.gather_modules([module])

    def release_modules(self, modules):
        for uid in self._unit_ids(modules):
            self._release_unit(uid)

    def release_module(self, module):
        self.release_modules([module])

    # embedding / LM head ---------------------------------------------------------------------
    def _gather_named(self, name: str):
        uid = self.uid_of_name[name]
        idx = self.unit_modules[name][0][2]
        if idx in self.replica_views:
            return self.replica_views[idx]
        b = self._finish_gather(uid)
        s = self.layout.slots[idx]
        return b.t[s.offset:s.offset + s.size].view(s.shape)

    def gather_embedding(self):
        return self._gather_named("embedding")

    def get_live_embedding(self):
        uid = self.uid_of_name["embedding"]
        idx = self.unit_modules["embedding"][0][2]
        if idx in self.replica_views:
            return self.replica_views[idx]
        if uid in self.live:
            return self._gather_named("embedding")
        return None

    def gather_head(self):
        return self._gather_named("embedding" if self.model.tie_embeddings else "lm_head")

    def release_embedding(self):
        self._release_unit(self.uid_of_name["embedding"])
        if not self.model.tie_embeddings:
            self._release_unit(self.uid_of_name["lm_head"])

    # ------------------------------------------------------------------ gradients
    def _grad_buf(self, uid: int) -> _Buf:
        b = self.cur_grad.get(uid)
        if b is not None:
            return b
        unit = self.layout.units[uid]
        if self.world_size == 1 and self.direct_grad:
            lo, hi = self.layout.unit_shard_range(uid)
            b = _Buf(self.grad_shard_f16[lo:hi])     # GEMMs write the shard itself
        else:
            b = self.grad_pool.get(unit.padded)
            self._wait(self.compute_stream, b.free_event)
        b.uid = uid
        b.flushed = []
        self.cur_grad[uid] = b
        return b

    def begin_grad_bucket(self, tag=None, modules=None):
        if modules:
            for uid in self._unit_ids(modules):
                if not self.layout.units[uid].empty:
                    self._grad_buf(uid)

    def grad_views(self, module):
        """Views of the current gradient bucket for each parameter of ``module`` (None for a
        replicated parameter, whose gradient is accumulated locally instead)."""
        uid = self.uid_of_module[id(module)]
        out = []
        for idx in module._zero3_param_indices:
            s = self.layout.slots[idx]
            if s.unit < 0:
                out.append(None)
            else:
                b = self._grad_buf(uid)
                out.append(b.t[s.offset:s.offset + s.size].view(s.shape))
        return out

    def add_grads_to_bucket(self, params, grads, module=None):
        """Gradients already written in place need nothing; others (replicated parameters, or
        layers that allocated their own) are copied / accumulated here."""
        for p, g in zip(params, grads):
            if g is None:
                continue
            idx = self._param_index_of(p)
            if idx is None:
                continue
            s = self.layout.slots[idx]
            if s.unit < 0:
                dst = self.replica_grad_views[idx]
                if self.micro_index == 0:
                    dst.copy_(g)
                else:
                    dst.add_(g.to(dst.dtype))
                continue
            b = self._grad_buf(s.unit)
            view = b.t[s.offset:s.offset + s.size].view(s.shape)
            if view.data_ptr() != g.data_ptr():
                view.copy_(g)

    accumulate_grads = add_grads_to_bucket

    def _param_index_of(self, p):
        if p is None:
            return None
        return self.live_param_to_idx.get(p.data_ptr())

    def _flush_unit(self, uid: int, tag=None):
        b = self.cur_grad.pop(uid, None)
        if b is None:
            return
        unit = self.layout.units[uid]
        lo, hi = self.layout.unit_shard_range(uid)
        dst = self.grad_shard_f16[lo:hi]
        if self.world_size == 1 and self.direct_grad:
            return                                   # written in place
        done_on = self.compute_stream
        if self.world_size == 1:
            F.accumulate(dst, b.t, 1.0)
        else:
            ev = self._record(self.compute_stream)
            with self._comm_ctx():
                self._wait(self.comm_stream, ev)
                if self.fused is not None:
                    early = sum(e - a for a, e in b.flushed)
                    for rng in self._unflushed_parts(b, unit.padded):
                        self._fused_reduce(b, dst, lo, hi, rng)
                    self.bytes_reduced -= early * (self.world_size - 1) // self.world_size * b.t.element_size()
                elif self.direct_grad:
                    self.comm.reduce_scatter(dst, b.t)
                else:
                    tmp = torch.empty(unit.padded // self.world_size, dtype=self.dtype, device=self.device)
                    self.comm.reduce_scatter(tmp, b.t)
                    F.accumulate(dst, tmp, 1.0)
                    if self.cuda:
                        tmp.record_stream(self.comm_stream)
            done_on = self.comm_stream
            self.bytes_reduced += (unit.padded - unit.padded // self.world_size) * b.t.element_size()
        b.free_event = self._record(done_on)
        self.pending_reduce_handles.append((b.free_event, tag))
        self.grad_pool.put(b)

    def _fused_reduce(self, b: _Buf, dst, lo: int, hi: int, elem_range):
        """One launch of the fused reduce-scatter on the communication stream for ``elem_range`` of bucket ``b``
        (shard range [lo, hi) of its unit)."""
        adam = None
        if self.fused_adam is not None and self.micro_index == self.accum_steps - 1 and self.direct_grad:
            # reduce-scatter -> cast -> scale -> AdamW in ONE kernel: the reduced gradient
            # of this unit never goes to memory, the parameter slice is updated in place
            fa, opt = self.fused_adam, self.fused_adam["opt"]
            adam = dict(m=opt.m[lo:hi], v=opt.v[lo:hi], master=opt.master_weight_shard[lo:hi],
                        param=self.param_shard_f16[lo:hi], lr=fa["lr"], beta1=opt.beta1, beta2=opt.beta2,
                        eps=opt.epsilon, weight_decay=opt.weight_decay,
                        m_corr=1.0 / (1.0 - opt.beta1 ** opt.t), v_corr=1.0 / (1.0 - opt.beta2 ** opt.t),
                        grad_scale=fa["grad_scale"])
        self.fused.reduce_scatter_accumulate(dst, b.t, accumulate=not self.direct_grad, stream=self.comm_stream,
                                             stats=self._stats, do_stats=self.micro_index == self.accum_steps - 1,
                                             adam=adam, elem_range=elem_range)

    def _split_range(self, lo: int, hi: int):
        """[lo, hi) cut into parts of at most ``grad_bucket_elems`` elements (multiples of 8). Not cut for the
        copy-engine reduce-scatter unless parts are flushed early: an element range covers only some ranks'
        slices, so every part would keep the other ranks idle between its two cross-GPU barriers (at 4 GPUs
        the three parts of the embedding unit ran one rank group after the other and the wait for the last
        bucket grew to 1.7 ms)."""
        step = self.grad_bucket_elems // 8 * 8 if self.grad_bucket_elems > 0 else 0
        if getattr(self.fused, "reduce_mode", "pull") == "copy" and not self.early_bucket_flush:
            step = 0
        if step <= 0 or hi - lo <= step:
            return [(lo, hi)] if hi > lo else []
        return [(a, min(a + step, hi)) for a in range(lo, hi, step)]

    def _unflushed_parts(self, b: _Buf, padded: int):
        """Element ranges of bucket ``b`` that have not been reduced yet, cut to the bucket limit."""
        parts, pos = [], 0
        for lo, hi in sorted(b.flushed):
            parts += self._split_range(pos, lo)
            pos = max(pos, hi)
        return parts + self._split_range(pos, padded)

    def flush_grad_ranges_async(self, modules, tag=None):
        """Reduce the gradients of ``modules``' weights now, ahead of the rest of their unit's bucket (fused
        collectives only; with NCCL, and for units within the bucket limit, the unit is reduced whole at the
        end of its backward). The model calls this when a block's MLP backward has been issued: its
        weight-gradient GEMMs run on the side stream, so the launch waits for that stream's event and for the
        compute stream, not for the whole block."""
        if self.fused is None or self.world_size == 1 or self.grad_bucket_elems <= 0 or not self.early_bucket_flush:
            return
        for uid in self._unit_ids(modules):
            b = self.cur_grad.get(uid)
            unit = self.layout.units[uid]
            if b is None or unit.padded <= self.grad_bucket_elems:
                continue
            lo_e, hi_e = None, None
            for m in modules:
                if self.uid_of_module.get(id(m)) != uid:
                    continue
                for idx in m._zero3_param_indices:
                    s = self.layout.slots[idx]
                    if s.unit != uid:
                        continue
                    a, e = s.offset // 8 * 8, (s.offset + s.size + 7) // 8 * 8
                    lo_e = a if lo_e is None else min(lo_e, a)
                    hi_e = e if hi_e is None else max(hi_e, e)
            if lo_e is None:
                continue
            # the range must hold nothing but these modules' parameters (they are laid out back to back)
            inside = [s for s in self.layout.slots if s.unit == uid and s.offset < hi_e and s.offset + s.size > lo_e]
            owned = {idx for m in modules for idx in m._zero3_param_indices}
            if any(s.index not in owned for s in inside):
                continue
            lo, hi = self.layout.unit_shard_range(uid)
            dst = self.grad_shard_f16[lo:hi]
            ev = self._record(self.compute_stream)
            wev = F.wgrad_event(self.device)
            with self._comm_ctx():
                self._wait(self.comm_stream, ev)
                self._wait(self.comm_stream, wev)
                for rng in self._split_range(lo_e, hi_e):
                    self._fused_reduce(b, dst, lo, hi, rng)
            b.flushed.append((lo_e, hi_e))
            self.bytes_reduced += (hi_e - lo_e) * (self.world_size - 1) // self.world_size * b.t.element_size()

    def flush_grad_bucket_async(self, tag=None):
        for uid in [u for u in list(self.cur_grad) if self.unit_names[u].startswith(("block", "final_norm"))]:
            self._flush_unit(uid, tag)

    def embedding_grad_view(self, which: str = "embedding"):
        name = "embedding" if which == "embedding" else "lm_head"
        idx = self.unit_modules[name][0][2]
        s = self.layout.slots[idx]
        if s.unit < 0:
            # replicated table: this micro-batch's gradient is built in a scratch tensor and
            # folded into the locally accumulated replica gradient at flush time
            tmp = self._replica_tmp.get(idx)
            if tmp is None:
                tmp = self._replica_tmp[idx] = torch.zeros(s.shape, dtype=self.dtype, device=self.device)
            return tmp
        b = self._grad_buf(s.unit)
        return b.t[s.offset:s.offset + s.size].view(s.shape)

    def flush_embedding_grad_bucket_async(self, tag=None):
        names = ["embedding", "lm_head"] if tag in (None, "embedding") else [tag]
        for name in names:
            uid = self.uid_of_name.get(name)
            if uid is None:
                continue
            idx = self.unit_modules[name][0][2]
            tmp = self._replica_tmp.pop(idx, None)
            if tmp is not None:
                dst = self.replica_grad_views[idx]
                if self.micro_index == 0:
                    dst.copy_(tmp)
                else:
                    dst.add_(tmp.to(dst.dtype))
            self._flush_unit(uid, tag)

    def accumulate_grad_slice(self, param, row_s, row_e, chunk):
        """Write rows [row_s, row_e) of the gradient of an embedding-like parameter."""
        which = "embedding"
        if not self.model.tie_embeddings and param is not None and self.model.head_para is not None \
                and self.model.head_para[0] is not None and param.data_ptr() == self.model.head_para[0].data_ptr():
            which = "lm_head"
        self.embedding_grad_view(which)[row_s:row_e].copy_(chunk)

    accumulate_grad_slice_bucketed = accumulate_grad_slice

    def accumulate_embedding_grads_chunked(self, param, idx, dout, padding_id, vocab_chunk_size=None):
        """Input-embedding gradient: scatter-add token rows into the dense table gradient. Every
        rank owns a full-size bucket for the unit, so the ranks need not agree on which vocab
        chunks are present (the reference needs an all-reduced bitmap and a host sync for that,
        model/ZeRO3.py:1558-1600)."""
        F.embedding_bwd(self.embedding_grad_view("embedding"), idx.reshape(-1).to(torch.int32), dout, padding_id)

    def flush_buckets(self):
        for uid in list(self.cur_grad):
            self._flush_unit(uid, "flush")

    def progress_async_reduces(self, max_pending: int = 8, force: bool = False):
        q = self.pending_reduce_handles
        while q and (q[0][0] is None or q[0][0].query()):
            q.popleft()
        limit = 0 if force else max_pending
        while len(q) > limit:
            ev, _ = q.popleft()
            if ev is not None:
                ev.synchronize()

    def synchronize(self):
        self.flush_buckets()
        self.progress_async_reduces(force=True)
        if self.cuda:
            if self.comm_stream is not self.compute_stream:
                self.compute_stream.wait_stream(self.comm_stream)
            if self.gather_stream is not self.compute_stream and self.gather_stream is not self.comm_stream:
                self.compute_stream.wait_stream(self.gather_stream)
            self.compute_stream.synchronize()

    def end_microbatch(self):
        """Order the compute stream after this micro-batch's reductions (no host block)."""
        self.flush_buckets()
        self.progress_async_reduces(self.max_pending_reduces)
        self.micro_index += 1
        if self.sync_after_each_microbatch:
            self.synchronize()

    def wait_reductions(self):
        """Make the compute stream wait for every gradient reduction issued so far (device-side
        ordering only). Called before the statistics / optimizer kernels read the shard."""
        self.flush_buckets()
        if self.cuda and self.comm_stream is not self.compute_stream:
            if self.profile_comm:
                e0 = self._record(self.compute_stream, True)
                self.compute_stream.wait_stream(self.comm_stream)
                self.exposed_pairs.append((e0, self._record(self.compute_stream, True)))
            else:
                self.compute_stream.wait_stream(self.comm_stream)

    def zero_grad(self):
        self.progress_async_reduces(force=True)
        self.micro_index = 0
        if self.fused is not None:
            self._stats.zero_()       # the fused reduce kernels add this step's statistics into it
        if not self.direct_grad:
            self.grad_shard_f16.zero_()
        if self.replica_grad_shard is not None:
            self.replica_grad_shard = None

    # ------------------------------------------------------------------ step boundary
    def calculate_global_grad_stats(self, to_host: bool = True):
        """(sum of squares of the global gradient, non-finite flag). One fused pass over the shard,
        one 2-float all-reduce (model/ZeRO3.py:1602-1648). Also leaves the device tensor in
        ``self.grad_stats_device`` for the optimizer's on-device clip / skip."""
        self.wait_reductions()
        st = self._stats
        if self.fused is None or self.world_size == 1:
            st.zero_()
            F.grad_stats(self.grad_shard_f16, st)
        if self.replica_grad_shard is not None and not self._replica_stats_fused:
            F.grad_stats(self.replica_grad_shard, st)
        if self.world_size > 1:
            self.comm.all_reduce(st)
        self.grad_stats_device = st
        if not to_host:
            return st
        vals = st.tolist()
        return float(vals[0]), bool(vals[1] != 0.0)

    def check_nan_inf(self) -> bool:
        return self.calculate_global_grad_stats()[1]

    def calculate_global_grad_norm(self) -> float:
        return self.calculate_global_grad_stats()[0] ** 0.5

    def calculate_global_param_norm(self) -> float:
        st = torch.zeros(2, dtype=torch.float32, device=self.device)
        F.grad_stats(self.param_shard_f16, st)
        if self.replica_param_f16 is not None and self.rank == 0:
            F.grad_stats(self.replica_param_f16, st)
        if self.world_size > 1:
            self.comm.all_reduce(st)
        return float(st[0]) ** 0.5

    def forward_unit_order(self):
        """Unit ids in the order the forward pass first needs them (embedding, blocks, final norm,
        head): the order in which a pipelined optimizer should finish them."""
        def key(uid):
            name = self.unit_names[uid]
            if name == "embedding":
                return (0, 0)
            if name.startswith("block"):
                digits = "".join(ch for ch in name if ch.isdigit())
                return (1, int(digits) if digits else 0)
            if name.startswith("final_norm"):
                return (2, 0)
            return (3, uid)
        return sorted((u for u in range(len(self.layout.units)) if not self.layout.units[u].empty), key=key)

    def after_optimizer_step(self, pipelined: bool = False):
        """Order the next gathers after the parameter update: locally with an event the comm stream
        waits on, and across GPUs (fused mode, where peers read this shard directly) with a
        device-side barrier. ``pipelined``: the optimizer has recorded one event per unit in
        ``unit_ready`` (and issued its own barriers), so there is nothing global to wait for."""
        if pipelined:
            return
        self.unit_ready = {}
        if not self.cuda or self.world_size == 1:
            return
        if self.fused is not None:
            self.fused.barrier(self.compute_stream, channel=3)
        self._params_ready_event = self._record(self.compute_stream)

    def get_param_shard_view(self):
        return self.param_shard_f16

    def set_param_shard(self, new_shard):
        if new_shard.data_ptr() != self.param_shard_f16.data_ptr():
            self.param_shard_f16.copy_(new_shard)

    # ------------------------------------------------------------------ ZeRO-2.5 replica handling
    def get_replica_optimizer_shard_view(self):
        if self.replica_param_f16 is None:
            return None
        n = self.replica_opt_shard_size
        return self.replica_param_f16[self.rank * n:(self.rank + 1) * n]

    def set_replica_optimizer_shard(self, new_shard):
        v = self.get_replica_optimizer_shard_view()
        if v is not None and new_shard.data_ptr() != v.data_ptr():
            v.copy_(new_shard)

    def prepare_replicated_grads_for_sharded_optimizer(self):
        """Reduce-scatter the locally accumulated replica gradients so each rank holds the summed
        slice its replica optimizer owns (the reference all-reduces the whole buffer and slices,
        model/ZeRO2_5.py:1240-1265). Call it BEFORE ``calculate_global_grad_stats``: the slices join
        the same global norm - in fused mode the reduce-scatter kernel adds their sum of squares and
        non-finite flag to the statistics itself, otherwise the statistics pass reads the slice."""
        if self.replica_grad_f16 is None:
            return None
        n = self.replica_opt_shard_size
        if self._replica_shard_buf is None:
            self._replica_shard_buf = torch.empty(n, dtype=self.replica_grad_f16.dtype, device=self.device)
        out = self._replica_shard_buf
        self._replica_stats_fused = False
        if self.world_size == 1:
            out.copy_(self.replica_grad_f16[:n])
        elif self.fused is not None:
            bucket = self.replica_grad_f16
            if self._replica_bucket is not None:
                self._replica_bucket.copy_(self.replica_grad_f16)        # fp32 accumulation -> bf16 bucket
                bucket = self._replica_bucket
            # On the communication stream, behind the unit reductions: two reduce-scatter kernels must never be
            # in flight at once, they share the barrier flags (a later epoch written into a flag an earlier
            # kernel still waits on, then overwritten by the peer's earlier epoch, leaves the later one waiting).
            ev = self._record(self.compute_stream)
            with self._comm_ctx():
                self._wait(self.comm_stream, ev)
                self.fused.reduce_scatter_accumulate(out, bucket, accumulate=False, stream=self.comm_stream,
                                                     stats=self._stats, do_stats=True)
            self._wait(self.compute_stream, self._record(self.comm_stream))
            self._replica_stats_fused = True
            self.bytes_reduced += (bucket.numel() - n) * bucket.element_size()
        else:
            self.comm.reduce_scatter(out, self.replica_grad_f16)
        self.replica_grad_shard = out
        return out

    def allgather_replicated_params_from_optimizer_shards(self):
        """Rebuild the full replica from the slices the replica optimizers just updated
        (model/ZeRO2_5.py:1272-1291), in place: every rank's slice already sits at its position."""
        if self.replica_param_f16 is None or self.world_size == 1:
            return
        mine = self.get_replica_optimizer_shard_view()
        if self.fused is not None and self.fused.gather:
            # every rank has finished writing its slice (channel 3: the optimizer's stream may have its own
            # per-unit barriers in flight on channel 1 at this moment)
            self.fused.barrier(self.compute_stream, channel=3)
            self.fused.all_gather(self.replica_param_f16, mine, self.compute_stream)
        elif getattr(self.comm, "backend", "") == "gloo":
            self.comm.all_gather_into(self.replica_param_f16, mine.clone())
        else:
            self.comm.all_gather_into(self.replica_param_f16, mine)
        self.bytes_gathered += (self.replica_param_f16.numel() - mine.numel()) * mine.element_size()

    # ------------------------------------------------------------------ accounting
    def exposed_comm_ms(self, reset: bool = True) -> float:
        """Time the compute stream spent blocked on gathers since the last call (needs
        ``profile_comm``; synchronises)."""
        if not self.cuda:
            return 0.0
        torch.cuda.synchronize(self.device)
        total = sum(a.elapsed_time(b) for a, b in self.exposed_pairs)
        if reset:
            self.exposed_pairs = []
        return total

    def materialize_all(self):
        """Gather every unit and keep it attached (inference / generation / export on a model that
        is managed by this object). Free with ``release_all``."""
        for uid in range(len(self.layout.units)):
            self._finish_gather(uid)

    def release_all(self):
        for uid in list(self.live):
            self._release_unit(uid)

    def memory_summary(self) -> dict:
        return {"shard_elems": self.shard_size, "gather_pool_bytes": self.gather_pool.total_bytes,
                "grad_pool_bytes": self.grad_pool.total_bytes, "replica_elems": self.replica_padded_total}


class MemoryZeRO2_5Manager(MemoryZeRO3Manager):
    """ZeRO-2.5: ``replica_ratio`` of the parameter elements (chosen by ``replica_policy``) stay
    replicated on every rank — no gather in forward/backward — while their gradients are
    reduce-scattered and their optimizer state sharded at the step boundary; the remaining
    parameters are handled exactly as in ZeRO-3. ``replica_ratio = 1`` is ZeRO-2."""

    def __init__(self, model, world_size, comm, rank, stream=None, *, replica_ratio=None, replica_policy=None, **kw):
        if replica_ratio is None:
            replica_ratio = float(model.model_dic.get("zero25_replica_ratio", 0.0))
        if replica_policy is None:
            replica_policy = str(model.model_dic.get("zero25_replica_policy", "largest_first"))
        super().__init__(model, world_size, comm, rank, stream, replica_ratio=replica_ratio,
                         replica_policy=replica_policy, **kw)


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
