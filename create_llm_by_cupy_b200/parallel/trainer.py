"""Per-rank training engine, the worker loop and the multi-process launcher.

Counterparts in the reference: ``TrainMultiGPU`` (model/ZeRO3.py:653-726, model/ZeRO2_5.py:694-771),
the worker ``training_worker_nccl_stream`` (model/ZeRO3.py:97-501, model/ZeRO2_5.py:95-542). The
duplicated ZeRO-3 / ZeRO-2.5 halves of the reference are one implementation here, selected by
``zero_stage``; the launcher adds what the reference lacks: a watchdog (child exit codes and
per-rank heartbeats, first failure tears the job down instead of leaving ranks blocked in a
collective), data partitioned across ranks, working validation, resume, and tokens/s accounting.
"""
from __future__ import annotations

import math
import os
import time
import traceback

import numpy as np
import torch

from ..models.model import Cupa_ver4
from ..optim.optimizer import ZeRO_Adam_Offload, ZeRO_Adam_ShardedGPU
from ..utils import checkpoint as ckpt
from ..utils.data import BatchStager, SplitDataset, get_batch, shard_for_rank, to_fixed_length
from ..utils.functions import ScaleGrad, print_memory_status
from ..utils.logging import MetricsLogger
from ..utils.profiler import nvtx_range
from .comm import SingleProcessComm, init_distributed, shutdown_distributed
from .zero import MemoryZeRO2_5Manager, MemoryZeRO3Manager


class Trainer:
    """One rank of a ZeRO-3 / ZeRO-2.5 data-parallel job: model + manager + optimizer(s).

    ``train_step(batches)`` runs ``len(batches)`` micro-batches (forward, backward, gradient
    reduction overlapped with backward), then the global-norm clip, the non-finite check and the
    AdamW update of this rank's shard, and returns host scalars.
    """

    def __init__(self, model_dic: dict, *, rank: int = 0, world_size: int = 1, comm=None, device=None,
                 zero_stage: str = "3", optimizer_device: str = "gpu", accum_step: int = 1,
                 lr_max: float = 3e-4, lr_mini: float = 3e-5, weight_decay: float = 0.1, warm_up: int = 100,
                 total_steps: int = 1000, beta1: float = 0.9, beta2: float = 0.99, epsilon: float = 1e-6,
                 max_grads: float = 1.0, GradScale_dic: dict | None = None, logger=None, fused=None,
                 profile_comm: bool = False, param_path: str | None = None, fused_adam: bool = False,
                 profile_phases: bool = False, adam_overlap: bool = True, cuda_graph: bool = False,
                 defer_host_read: bool = False, adam_overlap_ctas_per_sm: int = 2,
                 offload_delayed_update: bool = False):
        self.rank, self.world_size = rank, world_size
        self.profile_phases = bool(profile_phases)
        self._phase_marks = []
        self.comm = comm if comm is not None else SingleProcessComm()
        self.accum_step = int(accum_step)
        self.max_grads = float(max_grads)
        self.logger = logger
        self.model = Cupa_ver4(model_dic, param_path=param_path, device=device)
        self.device = self.model.device
        self.n_params = self.model.param_count()
        mgr_cls = MemoryZeRO2_5Manager if str(zero_stage) in ("2.5", "2_5", "25") else MemoryZeRO3Manager
        self.manager = mgr_cls(self.model, world_size, self.comm, rank, accum_steps=self.accum_step, fused=fused,
                               profile_comm=profile_comm)
        opt_cls = ZeRO_Adam_Offload if optimizer_device == "cpu" else ZeRO_Adam_ShardedGPU
        okw = dict(lr_max=lr_max, lr_mini=lr_mini, total_steps=total_steps, warm_up=warm_up,
                   weight_decay=weight_decay, beta1=beta1, beta2=beta2, epsilon=epsilon, logger=logger)
        if optimizer_device == "cpu":
            # torchrun pins OMP_NUM_THREADS to 1; the host AdamW wants its share of the cores
            okw["threads"] = max(1, (os.cpu_count() or 1) // max(world_size, 1))
        self.optimizer = opt_cls(self.manager.get_param_shard_view(), **okw)
        self.replica_optimizer = None
        if self.manager.replica_param_f16 is not None:
            self.replica_optimizer = opt_cls(self.manager.get_replica_optimizer_shard_view(), **okw)
        gs = dict(GradScale_dic or {})
        # bf16 has fp32's exponent range: loss scaling is kept for API parity and off by default
        self.scaler = ScaleGrad(gs.get("StartScale", 10.0), gs.get("UpRate", 2.0), gs.get("DownRate", 0.7),
                                gs.get("Scale_Up_Step"), enabled=bool(gs.get("enabled", False)))
        # Host-offloaded optimizer with a one-step delayed parameter update (the scheme of ZeRO-Offload): the host
        # AdamW of step k runs in a worker thread under the forward and backward of step k + 1, which still use
        # the parameters of step k - 1; its result is installed before step k + 2. The step then costs
        # max(GPU work, host AdamW) instead of their sum, at the price of gradients computed on parameters that
        # are one update old. Off by default (the update is then exact and on the critical path).
        self.offload_delayed_update = bool(offload_delayed_update and optimizer_device == "cpu"
                                           and self.device.type == "cuda" and self.replica_optimizer is None)
        self.iteration = 0
        self.last = {}
        # Deferred host read: the loss and the gradient statistics of step k are copied to pinned host
        # memory at the end of step k and read while step k + 1 is already queued, so the host never
        # waits for the device between steps (``train_step`` then returns the scalars of the step before;
        # ``flush_host_read`` returns the last one). The skip-on-non-finite decision stays on the device;
        # only the host's bookkeeping (schedule step count, logging) lags by one step. Not with loss
        # scaling: the scale of the next step depends on this step's overflow flag.
        self.defer_host_read = bool(defer_host_read and self.device.type == "cuda" and not self.scaler.enabled)
        self._pending_read = None
        self._host_slots = None
        self._host_slot_i = 0
        # Pipelined optimizer: AdamW runs unit by unit on its own stream in the order the next forward
        # needs the parameters, and the next step starts while it is still running (AdamW is bound by
        # HBM, the forward by the tensor cores). Needs the GPU optimizer, one micro-batch per step
        # (gradients are written in place, nothing is zeroed at the start of a step) and no replica
        # optimizer.
        self.adam_overlap = bool(adam_overlap and self.device.type == "cuda" and optimizer_device != "cpu"
                                 and self.accum_step == 1 and self.replica_optimizer is None and not fused_adam)
        self._adam_stream = torch.cuda.Stream(device=self.device) if self.adam_overlap else None
        # AdamW CTAs per SM while it runs beside the forward: few enough that the GEMM CTAs still fit
        self.adam_overlap_ctas_per_sm = int(adam_overlap_ctas_per_sm)
        self._adam_done = None
        # Whole-step CUDA graph (one GPU): forward, backward, gradient statistics and AdamW are captured
        # once and replayed; what changes from step to step (token ids, learning rate, bias corrections,
        # gradient scale) lives in device buffers the graph reads. Pays off when the step is bound by the
        # host's launch rate (small models); the eager path with the pipelined optimizer is the default.
        self.cuda_graph = bool(cuda_graph and self.device.type == "cuda" and world_size == 1
                               and optimizer_device != "cpu" and self.accum_step == 1
                               and self.replica_optimizer is None and not fused_adam
                               and not self.scaler.enabled and not self.profile_phases and not profile_comm)
        self._graph = None
        self._graph_warm = 0
        # Fully fused gradient path (reduce-scatter + AdamW in one kernel per unit, during backward).
        # The update of a unit then happens before the global gradient norm exists, so it is only
        # available without clipping (max_grads <= 0), with a GPU optimizer, one micro-batch per
        # step, no replicated parameters, and a non-finite step cannot be skipped after the fact.
        self.fused_adam = bool(fused_adam and fused is not None and self.max_grads <= 0 and self.accum_step == 1
                               and optimizer_device != "cpu" and self.replica_optimizer is None and world_size > 1)
        if fused is not None and world_size > 1 and self.device.type == "cuda":
            # The ranks enter their first step together: the first peer-memory kernel waits for the other ranks
            # with a bounded wait, and construction (module loading, allocations, optimizer state) can leave the
            # ranks seconds apart.
            torch.cuda.synchronize(self.device)
            self.comm.barrier()

    # ------------------------------------------------------------------ one optimizer step
    # ------------------------------------------------------------------ phase timing (optional)
    def _mark(self, name: str):
        """Record a CUDA event on the compute stream at a phase boundary (``profile_phases``)."""
        if self.profile_phases and self.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.device))
            self._phase_marks.append((name, ev))

    def phase_times(self, reset: bool = True) -> dict:
        """Mean milliseconds per step between consecutive phase marks since the last call
        (synchronises the device). Keys: forward, backward, grad_stats, optimizer, tail."""
        if not self._phase_marks:
            return {}
        torch.cuda.synchronize(self.device)
        tot, steps = {}, 0
        for (n0, e0), (n1, e1) in zip(self._phase_marks[:-1], self._phase_marks[1:]):
            if n1 == "start":
                continue
            tot[n1] = tot.get(n1, 0.0) + e0.elapsed_time(e1)
            steps += n1 == "end"
        if reset:
            self._phase_marks = []
        return {k: v / max(steps, 1) for k, v in tot.items()}

    def _graph_body(self, scale: float):
        """The device work of one step on static buffers (captured, then replayed)."""
        mgr = self.manager
        mgr.zero_grad()
        loss = self.model.forward(self._gx, self._gt, self._gpa, mgr)
        self.model.backward(scale, mgr)
        mgr.end_microbatch()
        stats = mgr.calculate_global_grad_stats(to_host=False)
        ranges = [mgr.layout.unit_shard_range(u) for u in mgr.forward_unit_order()]
        self.optimizer.update_ranges(mgr.grad_shard_f16, 1.0, ranges, mgr.get_param_shard_view(), stats=stats,
                                     max_grad_norm=self.max_grads, is_main_device=False, hyper=self._hyper)
        mgr.after_optimizer_step()
        return loss.detach().float().reshape(1).clone(), stats

    def _graph_step(self, batches, scale: float):
        """Returns (loss, stats, step_scale) device tensors of a replayed step, or None when this step
        has to run eagerly (warm-up steps, a batch of another shape)."""
        from ..ops import native
        x, t, x_pa = batches[0]
        if self._graph is None:
            if self._graph_warm < 2:          # lazy one-time set-up (tensor maps, attributes, streams) happens eagerly
                self._graph_warm += 1
                return None
            self.join_optimizer()
            self.manager.unit_ready = {}
            torch.cuda.synchronize(self.device)
            self._gx, self._gt, self._gpa = x.clone(), t.clone(), x_pa.clone()
            self._hyper = torch.zeros(4, dtype=torch.float32, device=self.device)
            self._hyper_host = torch.zeros(4, dtype=torch.float32).pin_memory()
            self._graph_scale = scale
            graph = torch.cuda.CUDAGraph()
            n0 = native.launch_count()
            with torch.cuda.graph(graph):
                self._g_loss, self._g_stats = self._graph_body(scale)
            self._graph_launches = native.launch_count() - n0
            self._graph = graph
        if x.shape != self._gx.shape or t.shape != self._gt.shape or scale != self._graph_scale:
            return None
        self._gx.copy_(x, non_blocking=True)
        self._gt.copy_(t, non_blocking=True)
        self._gpa.copy_(x_pa, non_blocking=True)
        self.optimizer.advance()
        step_scale = 1.0 / (self.world_size * scale)
        self._hyper_host.copy_(torch.tensor(self.optimizer.hyper_values(step_scale), dtype=torch.float32))
        self._hyper.copy_(self._hyper_host, non_blocking=True)
        self._graph.replay()
        native.bump(self._graph_launches)
        return self._g_loss, self._g_stats, step_scale

    def _account(self, host, n_micro: int, step_scale: float, scale: float, iteration: int) -> dict:
        """Host-side bookkeeping of one finished step from its scalars [loss sum, sum g^2, non-finite flag]."""
        loss_val = host[0] / n_micro
        bad = host[2] != 0.0 or not math.isfinite(host[1])
        if bad and not self.fused_adam:   # the kernels skipped the update; keep the schedule where it was
            self.optimizer.t -= 1
            if self.replica_optimizer is not None:
                self.replica_optimizer.t -= 1
        self.scaler.UpdateScale(bad)
        gnorm = math.sqrt(max(host[1], 0.0)) * step_scale if not bad else float("nan")
        self.last = {"loss": loss_val, "grad_norm": gnorm, "skipped": bad, "GradScale": scale,
                     "lr": self.optimizer.current_lr, "iteration": iteration}
        return self.last

    def _finish_step(self, loss_acc, stats, n_micro: int, step_scale: float, scale: float) -> dict:
        """One host read per step (loss, gradient statistics) and the host-side bookkeeping. With
        ``defer_host_read`` the read is of the PREVIOUS step (see the constructor); the first call then
        returns a placeholder with ``pending`` set."""
        parts = [loss_acc.reshape(1).float(), stats.reshape(-1)]
        if self.device.type == "cuda":
            # the native status word travels with the step's scalars: a kernel that gave up a bounded wait (a peer
            # that never arrived) ends the run at the next read instead of after minutes of stacked time-outs
            from ..ops import native
            parts.append(native.status_tensor(self.device)[:2].float())
        dev = torch.cat(parts)
        self.iteration += 1
        if not self.defer_host_read:
            host = dev.tolist()
            self._check_status(host)
            return self._account(host, n_micro, step_scale, scale, self.iteration)
        if self._host_slots is None:
            self._host_slots = [torch.zeros(dev.numel(), dtype=torch.float32).pin_memory() for _ in range(2)]
        slot = self._host_slots[self._host_slot_i]
        self._host_slot_i ^= 1
        slot.copy_(dev, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        prev, self._pending_read = self._pending_read, (slot, ev, n_micro, step_scale, scale, self.iteration)
        if prev is None:
            return {"loss": float("nan"), "grad_norm": float("nan"), "skipped": False, "GradScale": scale,
                    "lr": self.optimizer.current_lr, "iteration": 0, "pending": True}
        return self._read_pending(prev)

    def _check_status(self, host):
        if len(host) >= 5 and host[3] != 0.0:
            from ..ops import native
            raise native.NativeError(f"native kernel {int(host[4])} reported error {int(host[3])} during a training step "
                                     f"(1: mbarrier wait timed out, 2: wait for another GPU timed out, 4: index out of range)")

    def _read_pending(self, rec) -> dict:
        slot, ev, n_micro, step_scale, scale, it = rec
        ev.synchronize()
        host = slot.tolist()
        self._check_status(host)
        return self._account(host, n_micro, step_scale, scale, it)

    def flush_delayed_update(self):
        """Install a delayed host update that is still in flight (before anything reads the parameters for
        another purpose than the next training step: checkpoint, validation, generation, the end of a run)."""
        if self.offload_delayed_update and self.optimizer.finish_pending(self.manager.get_param_shard_view()):
            self.manager.after_optimizer_step()

    def flush_host_read(self) -> dict:
        """Scalars of the most recent step (waits for it when the read was deferred)."""
        if self._pending_read is not None:
            rec, self._pending_read = self._pending_read, None
            return self._read_pending(rec)
        return self.last

    def train_step(self, batches) -> dict:
        mgr, model = self.manager, self.model
        scale = float(self.scaler.Scale)
        if self.cuda_graph and len(batches) == 1:
            out = self._graph_step(batches, scale)
            if out is not None:
                return self._finish_step(out[0], out[1], 1, out[2], scale)
        self._mark("start")
        mgr.zero_grad()
        if self.fused_adam:
            lr = self.optimizer._update_learning_rate()
            mgr.fused_adam = {"opt": self.optimizer, "lr": lr,
                              "grad_scale": 1.0 / (self.world_size * len(batches) * scale)}
        loss_acc = None
        for (x, t, x_pa) in batches:
            with nvtx_range("forward"):
                loss = model.forward(x, t, x_pa, mgr)
            self._mark("forward")
            self.join_optimizer()          # the gradients are about to be overwritten
            with nvtx_range("backward"):
                model.backward(scale, mgr)
            mgr.end_microbatch()
            self._mark("backward")
            loss_acc = loss.detach().clone() if loss_acc is None else loss_acc + loss
        n_micro = len(batches)
        if getattr(self, "inject_nan_next", False):      # host-side fault injection (tests)
            mgr.wait_reductions()
            mgr.grad_shard_f16[:1] = float("nan")
            self.inject_nan_next = False
        with nvtx_range("optimizer"):
            rgrad = None
            if self.replica_optimizer is not None:
                # first, so that the replica slices join the one statistics pass / all-reduce below
                rgrad = mgr.prepare_replicated_grads_for_sharded_optimizer()
            stats = mgr.calculate_global_grad_stats(to_host=False)
            self._mark("grad_stats")
            step_scale = 1.0 / (self.world_size * n_micro * scale)
            pipelined = False
            if self.adam_overlap and mgr.direct_grad:
                pipelined = True
                order = mgr.forward_unit_order()
                ranges = [mgr.layout.unit_shard_range(u) for u in order]
                cur = torch.cuda.current_stream(self.device)
                stats_in = stats.clone()           # the manager reuses its statistics buffer next step
                self._adam_stream.wait_stream(cur)

                def unit_done(i):
                    if mgr.fused is not None and self.world_size > 1:
                        mgr.fused.barrier(self._adam_stream, channel=1)   # peers pull this slice straight from the shard
                    ev = torch.cuda.Event()
                    ev.record(self._adam_stream)
                    mgr.unit_ready[order[i]] = ev

                from ..ops import native
                sms = torch.cuda.get_device_properties(self.device).multi_processor_count
                prev = native.lib().b200_adamw_max_blocks(self.adam_overlap_ctas_per_sm * sms)
                with torch.cuda.stream(self._adam_stream):
                    self.optimizer.update_ranges(mgr.grad_shard_f16, step_scale, ranges, mgr.get_param_shard_view(),
                                                 stats=stats_in, max_grad_norm=self.max_grads, after_each=unit_done,
                                                 is_main_device=self.rank == 0)
                    self._adam_done = torch.cuda.Event()
                    self._adam_done.record(self._adam_stream)
                native.lib().b200_adamw_max_blocks(prev)
                stats_in.record_stream(self._adam_stream)
            elif self.offload_delayed_update:
                # install the update that has been running under this step, then start this step's
                self.optimizer.finish_pending(mgr.get_param_shard_view())
                self.optimizer.update_async(mgr.grad_shard_f16, step_scale, self.rank == 0, stats=stats,
                                            max_grad_norm=self.max_grads)
            elif not self.fused_adam:
                self.optimizer.update(mgr.grad_shard_f16, step_scale, self.rank == 0,
                                      out_shard=mgr.get_param_shard_view(), stats=stats,
                                      max_grad_norm=self.max_grads)
            if self.replica_optimizer is not None:
                self.replica_optimizer.update(rgrad, step_scale, False,
                                              out_shard=mgr.get_replica_optimizer_shard_view(), stats=stats,
                                              max_grad_norm=self.max_grads)
                mgr.allgather_replicated_params_from_optimizer_shards()
            mgr.after_optimizer_step(pipelined=pipelined)
        self._mark("end")
        return self._finish_step(loss_acc, stats, n_micro, step_scale, scale)

    def join_optimizer(self):
        """Make the current stream wait for a pipelined optimizer step that may still be running.
        Called before anything reads optimizer state or overwrites the gradients."""
        if self._adam_done is not None:
            torch.cuda.current_stream(self.device).wait_event(self._adam_done)
            self._adam_done = None

    @torch.no_grad()
    def validate(self, batches) -> float:
        """Mean validation loss over ``batches`` and over ranks (model/ZeRO3.py:388-449 intent)."""
        self.flush_delayed_update()
        tot = torch.zeros(1, dtype=torch.float32, device=self.device)
        for (x, t, x_pa) in batches:
            tot += self.model.predict(x, t, x_pa, self.manager).float()
        tot /= max(len(batches), 1)
        if self.world_size > 1:
            self.comm.all_reduce(tot)
            tot /= self.world_size
        return float(tot)

    def generate(self, prompt, **kw):
        """Generation on a sharded model: gather everything, decode, release."""
        self.flush_delayed_update()
        self.join_optimizer()
        self.manager.materialize_all()
        try:
            return self.model.generate(prompt, **kw)
        finally:
            self.manager.release_all()

    # ------------------------------------------------------------------ checkpoint
    def save(self, directory: str, extra: dict | None = None):
        self.flush_delayed_update()
        self.flush_host_read()
        gen = getattr(self.model, "_gen", None)
        state = {"iteration": self.iteration, "scaler": self.scaler.state_dict(),
                 "torch_rng": torch.get_rng_state(), "numpy_rng": np.random.get_state(),
                 "model_rng": gen.get_state().cpu() if gen is not None else None, "extra": extra or {}}
        self.join_optimizer()
        self.manager.synchronize()
        ckpt.save_checkpoint(directory, self.manager, self.optimizer, self.replica_optimizer, state)
        if self.world_size > 1:
            self.comm.barrier()

    def load(self, directory: str) -> dict | None:
        """Restore shard, optimizer state (re-seeded from the weights when the checkpoint has none),
        iteration, loss scale and the random-number states. Ends with a device synchronise and a barrier
        across ranks: in fused mode peers read this rank's shard directly, so nobody may start a step
        before every rank has finished loading."""
        self.flush_host_read()
        self.join_optimizer()
        self.manager.synchronize()
        st = ckpt.load_checkpoint(directory, self.manager, self.optimizer, self.replica_optimizer)
        if st is not None:
            self.iteration = int(st.get("iteration", 0))
            self.scaler.load_state_dict(st.get("scaler", self.scaler.state_dict()))
            if st.get("torch_rng") is not None:
                torch.set_rng_state(torch.as_tensor(st["torch_rng"], dtype=torch.uint8))
            if st.get("numpy_rng") is not None:
                np.random.set_state(st["numpy_rng"])
            gen = getattr(self.model, "_gen", None)
            if gen is not None and st.get("model_rng") is not None:
                gen.set_state(torch.as_tensor(st["model_rng"], dtype=torch.uint8))
        self.manager.unit_ready = {}
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.world_size > 1:
            self.comm.barrier()
        return st

    def close(self):
        """Release what outlives the Python objects: the symmetric heap of the fused collectives
        (checked for overwritten guard blocks on the way out)."""
        self.flush_delayed_update()
        self.flush_host_read()
        self.join_optimizer()
        self.manager.synchronize()
        if self.world_size > 1:
            self.comm.barrier()
        if self.manager.fused is not None:
            self.manager.fused.close()


# ------------------------------------------------------------------------------- worker
def prefer_eager_module_loading():
    """Ask the CUDA runtime to load every kernel when its module is registered instead of at first launch
    (``CUDA_MODULE_LOADING=EAGER``; call before the process touches CUDA). A multi-GPU job keeps kernels in
    flight that wait for a peer GPU; loading a kernel lazily at its first launch can need a context-wide
    synchronisation, and a host that sits in such a load cannot launch the kernel its peer is waiting for. Costs
    about 3 s of start-up and 0.7 GB per process (measured); single-GPU runs keep the lazy default."""
    os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")


class InjectedFault(RuntimeError):
    pass


def _maybe_inject(fault: dict | None, rank: int, it: int, trainer: Trainer | None = None):
    """Host-side fault injection for the failure-detection tests: a rank raises, exits, stalls
    (sleeps) or poisons its gradient with NaN at a chosen iteration. Nothing here touches a GPU in
    a way that could fault it."""
    if not fault or fault.get("rank") != rank or fault.get("iter") != it:
        return
    kind = fault.get("kind", "raise")
    if kind == "raise":
        raise InjectedFault(f"injected failure on rank {rank} at iteration {it}")
    if kind == "exit":
        os._exit(int(fault.get("code", 17)))
    if kind == "stall":
        time.sleep(float(fault.get("seconds", 3600)))
    if kind == "nan" and trainer is not None:
        trainer.inject_nan_next = True


def _heartbeat(path: str | None, rank: int, it: int):
    if path:
        with open(os.path.join(path, f"heartbeat_rank{rank}"), "w") as f:
            f.write(f"{time.time()} {it}\n")


def training_worker_nccl_stream(rank: int, world_size: int, args: dict):
    """One process per device: bind the device, join the process group, build the trainer and run
    the epoch / iteration loop with logging, validation and checkpoints."""
    a = args
    use_devices = a.get("use_devices") or list(range(world_size))
    if world_size > 1:
        prefer_eager_module_loading()
    on_gpu = torch.cuda.is_available() and a.get("backend", None) != "gloo"
    device = "cpu"
    if on_gpu:
        torch.cuda.set_device(use_devices[rank])
        device = torch.device("cuda", use_devices[rank])
    comm = init_distributed(rank, world_size, backend=a.get("backend"), master_port=int(a.get("master_port", 29511)),
                            timeout_s=float(a.get("collective_timeout_s", 600.0)),
                            device_id=use_devices[rank] if on_gpu else None)
    logger = MetricsLogger(rank, wand=bool(a.get("wand", False)), config=a.get("model_dic"),
                           jsonl_path=a.get("metrics_path"), console=bool(a.get("console", True)))
    result = {}
    trainer = None
    try:
        md = a["model_dic"]
        B, T, accum = int(a["batch_size"]), int(md["time_size"]), int(a.get("accum_step", 1))
        max_iters = int(a["max_iters"])
        # Peer-memory collectives (fused reduce-scatter + statistics, copy-engine / pull gathers) are what a
        # multi-GPU job runs by default; ``zero3_fused_collectives=False`` selects the NCCL path.
        fused = None
        if on_gpu and world_size > 1 and bool(md.get("zero3_fused_collectives", True)) \
                and getattr(comm, "backend", "") == "nccl":
            from .symm import FusedCollectives
            fkw = {}
            if a.get("peer_wait_s") is not None:
                fkw["wait_ns"] = int(float(a["peer_wait_s"]) * 1e9)
            if md.get("zero3_copy_min_bytes") is not None:       # smaller slices use the pull kernel
                fkw["copy_min_bytes"] = int(md["zero3_copy_min_bytes"])
            fused = FusedCollectives(comm, device, gather_mode=str(md.get("zero3_gather_mode", "copy")),
                                     reduce_mode=str(md.get("zero3_reduce_mode", "copy")), **fkw)
        trainer = Trainer(md, rank=rank, world_size=world_size, comm=comm, device=device,
                          zero_stage=a.get("zero_stage", "3"), optimizer_device=a.get("optimizer_device", "gpu"),
                          accum_step=accum, lr_max=a.get("lr_max", 3e-4), lr_mini=a.get("lr_mini", 3e-5),
                          weight_decay=a.get("weight_decay", 0.1), warm_up=a.get("warm_up", 100),
                          total_steps=max_iters * int(a.get("max_epoch", 1)), beta1=a.get("beta1", 0.9),
                          beta2=a.get("beta2", 0.99), epsilon=a.get("epsilon", 1e-6), max_grads=a.get("max_grads", 1.0),
                          GradScale_dic=a.get("GradScale_dic"), logger=logger, param_path=a.get("train_continue_path"),
                          profile_comm=bool(a.get("profile_timing", False)), fused=fused,
                          defer_host_read=bool(a.get("defer_host_read", True)))
        if a.get("resume_dir") and os.path.exists(ckpt.model_shard_path(a["resume_dir"], rank)):
            trainer.load(a["resume_dir"])
        if rank == 0:
            logger.line(f"parameters: {trainer.n_params:,}; shard {trainer.manager.shard_size * 2 / 2**30:.3f} GiB/rank; "
                        f"world {world_size}; ZeRO-{a.get('zero_stage', '3')}; collectives: "
                        + ("nccl" if fused is None else f"peer memory (gather: {fused.gather_mode})"))
            print_memory_status("after init", printer=logger.line)

        pad = int(md["padding_id"])
        if a.get("data_dir"):
            from ..utils.data import load_input_ids_from_dir
            ids, vl = to_fixed_length(load_input_ids_from_dir(a["data_dir"], int(a.get("max_samples", 100000))), T, pad)
            ds = SplitDataset(ids, vl, n_val=B * accum * world_size if a.get("vali") else 0,
                              n_gen=int(a.get("n_gen", 0)), seed=int(a.get("data_seed", 0)))
        else:
            n_train = int(a.get("synthetic_samples", max(B * accum * world_size * 4, 64)))
            ds = SplitDataset.synthetic(int(md["vocab_size"]), T, n_train, B * accum * world_size,
                                        int(a.get("n_gen", 4)), pad)
        tr_ids, tr_vl = shard_for_rank(*ds.train, rank, world_size)
        va_ids, va_vl = shard_for_rank(*ds.val, rank, world_size)
        gen_ids, gen_vl = ds.gen
        stager = BatchStager(B, T, device, depth=max(4, 2 * accum))      # the host stages a whole step ahead
        val_batches = None
        tokens_per_step = B * T * accum * world_size
        losses = {}
        samples = []
        # a resumed job continues where the saved one stopped: same epoch, same position in the data
        start_epoch, start_it = divmod(trainer.iteration, max_iters)
        time_idx = trainer.iteration * accum
        hb = a.get("heartbeat_dir")
        t_last = time.perf_counter()

        def report(out):
            nonlocal t_last
            if out.get("pending"):
                return
            losses[out["iteration"]] = out["loss"]
            now = time.perf_counter()
            tok_s = tokens_per_step / max(now - t_last, 1e-9)
            t_last = now
            logger.log({"loss": out["loss"], "Perplexity": math.exp(min(out["loss"], 30.0)),
                        "Grad Norm": out["grad_norm"], "GradScale": out["GradScale"],
                        "tokens_per_s": tok_s}, step=out["iteration"])
            e, i = divmod(out["iteration"] - 1, max_iters)
            logger.step_line(e, i + 1, max_iters, out["loss"],
                             {"gnorm": out["grad_norm"], "tok/s": tok_s, "skipped": out["skipped"]})

        stop_after = int(a.get("stop_after") or 0)      # leave after this many iterations in total (0: run to the end)
        for epoch in range(start_epoch, int(a.get("max_epoch", 1))):
            for it in range(start_it if epoch == start_epoch else 0, max_iters):
                if stop_after and trainer.iteration >= stop_after:
                    break
                _heartbeat(hb, rank, it)
                _maybe_inject(a.get("fault"), rank, it, trainer)
                batches = []
                for _ in range(accum):
                    xb, vb, time_idx = get_batch(tr_ids, tr_vl, B, time_idx)
                    batches.append(stager.stage(xb, vb, pad))
                report(trainer.train_step(batches))
                if a.get("vali") and (it + 1) % int(a.get("vali_step", 600)) == 0:
                    report(trainer.flush_host_read())
                    if len(va_ids) >= B:
                        if val_batches is None:
                            val_batches = [stager.stage(va_ids[i:i + B], va_vl[i:i + B], pad)
                                           for i in range(0, len(va_ids) - B + 1, B)]
                        v = trainer.validate(val_batches)
                        logger.log({"validation": v}, step=trainer.iteration)
                        logger.line(f"validation loss {v:.4f}")
                    # Generation split (the third part of the reference's "Train, Validation, Generation"):
                    # every rank takes part in the gathers, the samples are logged once.
                    n_prompt = int(a.get("gen_prompt_tokens", 16))
                    for g in range(min(len(gen_ids), int(a.get("gen_samples", 1)))):
                        prompt = [int(v) for v in gen_ids[g][:min(n_prompt, int(gen_vl[g]), T - 2)] if int(v) != pad]
                        if not prompt:
                            continue
                        toks = trainer.generate(prompt, max_new_tokens=int(a.get("gen_tokens", 32)),
                                                greedy=bool(a.get("gen_greedy", True)), padding_id=pad)
                        samples.append({"iteration": trainer.iteration, "prompt": prompt, "tokens": toks})
                        logger.log({"generated_tokens": len(toks)}, step=trainer.iteration)
                        logger.line(f"generation sample {g}: prompt {prompt} -> {toks}")
                if a.get("save") and a.get("save_dir") and (it + 1) % int(a.get("save_step", 2000)) == 0:
                    report(trainer.flush_host_read())
                    trainer.save(a["save_dir"])
        report(trainer.flush_host_read())
        trainer.manager.synchronize()
        from ..ops import native
        if on_gpu:
            native.raise_on_status()
        result = {"losses": [losses[k] for k in sorted(losses)], "iteration": trainer.iteration,
                  "generation": samples, "native_launches": native.launch_count(),
                  "fused_launches": fused.launches if fused is not None else 0,
                  "copy_engine_transfers": fused.copies if fused is not None else 0,
                  "collectives": "nccl" if fused is None else f"fused:{fused.gather_mode}"}
        if a.get("result_dir"):
            ckpt.atomic_pickle_gzip(result, os.path.join(a["result_dir"], f"result_rank{rank}.pkl.gz"))
        trainer.close()
    except BaseException:
        traceback.print_exc()
        logger.close()
        os._exit(13)      # leave without waiting on peers that may be blocked in a collective
    logger.close()
    if world_size > 1:
        comm.barrier()
        shutdown_distributed()
    return result


# ------------------------------------------------------------------------------- launcher
class WorkerFailure(RuntimeError):
    pass


class TrainMultiGPU:
    """Launcher: one process per entry of ``use_devices`` (spawn), watched until all finish.

    ``fit(data_size)`` keeps the reference's contract (``max_iters = data_size // (batch_size *
    accum_step)``, model/ZeRO3.py:692-693) except that the count is also divided by the number of
    ranks, because here ranks consume different samples.
    """

    zero_stage = "3"

    def __init__(self, model_dic, GradScale_dic=None, use_devices=(0,), batch_size=1, max_epoch=1, lr_max=3e-4,
                 lr_mini=3e-5, weight_decay=0.1, warm_up=100, max_grads=1.0, accum_step=1, save=False,
                 save_step=2000, vali=False, vali_step=600, wand=False, optimizer_device="gpu",
                 train_continue_path=None, **extra):
        self.args = dict(model_dic=dict(model_dic), GradScale_dic=dict(GradScale_dic or {}), use_devices=list(use_devices),
                         batch_size=batch_size, max_epoch=max_epoch, lr_max=lr_max, lr_mini=lr_mini,
                         weight_decay=weight_decay, warm_up=warm_up, max_grads=max_grads, accum_step=accum_step,
                         save=save, save_step=save_step, vali=vali, vali_step=vali_step, wand=wand,
                         optimizer_device=optimizer_device, train_continue_path=train_continue_path,
                         zero_stage=self.zero_stage)
        self.args.update(extra)
        self.heartbeat_timeout_s = float(extra.get("heartbeat_timeout_s", 1800.0))

    def fit(self, data_size: int):
        a = self.args
        world = len(a["use_devices"])
        a["max_iters"] = max(1, int(data_size) // (int(a["batch_size"]) * int(a["accum_step"]) * world))
        if world == 1 and not a.get("force_spawn"):
            return [training_worker_nccl_stream(0, 1, a)]
        return self._spawn(world)

    def _spawn(self, world: int):
        import tempfile
        import torch.multiprocessing as mp
        a = self.args
        prefer_eager_module_loading()       # inherited by the workers, which set it again before they touch CUDA
        hb_dir = a.get("heartbeat_dir") or tempfile.mkdtemp(prefix="b200_hb_")
        a["heartbeat_dir"] = hb_dir
        a.setdefault("master_port", 29500 + (os.getpid() % 2000))
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=training_worker_nccl_stream, args=(r, world, a), daemon=False) for r in range(world)]
        for p in procs:
            p.start()
        t0 = time.time()
        failure = None
        while True:
            alive = [p.is_alive() for p in procs]
            codes = [p.exitcode for p in procs]
            bad = [(r, c) for r, c in enumerate(codes) if c not in (None, 0)]
            if bad:
                failure = f"rank {bad[0][0]} exited with code {bad[0][1]}"
                break
            if not any(alive):
                break
            now = time.time()
            for r in range(world):
                hp = os.path.join(hb_dir, f"heartbeat_rank{r}")
                last = os.path.getmtime(hp) if os.path.exists(hp) else t0
                if alive[r] and now - last > self.heartbeat_timeout_s:
                    failure = f"rank {r} stalled: no heartbeat for {now - last:.0f} s"
                    break
            if failure:
                break
            time.sleep(0.2)
        if failure:
            for p in procs:
                if p.is_alive():
                    p.terminate()
            for p in procs:
                p.join(timeout=10)
                if p.is_alive():
                    p.kill()
            raise WorkerFailure(failure)
        for p in procs:
            p.join()
        return [p.exitcode for p in procs]


class TrainMultiGPU_ZeRO25(TrainMultiGPU):
    zero_stage = "2.5"

    def __init__(self, model_dic, *args, zero25_replica_ratio=None, zero25_replica_policy=None, **kw):
        md = dict(model_dic)
        if zero25_replica_ratio is not None:
            md["zero25_replica_ratio"] = zero25_replica_ratio
        if zero25_replica_policy is not None:
            md["zero25_replica_policy"] = zero25_replica_policy
        super().__init__(md, *args, **kw)
