"""AdamW over a rank's flat shard: GPU-resident (``ZeRO_Adam_ShardedGPU``) or host-offloaded
(``ZeRO_Adam_Offload``), with the reference's schedule (linear warm-up, cosine decay) and state
(fp32 master / m / v, step counter). Reference: model/optimizer.py:6-109 and :112-227.

Differences by design
  * betas / eps are constructor arguments (the reference hard-codes beta2 = 0.99, eps = 1e-6; those
    stay the defaults);
  * gradients may be bf16 or fp32; the clip coefficient and the skip-on-non-finite decision can be
    taken on the device from a statistics tensor (``stats=``), so no host sync sits between the
    gradient norm and the update;
  * the offload tier keeps master/m/v in pinned host memory, moves the gradient shard D2H and the
    updated bf16 parameters H2D with ``cudaMemcpyAsync`` on a side stream in chunks, and runs a
    multi-threaded C++ AdamW on each chunk while the next one is in flight (the reference does one
    blocking copy and ~12 single-threaded NumPy passes).
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from ..ops import functional as F
from ..ops import native


def cosine_lr(step: int, lr_max: float, lr_mini: float, warm_up: int, total_steps: int) -> float:
    if step < warm_up:
        return lr_max * step / max(1, warm_up)
    progress = (step - warm_up) / max(1, total_steps - warm_up)
    return lr_mini + 0.5 * (lr_max - lr_mini) * (1 + math.cos(math.pi * progress))


class _AdamBase:
    def __init__(self, lr_max, lr_mini, total_steps, warm_up, weight_decay, beta1, beta2, epsilon, wand=False,
                 logger=None):
        self.lr_max, self.lr_mini = float(lr_max), float(lr_mini)
        self.total_steps, self.warm_up = int(total_steps), int(warm_up)
        self.weight_decay = float(weight_decay)
        self.beta1, self.beta2, self.epsilon = float(beta1), float(beta2), float(epsilon)
        self.wand = wand
        self.logger = logger
        self.t = 0
        self.current_lr = 0.0

    def _update_learning_rate(self) -> float:
        self.t += 1
        self.current_lr = cosine_lr(self.t, self.lr_max, self.lr_mini, self.warm_up, self.total_steps)
        return self.current_lr

    def _log_lr(self, is_main_device: bool):
        if is_main_device and self.logger is not None:
            self.logger.log({"learning_rate": float(self.current_lr)})


class ZeRO_Adam_ShardedGPU(_AdamBase):
    """AdamW whose state lives beside the shard on the GPU: 12 bytes per shard element
    (fp32 master + m + v), one fused kernel per step (model/optimizer.py:112-227)."""

    def __init__(self, param_shard: torch.Tensor, lr_max=3e-4, lr_mini=3e-5, total_steps=1000, warm_up=100,
                 weight_decay=0.1, beta1=0.9, beta2=0.99, epsilon=1e-6, wand=False, logger=None):
        super().__init__(lr_max, lr_mini, total_steps, warm_up, weight_decay, beta1, beta2, epsilon, wand, logger)
        self.master_weight_shard = param_shard.detach().float().clone()
        self.m = torch.zeros_like(self.master_weight_shard)
        self.v = torch.zeros_like(self.master_weight_shard)

    def update(self, grad_shard, scale: float, is_main_device: bool = True, out_shard=None, stream=None,
               stats=None, max_grad_norm: float = 0.0, skip: bool = False):
        """One step. ``scale`` multiplies the gradient (1 / (world * accum * loss_scale), times a
        host-computed clip coefficient if the caller clips on the host). With ``stats`` the clip
        and the non-finite skip happen on the device. ``skip`` = host already knows the step is
        bad: only the schedule advances, as in the reference's NaN path."""
        lr = self._update_learning_rate()
        if skip:
            return out_shard
        if out_shard is None:
            out_shard = torch.empty(grad_shard.shape, dtype=torch.bfloat16 if grad_shard.is_cuda else grad_shard.dtype,
                                    device=grad_shard.device)
        F.adamw_step(grad_shard, self.m, self.v, self.master_weight_shard, out_shard, lr=lr, beta1=self.beta1,
                     beta2=self.beta2, eps=self.epsilon, weight_decay=self.weight_decay, step=self.t,
                     grad_scale=float(scale), max_grad_norm=float(max_grad_norm), stats=stats)
        self._log_lr(is_main_device)
        return out_shard

    def hyper_values(self, scale: float):
        """[lr, m_corr, v_corr, grad_scale] of the step that ``advance()`` has just opened."""
        return [self.current_lr, 1.0 / (1.0 - self.beta1 ** self.t), 1.0 / (1.0 - self.beta2 ** self.t), float(scale)]

    def advance(self) -> float:
        """Open the next step on the host (step count, learning-rate schedule)."""
        return self._update_learning_rate()

    def update_ranges(self, grad_shard, scale: float, ranges, out_shard, stats=None, max_grad_norm: float = 0.0,
                      after_each=None, is_main_device: bool = True, hyper=None):
        """The same step as ``update`` issued as one kernel per ``(lo, hi)`` range of the shard, in the
        given order; ``after_each(i)`` runs after range i has been launched (the caller records an
        event there, so that whoever needs that part of the parameters waits for it alone). With
        ``hyper`` (device tensor, see ``hyper_values``) the step-dependent scalars are read on the
        device and the host schedule is NOT advanced here: the caller calls ``advance()`` once per
        replay of the captured launches."""
        lr = self.current_lr if hyper is not None else self._update_learning_rate()
        for i, (lo, hi) in enumerate(ranges):
            if hi > lo:
                F.adamw_step(grad_shard[lo:hi], self.m[lo:hi], self.v[lo:hi], self.master_weight_shard[lo:hi],
                             out_shard[lo:hi], lr=lr, beta1=self.beta1, beta2=self.beta2, eps=self.epsilon,
                             weight_decay=self.weight_decay, step=max(self.t, 1), grad_scale=float(scale),
                             max_grad_norm=float(max_grad_norm), stats=stats, hyper=hyper)
            if after_each is not None:
                after_each(i)
        self._log_lr(is_main_device)
        return out_shard

    def reseed_from_params(self, param_shard: torch.Tensor):
        """Start a fresh optimizer state from (newly loaded) parameters: fp32 master = the shard, m = v = 0,
        step 0. Used when a checkpoint carries weights but no optimizer file."""
        self.master_weight_shard.copy_(param_shard.detach().float())
        self.m.zero_()
        self.v.zero_()
        self.t = 0

    def state_dict(self) -> dict:
        return {"m": self.m, "v": self.v, "w_fp32": self.master_weight_shard, "t": self.t}

    def load_state_dict(self, sd: dict):
        self.m.copy_(torch.as_tensor(sd["m"]).to(self.m.device))
        self.v.copy_(torch.as_tensor(sd["v"]).to(self.v.device))
        self.master_weight_shard.copy_(torch.as_tensor(sd["w_fp32"]).to(self.m.device))
        self.t = int(sd["t"])


class ZeRO_Adam_Offload(_AdamBase):
    """AdamW with master / m / v in pinned host DRAM (model/optimizer.py:6-109).

    Per step the gradient shard streams to the host in chunks on a side stream; as each chunk
    lands, the C++ AdamW (OpenMP, vectorised) updates it and the refreshed bf16 parameters stream
    back, so PCIe/C2C transfers in both directions overlap the CPU arithmetic.
    """

    CHUNK = 8 * 1024 * 1024  # elements per pipeline stage

    def __init__(self, param_shard: torch.Tensor, lr_max=3e-4, lr_mini=3e-5, total_steps=1000, warm_up=100,
                 weight_decay=0.1, beta1=0.9, beta2=0.99, epsilon=1e-6, wand=False, logger=None, threads: int = 0):
        super().__init__(lr_max, lr_mini, total_steps, warm_up, weight_decay, beta1, beta2, epsilon, wand, logger)
        n = param_shard.numel()
        pin = param_shard.is_cuda
        self.n = n
        self.device = param_shard.device
        self.master_weight_shard = torch.empty(n, dtype=torch.float32, pin_memory=pin)
        self.master_weight_shard.copy_(param_shard.detach().float().cpu())
        self.m = torch.zeros(n, dtype=torch.float32, pin_memory=pin)
        self.v = torch.zeros(n, dtype=torch.float32, pin_memory=pin)
        self.grad_dtype = None
        self.grad_cpu = None
        self.out_cpu = torch.empty(n, dtype=param_shard.dtype, pin_memory=pin)
        self.threads = int(threads)
        self._pending = None            # (thread, result) of a background update (delayed parameter update)
        self._grad_snapshot = None
        self._param_staging = None
        self.side_stream = torch.cuda.Stream(device=self.device) if pin else None
        self._lib = native.lib() if pin or _cpu_lib_ok() else None

    def _ensure_grad_staging(self, dtype):
        if self.grad_cpu is None or self.grad_dtype != dtype:
            self.grad_cpu = torch.empty(self.n, dtype=dtype, pin_memory=self.device.type == "cuda")
            self.grad_dtype = dtype

    def _cpu_adam(self, lo: int, hi: int, lr: float, gmul: float, step: int | None = None):
        g = self.grad_cpu[lo:hi]
        m, v, w, o = self.m[lo:hi], self.v[lo:hi], self.master_weight_shard[lo:hi], self.out_cpu[lo:hi]
        step = self.t if step is None else step
        m_corr = 1.0 / (1.0 - self.beta1 ** step)
        v_corr = 1.0 / (1.0 - self.beta2 ** step)
        if self._lib is not None and g.dtype in (torch.bfloat16, torch.float32) and o.dtype in (torch.bfloat16, torch.float32):
            rc = self._lib.b200_cpu_adamw(
                ctypes.c_void_p(g.data_ptr()), int(g.dtype == torch.float32), ctypes.c_void_p(m.data_ptr()),
                ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(o.data_ptr()),
                int(o.dtype == torch.float32), ctypes.c_longlong(hi - lo), ctypes.c_float(lr),
                ctypes.c_float(self.beta1), ctypes.c_float(self.beta2), ctypes.c_float(self.epsilon),
                ctypes.c_float(self.weight_decay), ctypes.c_float(m_corr), ctypes.c_float(v_corr),
                ctypes.c_float(gmul), self.threads)
            if rc != 0:
                raise RuntimeError(f"b200_cpu_adamw failed ({rc})")
            return
        gf = g.float() * gmul
        m.mul_(self.beta1).add_(gf, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(gf, gf, value=1 - self.beta2)
        if self.weight_decay > 0:
            w.mul_(1 - lr * self.weight_decay)
        w.sub_(lr * (m * m_corr) / (torch.sqrt(v * v_corr) + self.epsilon))
        o.copy_(w.to(o.dtype))

    def update(self, grad_shard, scale: float, is_main_device: bool = True, out_shard=None, stream=None,
               stats=None, max_grad_norm: float = 0.0, skip: bool = False):
        lr = self._update_learning_rate()
        if skip:
            return out_shard
        gmul = float(scale)
        if stats is not None:
            s = stats.detach().float().cpu()
            if float(s[1]) != 0.0:
                return out_shard
            if max_grad_norm > 0:
                gmul *= min(1.0, max_grad_norm / (math.sqrt(float(s[0])) * float(scale) + 1e-6))
        self._ensure_grad_staging(grad_shard.dtype)
        n = self.n
        if out_shard is None:
            out_shard = torch.empty(n, dtype=self.out_cpu.dtype, device=grad_shard.device)
        if not grad_shard.is_cuda:
            self.grad_cpu.copy_(grad_shard)
            self._cpu_adam(0, n, lr, gmul)
            out_shard.copy_(self.out_cpu)
            self._log_lr(is_main_device)
            return out_shard
        side = self.side_stream
        side.wait_stream(torch.cuda.current_stream(self.device))
        bounds = [(lo, min(lo + self.CHUNK, n)) for lo in range(0, n, self.CHUNK)]
        events = []
        with torch.cuda.stream(side):
            for lo, hi in bounds:
                self.grad_cpu[lo:hi].copy_(grad_shard[lo:hi], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(side)
                events.append(ev)
        for (lo, hi), ev in zip(bounds, events):
            ev.synchronize()                       # chunk landed in pinned memory
            self._cpu_adam(lo, hi, lr, gmul)       # CPU works while later chunks are still moving
            with torch.cuda.stream(side):
                out_shard[lo:hi].copy_(self.out_cpu[lo:hi], non_blocking=True)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self._log_lr(is_main_device)
        return out_shard

    def reseed_from_params(self, param_shard: torch.Tensor):
        """As ``ZeRO_Adam_ShardedGPU.reseed_from_params``, on the host-resident state."""
        self.master_weight_shard.copy_(param_shard.detach().float().cpu())
        self.m.zero_()
        self.v.zero_()
        self.t = 0

    # ------------------------------------------------------------------ delayed parameter update
    def update_async(self, grad_shard, scale: float, is_main_device: bool = True, stats=None,
                     max_grad_norm: float = 0.0):
        """Start this step's update in the background and return at once: a snapshot of the gradient shard is
        taken on the device, a worker thread moves it to the host, runs the C++ AdamW and sends the new bf16
        parameters into a device staging buffer. ``finish_pending(out_shard)`` later installs them. Used for the
        one-step delayed parameter update: the host arithmetic of step k runs under the forward and backward of
        step k + 1, which still see the parameters of step k - 1."""
        import threading
        assert grad_shard.is_cuda and self._pending is None
        lr = self._update_learning_rate()
        if self._grad_snapshot is None or self._grad_snapshot.dtype != grad_shard.dtype:
            self._grad_snapshot = torch.empty_like(grad_shard)
            self._param_staging = torch.empty(self.n, dtype=self.out_cpu.dtype, device=grad_shard.device)
        self._grad_snapshot.copy_(grad_shard)
        stats_snap = stats.detach().clone() if stats is not None else None
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        self._ensure_grad_staging(grad_shard.dtype)
        result = {"done": None, "applied": False, "error": None}
        t_step = self.t

        def work():
            try:
                torch.cuda.set_device(self.device)
                side = self.side_stream
                side.wait_event(ready)
                gmul = float(scale)
                if stats_snap is not None:
                    with torch.cuda.stream(side):
                        s = stats_snap.float().cpu()
                    if float(s[1]) != 0.0:
                        return                               # non-finite gradient: this step changes nothing
                    if max_grad_norm > 0:
                        gmul *= min(1.0, max_grad_norm / (math.sqrt(float(s[0])) * float(scale) + 1e-6))
                n = self.n
                bounds = [(lo, min(lo + self.CHUNK, n)) for lo in range(0, n, self.CHUNK)]
                events = []
                with torch.cuda.stream(side):
                    for lo, hi in bounds:
                        self.grad_cpu[lo:hi].copy_(self._grad_snapshot[lo:hi], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(side)
                        events.append(ev)
                saved_t, self_t = self.t, t_step
                for (lo, hi), ev in zip(bounds, events):
                    ev.synchronize()
                    self._cpu_adam(lo, hi, lr, gmul, step=self_t)
                    with torch.cuda.stream(side):
                        self._param_staging[lo:hi].copy_(self.out_cpu[lo:hi], non_blocking=True)
                done = torch.cuda.Event()
                done.record(side)
                result["done"] = done
                result["applied"] = True
                del saved_t
            except BaseException as e:       # surfaced by finish_pending on the main thread
                result["error"] = e

        th = threading.Thread(target=work, name="b200-offload-adam", daemon=True)
        th.start()
        self._pending = (th, result)
        self._log_lr(is_main_device)

    def finish_pending(self, out_shard=None) -> bool:
        """Wait for the background update (if one is running) and copy its parameters into ``out_shard``.
        Returns True when parameters were installed."""
        if self._pending is None:
            return False
        th, result = self._pending
        self._pending = None
        th.join()
        if result["error"] is not None:
            raise result["error"]
        if not result["applied"]:
            return False
        torch.cuda.current_stream(self.device).wait_event(result["done"])
        if out_shard is not None:
            out_shard.copy_(self._param_staging)
        return True

    def state_dict(self) -> dict:
        self.finish_pending(None)
        return {"m": self.m, "v": self.v, "w_fp32": self.master_weight_shard, "t": self.t}

    def load_state_dict(self, sd: dict):
        self.m.copy_(torch.as_tensor(sd["m"]).cpu())
        self.v.copy_(torch.as_tensor(sd["v"]).cpu())
        self.master_weight_shard.copy_(torch.as_tensor(sd["w_fp32"]).cpu())
        self.t = int(sd["t"])


def _cpu_lib_ok() -> bool:
    try:
        native.lib()
        return True
    except Exception:
        return False
