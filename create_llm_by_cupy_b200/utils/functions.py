"""Training utilities: loss-scale controller, gradient clipping helpers, initialisers, memory
report. Counterpart of the reference's model/functions.py (ScaleGrad :211-235, clipping variants
:100-195, init_weight :62-63, print_memory_status :199-207)."""
from __future__ import annotations

import math
import random

import torch


class ScaleGrad:
    """Dynamic loss scale: shrink on a non-finite step, double after ``Scale_Up_Step`` good ones.

    Same policy as the reference (start 10, x0.7 on overflow, reset to ``StartScale`` plus a random
    1000..2000 when the scale collapses below 0.01, x``UpRate`` every ``Scale_Up_Step`` good
    steps), except that the down-scaled value is not truncated to an integer (the reference's
    ``int()`` floors e.g. 1.4 -> 1 and can never recover from 0). bf16 training does not need loss
    scaling: ``enabled=False`` pins the scale to 1.
    """

    def __init__(self, StartScale: float = 10.0, UpRate: float = 2.0, DownRate: float = 0.7,
                 Scale_Up_Step: int | None = None, enabled: bool = True, seed: int | None = None):
        self.StartScale = float(StartScale)
        self.UpRate = float(UpRate)
        self.DownRate = float(DownRate)
        self.Scale_Up_Step = int(Scale_Up_Step if Scale_Up_Step is not None else StartScale)
        self.enabled = enabled
        self.Scale = self.StartScale if enabled else 1.0
        self.good_steps = 0
        self.skipped = 0
        self._rng = random.Random(seed)

    def UpdateScale(self, nan_flag: bool) -> float:
        if not self.enabled:
            if nan_flag:
                self.skipped += 1
            return self.Scale
        if nan_flag:
            self.skipped += 1
            self.good_steps = 0
            self.Scale *= self.DownRate
            if self.Scale <= 0.01:
                self.Scale = self.StartScale + self._rng.randint(1000, 2000)
        else:
            self.good_steps += 1
            if self.good_steps >= self.Scale_Up_Step:
                self.Scale *= self.UpRate
                self.good_steps = 0
        return self.Scale

    def state_dict(self) -> dict:
        return {"Scale": self.Scale, "good_steps": self.good_steps, "skipped": self.skipped}

    def load_state_dict(self, sd: dict):
        self.Scale = float(sd["Scale"])
        self.good_steps = int(sd.get("good_steps", 0))
        self.skipped = int(sd.get("skipped", 0))


def init_weight(shape, std: float, dtype=torch.bfloat16, device="cpu", generator=None) -> torch.Tensor:
    w = torch.randn(*shape, dtype=torch.float32, device=generator.device if generator is not None else device,
                    generator=generator) * std
    return w.to(device=device, dtype=dtype)


def xavier_initialization(shape, dtype=torch.float32, device="cpu", generator=None) -> torch.Tensor:
    fan_in, fan_out = shape[0], shape[-1]
    return init_weight(shape, math.sqrt(2.0 / (fan_in + fan_out)), dtype, device, generator)


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return torch.sigmoid(x)


def softmax(x: torch.Tensor) -> torch.Tensor:
    return torch.softmax(x.float(), dim=-1).to(x.dtype)


def place_enco(T: int, H: int, device="cpu") -> torch.Tensor:
    """Sinusoidal position table [T, H] (legacy helper of the reference, unused by the model)."""
    pos = torch.arange(T, dtype=torch.float32, device=device)[:, None]
    i = torch.arange(0, H, 2, dtype=torch.float32, device=device)[None, :]
    ang = pos / torch.pow(torch.tensor(10000.0, device=device), i / H)
    out = torch.zeros(T, H, device=device)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang)[:, : out[:, 1::2].shape[1]]
    return out


def clip_coefficient(global_sq_sum: float, max_grads: float) -> float:
    """min(1, max / (norm + 1e-6)) (model/ZeRO3.py:358-360)."""
    return min(1.0, max_grads / (math.sqrt(max(global_sq_sum, 0.0)) + 1e-6))


def total_clip_grads(grads, max_norm: float):
    """In-place global-norm clip of a list of full gradients (single-process helper)."""
    sq = sum(float((g.float() ** 2).sum()) for g in grads if g is not None)
    coef = clip_coefficient(sq, max_norm)
    if coef < 1.0:
        for g in grads:
            if g is not None:
                g.mul_(coef)
    return math.sqrt(sq)


def ZeRO_clip_grads(grad_shard: torch.Tensor, comm, max_norm: float) -> float:
    """Global-norm clip of a sharded gradient: local sum of squares, one scalar all-reduce."""
    sq = (grad_shard.float() ** 2).sum().reshape(1)
    if comm is not None and comm.world_size > 1:
        comm.all_reduce(sq)
    norm = math.sqrt(float(sq))
    coef = min(1.0, max_norm / (norm + 1e-6))
    if coef < 1.0:
        grad_shard.mul_(coef)
    return norm


def print_memory_status(tag: str = "", device=None, printer=print) -> dict:
    """Allocated / reserved device memory in GiB at a labelled point."""
    if not torch.cuda.is_available():
        info = {"tag": tag, "allocated_gib": 0.0, "reserved_gib": 0.0}
    else:
        info = {"tag": tag,
                "allocated_gib": torch.cuda.memory_allocated(device) / 2 ** 30,
                "reserved_gib": torch.cuda.memory_reserved(device) / 2 ** 30}
    if printer is not None:
        printer(f"[mem] {tag}: allocated {info['allocated_gib']:.2f} GiB, reserved {info['reserved_gib']:.2f} GiB")
    return info


def look_list(ids, word_id_path: str = "word_id.pkl.gz", printer=print):
    """Debug helper: print the words of a list of token ids using a gzip-pickled ``{word: id}``
    (or ``{id: word}``) dictionary (model/ZeRO3.py:503-515)."""
    import gzip
    import pickle
    with gzip.open(word_id_path, "rb") as f:
        table = pickle.load(f)
    if table and not isinstance(next(iter(table)), int):
        table = {v: k for k, v in table.items()}
    words = [str(table.get(int(i), f"<{int(i)}>")) for i in ids]
    if printer is not None:
        printer(" ".join(words))
    return words


def pad_mask_to_valid_len(mask, T: int):
    """Accept the pad-mask forms the reference's attention takes (model/fast_layers.py:126-202,
    model/flash_attention.py:28-41) and return valid key lengths [B] (int32), which is what the
    attention kernels consume:

      * a 1-D integer vector is taken as the valid lengths themselves;
      * a boolean mask of shape [B, T], [B, 1, 1, T] or [B, 1, 1, 1, T] with True = padded key;
      * an additive mask of those shapes with -inf (or a large negative value) at padded keys.

    Padding must be a suffix of each row (keys 0 .. len-1 valid), as produced by make_mask."""
    m = torch.as_tensor(mask)
    if m.dim() == 1 and not m.dtype.is_floating_point and m.dtype != torch.bool:
        return m.to(torch.int32)
    m = m.reshape(m.shape[0], -1)[:, -T:] if m.dim() > 2 else m
    if m.dtype == torch.bool:
        padded = m
    else:
        padded = m < -1e4
    valid = (~padded).to(torch.int32)
    lens = valid.sum(-1).to(torch.int32)
    # suffix check: the first `len` keys must be the valid ones
    idx = torch.arange(T, device=m.device)[None, :]
    if not bool(((idx < lens[:, None]) == (valid > 0)).all()):
        raise ValueError("pad mask is not a suffix mask; only right-padded sequences are supported")
    return lens
