"""Data pipeline: Train / Validation / Generation streams, batching and padding.

The reference pulls ``*.jsonl.gz`` shards of ``{"input_ids": [...]}`` records from Google Drive
through ``rclone`` (model/ZeRO3.py:550-647), gives every rank the *same* samples, and cuts batches
with strided offsets (:32-49) and a pad/shift step (:52-65). Here:

  * sources are a local directory of the same ``jsonl.gz`` records, an optional ``rclone`` remote
    (same command line, only when the binary exists), or synthetic uniform-random token ids —
    seeds 0 / 1 / 2 for the train / validation / generation splits;
  * samples are partitioned across data-parallel ranks (rank r takes every world-th sample);
  * batches are assembled into pinned host tensors, so the H2D copy of each step is asynchronous.
"""
from __future__ import annotations

import glob
import gzip
import json
import os
import shutil
import subprocess

import numpy as np
import torch

SPLIT_SEEDS = {"train": 0, "validation": 1, "generation": 2}


# --------------------------------------------------------------------------- sources
def synthetic_token_stream(n_samples: int, seq_len: int, vocab_size: int, split: str = "train",
                           padding_id: int | None = None, low: int = 0) -> np.ndarray:
    """``[n_samples, seq_len]`` int32 ids drawn uniformly from the vocabulary with the split's seed.
    ``padding_id`` (if inside the range) is never drawn, so every position is a valid token."""
    rng = np.random.default_rng(SPLIT_SEEDS.get(split, split if isinstance(split, int) else 0))
    ids = rng.integers(low, vocab_size, size=(n_samples, seq_len), dtype=np.int64).astype(np.int32)
    if padding_id is not None and low <= padding_id < vocab_size:
        repl = (padding_id + 1) % vocab_size if (padding_id + 1) % vocab_size >= low else low
        ids[ids == padding_id] = repl
    return ids


def iter_jsonl_gz(path: str):
    with gzip.open(path, "rt", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                yield json.loads(line)["input_ids"]


def load_input_ids_from_dir(directory: str, max_samples: int = 100000):
    """All ``input_ids`` lists from ``*.jsonl.gz`` under ``directory`` (sorted), up to max_samples."""
    out = []
    for p in sorted(glob.glob(os.path.join(directory, "*.jsonl.gz"))):
        for ids in iter_jsonl_gz(p):
            out.append(ids)
            if len(out) >= max_samples:
                return out
    return out


def load_input_ids_from_drive(remote: str = "gdrive:sample_dataset1024tokens80kvocab", max_samples: int = 100000,
                              local_fallback: str | None = None):
    """Stream records through ``rclone cat`` as the reference does (model/ZeRO3.py:628-647). Without
    the ``rclone`` binary the local directory ``local_fallback`` is read instead."""
    if shutil.which("rclone") is None:
        if local_fallback is not None:
            return load_input_ids_from_dir(local_fallback, max_samples)
        raise RuntimeError("rclone is not installed and no local_fallback directory was given")
    names = subprocess.run(["rclone", "lsf", remote, "--include", "*.jsonl.gz"], check=True, capture_output=True,
                           text=True).stdout.split()
    out = []
    for name in sorted(names):
        proc = subprocess.Popen(["rclone", "cat", f"{remote}/{name}"], stdout=subprocess.PIPE)
        with gzip.open(proc.stdout, "rt", encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    out.append(json.loads(line)["input_ids"])
                    if len(out) >= max_samples:
                        proc.kill()
                        return out
        if proc.wait() != 0:
            raise RuntimeError(f"rclone cat {remote}/{name} failed")
    return out


# --------------------------------------------------------------------------- batching
def valid_length(ids, padding_id: int) -> int:
    """Index of the first pad token, or the length when there is none (model/ZeRO3.py:251-257)."""
    arr = np.asarray(ids)
    hit = np.nonzero(arr == padding_id)[0]
    return int(hit[0]) if hit.size else int(arr.shape[0])


def to_fixed_length(samples, time_size: int, padding_id: int) -> tuple[np.ndarray, np.ndarray]:
    """Right-pad / truncate to ``time_size``; returns (ids [N, T] int32, valid_len [N] int32)."""
    N = len(samples)
    ids = np.full((N, time_size), padding_id, dtype=np.int32)
    vl = np.zeros(N, dtype=np.int32)
    for i, s in enumerate(samples):
        s = np.asarray(s, dtype=np.int32)[:time_size]
        ids[i, :len(s)] = s
        vl[i] = valid_length(ids[i], padding_id)
    return ids, vl


def data_shuffle(ids: np.ndarray, vl: np.ndarray, seed: int | None = None):
    perm = np.random.default_rng(seed).permutation(len(ids))
    return ids[perm], vl[perm]


def shard_for_rank(ids: np.ndarray, vl: np.ndarray, rank: int, world_size: int):
    """Rank r keeps samples r, r + W, r + 2W, ... (the reference feeds every rank the same data)."""
    return ids[rank::world_size], vl[rank::world_size]


def get_batch(ids: np.ndarray, vl: np.ndarray, batch_size: int, time_idx: int):
    """Strided batch as in the reference (model/ZeRO3.py:32-49): row i starts at offset
    ``i * (N // batch_size)`` and advances by one sample per call. Returns (x, valid_len, next idx)."""
    N = len(ids)
    jump = max(N // batch_size, 1)
    rows = [(i * jump + time_idx) % N for i in range(batch_size)]
    return ids[rows], vl[rows], time_idx + 1


def padding_proceccing(xdata, xvalid, padding_ID: int, out=None):
    """Build model inputs from raw samples (model/ZeRO3.py:52-65; the spelling is the reference's):

      * the last valid token of each row is replaced by the pad id (it has no target),
      * targets are the ids shifted left by one with a pad appended,
      * ``x_pa = valid_len - 1`` is the number of attendable keys.

    Returns torch int32 tensors (x [B, T], t [B, T], x_pa [B]); when ``out`` gives pinned tensors they
    are filled in place."""
    x = np.array(xdata, dtype=np.int32, copy=True)
    B, T = x.shape
    x_pa = np.maximum(np.asarray(xvalid, dtype=np.int32) - 1, 0)
    t = np.concatenate([x[:, 1:], np.full((B, 1), padding_ID, dtype=np.int32)], axis=1)
    x[np.arange(B), x_pa] = padding_ID
    # targets at and after the last valid input position carry no loss
    pos = np.arange(T)[None, :]
    t[pos >= x_pa[:, None]] = padding_ID
    if out is None:
        return torch.from_numpy(x), torch.from_numpy(t), torch.from_numpy(x_pa)
    out[0].copy_(torch.from_numpy(x))
    out[1].copy_(torch.from_numpy(t))
    out[2].copy_(torch.from_numpy(x_pa))
    return out


class BatchStager:
    """Pinned host staging for micro-batches and their asynchronous copy to the device.

    A small ring of pinned buffer sets: the host may run several steps ahead of the device, so the set of
    micro-batch i must not be rewritten before its host-to-device copy has executed. Every set carries the event
    of its last copy, and the host waits for that event (normally long past) before it reuses the set."""

    def __init__(self, batch_size: int, time_size: int, device, depth: int = 4):
        self.device = torch.device(device)
        pin = self.device.type == "cuda"

        def make():
            return (torch.empty((batch_size, time_size), dtype=torch.int32, pin_memory=pin),
                    torch.empty((batch_size, time_size), dtype=torch.int32, pin_memory=pin),
                    torch.empty((batch_size,), dtype=torch.int32, pin_memory=pin))
        self.ring = [[make(), None] for _ in range(max(int(depth), 1) if pin else 1)]
        self.pos = 0
        self.host = self.ring[0][0]
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in self.host)

    def stage(self, xdata, xvalid, padding_ID: int):
        slot = self.ring[self.pos]
        self.pos = (self.pos + 1) % len(self.ring)
        host, ev = slot
        if ev is not None:
            ev.synchronize()                     # the copy that last read this set has run
        padding_proceccing(xdata, xvalid, padding_ID, out=host)
        if self.device.type != "cuda":
            return tuple(t.clone() for t in host)
        out = tuple(t.to(self.device, non_blocking=True) for t in host)
        slot[1] = torch.cuda.Event()
        slot[1].record(torch.cuda.current_stream(self.device))
        return out


class SplitDataset:
    """Train / Validation / Generation split of one token source (README of the reference: "data
    split: Train, Validation, Generation"). Validation = the first ``n_val`` samples of the
    shuffled pool, held fixed; generation prompts = the next ``n_gen`` samples; the rest trains."""

    def __init__(self, ids: np.ndarray, vl: np.ndarray, n_val: int, n_gen: int = 0, seed: int = 0):
        ids, vl = data_shuffle(ids, vl, seed)
        self.val = (ids[:n_val], vl[:n_val])
        self.gen = (ids[n_val:n_val + n_gen], vl[n_val:n_val + n_gen])
        self.train = (ids[n_val + n_gen:], vl[n_val + n_gen:])

    @classmethod
    def synthetic(cls, vocab_size: int, time_size: int, n_train: int, n_val: int, n_gen: int, padding_id: int):
        tr = synthetic_token_stream(n_train, time_size, vocab_size, "train", padding_id)
        va = synthetic_token_stream(n_val, time_size, vocab_size, "validation", padding_id)
        ge = synthetic_token_stream(n_gen, time_size, vocab_size, "generation", padding_id)
        obj = cls.__new__(cls)
        full = lambda a: (a, np.full(len(a), time_size, dtype=np.int32))
        obj.train, obj.val, obj.gen = full(tr), full(va), full(ge)
        return obj
