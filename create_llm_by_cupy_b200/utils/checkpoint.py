"""Checkpoint write / read / convert.

Written files keep the reference's per-rank layout and key names (model/ZeRO3.py:469-497,
model/ZeRO2_5.py:499-538):

    model_shard_rank{r}.pkl.gz : param_shard_f16, rank, world_size, shard_size, padded_total,
                                 param_offsets, param_shapes, param_sizes
                                 (+ replica_param_f16, replica_offsets, replica_total,
                                  replica_padded_total, replica_opt_shard_size,
                                  replicated_param_indices, zero25_replica_ratio for ZeRO-2.5)
    optimizer_rank{r}.pkl.gz   : m, v, w_fp32, t (+ replica_m, replica_v, replica_w_fp32, replica_t)

plus what the reference lacks: a ``dtype`` key (bf16 payloads are stored as raw uint16 bits), the
unit layout description, trainer state (iteration, loss scale, RNG), atomic writes (temp file +
rename), a loader for these shard files, shards -> flat and flat -> shards converters and
re-sharding to another world size. The reference can only read one flat fp16 array of all
parameters (model/model.py:551-571); that format is still read and written
(``Cupa_ver4.load_weights_from_flat_file`` / ``save_weights_to_flat_file``).
"""
from __future__ import annotations

import gzip
import os
import pickle
import shutil
import subprocess

import numpy as np
import torch

from ..parallel.layout import FlatLayout


# --------------------------------------------------------------------------- tensor <-> numpy
def _to_np(t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), "bf16"
    if t.dtype == torch.float16:
        return t.numpy(), "fp16"
    return t.float().numpy(), "fp32"


def _from_np(a, dtype_name: str) -> torch.Tensor:
    a = np.asarray(a)
    if dtype_name == "bf16":
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    if dtype_name == "fp16":
        return torch.from_numpy(a.astype(np.float16))
    return torch.from_numpy(a.astype(np.float32))


def atomic_pickle_gzip(obj, path: str, compresslevel: int = 1):
    """Write ``obj`` to ``path`` so that a crash never leaves a half-written file in its place."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = f"{path}.tmp.{os.getpid()}"
    with gzip.open(tmp, "wb", compresslevel=compresslevel) as f:
        pickle.dump(obj, f, protocol=pickle.HIGHEST_PROTOCOL)
        f.flush()
    os.replace(tmp, path)


def read_pickle_gzip(path: str):
    with gzip.open(path, "rb") as f:
        return pickle.load(f)


def save_pickle_gzip_to_drive(obj, remote_path: str, local_dir: str | None = None):
    """Reference behaviour (model/ZeRO3.py:520-544): stream to ``rclone rcat``. Used only when
    ``rclone`` exists; otherwise (or additionally, with ``local_dir``) the file is written locally."""
    name = os.path.basename(remote_path)
    if local_dir is not None or shutil.which("rclone") is None:
        atomic_pickle_gzip(obj, os.path.join(local_dir or ".", name))
        if shutil.which("rclone") is None:
            return
    proc = subprocess.Popen(["rclone", "rcat", remote_path], stdin=subprocess.PIPE)
    with gzip.GzipFile(fileobj=proc.stdin, mode="wb") as gz:
        pickle.dump(obj, gz, protocol=pickle.HIGHEST_PROTOCOL)
    proc.stdin.close()
    if proc.wait() != 0:
        raise RuntimeError(f"rclone rcat {remote_path} failed")


# --------------------------------------------------------------------------- save / load shards
def model_shard_path(d: str, rank: int) -> str:
    return os.path.join(d, f"model_shard_rank{rank}.pkl.gz")


def optimizer_path(d: str, rank: int) -> str:
    return os.path.join(d, f"optimizer_rank{rank}.pkl.gz")


def trainer_state_path(d: str) -> str:
    return os.path.join(d, "trainer_state.pkl.gz")


def save_checkpoint(directory: str, manager, optimizer, replica_optimizer=None, trainer_state: dict | None = None):
    """Every rank writes its own two files; rank 0 also writes the trainer state."""
    r = manager.rank
    arr, dt = _to_np(manager.param_shard_f16)
    desc = manager.layout.describe()
    shard = {"param_shard_f16": arr, "dtype": dt, "rank": r, "world_size": manager.world_size,
             "shard_size": manager.shard_size, "padded_total": manager.padded_total,
             "param_offsets": desc["param_offsets"], "param_shapes": desc["param_shapes"],
             "param_sizes": desc["param_sizes"], "layout": desc}
    if manager.replica_param_f16 is not None:
        rarr, _ = _to_np(manager.replica_param_f16)
        shard.update({"replica_param_f16": rarr, "replica_offsets": desc["replica_offsets"],
                      "replica_total": desc["replica_total"], "replica_padded_total": desc["replica_padded_total"],
                      "replica_opt_shard_size": desc["replica_opt_shard_size"],
                      "replicated_param_indices": desc["replicated_param_indices"],
                      "zero25_replica_ratio": manager.replica_ratio})
    atomic_pickle_gzip(shard, model_shard_path(directory, r))
    sd = optimizer.state_dict()
    opt = {"m": sd["m"].detach().cpu().numpy(), "v": sd["v"].detach().cpu().numpy(),
           "w_fp32": sd["w_fp32"].detach().cpu().numpy(), "t": int(sd["t"])}
    if replica_optimizer is not None:
        rs = replica_optimizer.state_dict()
        opt.update({"replica_m": rs["m"].detach().cpu().numpy(), "replica_v": rs["v"].detach().cpu().numpy(),
                    "replica_w_fp32": rs["w_fp32"].detach().cpu().numpy(), "replica_t": int(rs["t"])})
    atomic_pickle_gzip(opt, optimizer_path(directory, r))
    if r == 0 and trainer_state is not None:
        atomic_pickle_gzip(trainer_state, trainer_state_path(directory))


def load_checkpoint(directory: str, manager, optimizer=None, replica_optimizer=None) -> dict | None:
    """Restore this rank's parameter shard (and optimizer state) from files written with the same
    world size and layout. Returns the trainer state dict if present."""
    shard = read_pickle_gzip(model_shard_path(directory, manager.rank))
    if shard["world_size"] != manager.world_size or shard["shard_size"] != manager.shard_size:
        raise ValueError(f"checkpoint was written for world_size={shard['world_size']} shard_size="
                         f"{shard['shard_size']}; use reshard_checkpoint() first")
    manager.param_shard_f16.copy_(_from_np(shard["param_shard_f16"], shard.get("dtype", "fp16")).to(manager.dtype))
    if manager.replica_param_f16 is not None and "replica_param_f16" in shard:
        manager.replica_param_f16.copy_(_from_np(shard["replica_param_f16"], shard.get("dtype", "fp16")).to(manager.dtype))
    have_opt = os.path.exists(optimizer_path(directory, manager.rank))
    opt = read_pickle_gzip(optimizer_path(directory, manager.rank)) if have_opt else {}
    if optimizer is not None:
        if have_opt:
            optimizer.load_state_dict({k: torch.from_numpy(np.asarray(opt[k])) if k != "t" else opt[k]
                                       for k in ("m", "v", "w_fp32", "t")})
        else:
            # Weights without optimizer state (flat_to_shards, reshard_checkpoint(with_optimizer=False)): the
            # fp32 master must follow the loaded shard, or the first AdamW step would write back values
            # derived from the master of the randomly initialised model.
            optimizer.reseed_from_params(manager.param_shard_f16)
    if replica_optimizer is not None:
        if "replica_m" in opt:
            replica_optimizer.load_state_dict({"m": torch.from_numpy(np.asarray(opt["replica_m"])),
                                               "v": torch.from_numpy(np.asarray(opt["replica_v"])),
                                               "w_fp32": torch.from_numpy(np.asarray(opt["replica_w_fp32"])),
                                               "t": opt["replica_t"]})
        else:
            replica_optimizer.reseed_from_params(manager.get_replica_optimizer_shard_view())
    p = trainer_state_path(directory)
    return read_pickle_gzip(p) if os.path.exists(p) else None


# --------------------------------------------------------------------------- converters
def _layout_from_desc(desc: dict, world_size: int | None = None) -> FlatLayout:
    unit_defs = [(u["name"], u["param_indices"]) for u in desc["units"]]
    return FlatLayout.build(desc["param_shapes"], unit_defs, world_size or desc["world_size"],
                            desc["replicated_param_indices"])


def shards_to_param_list(directory: str, world_size: int | None = None) -> list:
    """Read every rank's model shard and return the full parameters (fp32 tensors, params order)."""
    first = read_pickle_gzip(model_shard_path(directory, 0))
    W = world_size or first["world_size"]
    desc = first["layout"]
    lay = _layout_from_desc(desc)
    shards = [first] + [read_pickle_gzip(model_shard_path(directory, r)) for r in range(1, W)]
    flat = [_from_np(s["param_shard_f16"], s.get("dtype", "fp16")).float() for s in shards]
    out = []
    rep = _from_np(first["replica_param_f16"], first.get("dtype", "fp16")).float() if "replica_param_f16" in first else None
    for slot in lay.slots:
        if slot.unit < 0:
            out.append(rep[slot.offset:slot.offset + slot.size].view(slot.shape).clone())
            continue
        unit = lay.units[slot.unit]
        sl = unit.padded // W
        full = torch.cat([f[unit.shard_offset:unit.shard_offset + sl] for f in flat])
        out.append(full[slot.offset:slot.offset + slot.size].view(slot.shape).clone())
    return out


def shards_to_flat(directory: str, out_path: str):
    """Per-rank shard files -> one flat fp16 array in ``params`` order (the reference's resume
    format, readable by ``Cupa_ver4(model_dic, param_path=...)``)."""
    params = shards_to_param_list(directory)
    flat = torch.cat([p.reshape(-1) for p in params]).numpy().astype(np.float16)
    atomic_pickle_gzip(flat, out_path)
    return flat.size


def flat_to_shards(flat_path: str, directory: str, param_shapes, unit_defs, world_size: int,
                   replicated=(), dtype_name: str = "bf16"):
    """One flat array in ``params`` order -> per-rank model shard files for ``world_size`` ranks."""
    flat = torch.from_numpy(np.asarray(read_pickle_gzip(flat_path)).astype(np.float32))
    lay = FlatLayout.build(param_shapes, unit_defs, world_size, replicated)
    params, off = [], 0
    for slot in lay.slots:
        params.append(flat[off:off + slot.size])
        off += slot.size
    _write_model_shards(directory, lay, params, dtype_name)


def _write_model_shards(directory: str, lay: FlatLayout, params, dtype_name: str, ratio: float = 0.0):
    W = lay.world_size
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[dtype_name]
    shards = [torch.zeros(lay.shard_size, dtype=torch.float32) for _ in range(W)]
    for uid, unit in enumerate(lay.units):
        if unit.empty:
            continue
        full = torch.zeros(unit.padded, dtype=torch.float32)
        for i in unit.param_indices:
            s = lay.slots[i]
            if s.unit == uid:
                full[s.offset:s.offset + s.size] = params[i].reshape(-1).float()
        sl = unit.padded // W
        for r in range(W):
            shards[r][unit.shard_offset:unit.shard_offset + sl] = full[r * sl:(r + 1) * sl]
    rep = None
    if lay.replica_padded_total:
        rep = torch.zeros(lay.replica_padded_total, dtype=torch.float32)
        for i in lay.replicated_param_indices:
            s = lay.slots[i]
            rep[s.offset:s.offset + s.size] = params[i].reshape(-1).float()
    desc = lay.describe()
    for r in range(W):
        arr, dt = _to_np(shards[r].to(tdt))
        shard = {"param_shard_f16": arr, "dtype": dt, "rank": r, "world_size": W, "shard_size": lay.shard_size,
                 "padded_total": lay.padded_total, "param_offsets": desc["param_offsets"],
                 "param_shapes": desc["param_shapes"], "param_sizes": desc["param_sizes"], "layout": desc}
        if rep is not None:
            rarr, _ = _to_np(rep.to(tdt))
            shard.update({"replica_param_f16": rarr, "replica_offsets": desc["replica_offsets"],
                          "replica_total": desc["replica_total"], "replica_padded_total": desc["replica_padded_total"],
                          "replica_opt_shard_size": desc["replica_opt_shard_size"],
                          "replicated_param_indices": desc["replicated_param_indices"],
                          "zero25_replica_ratio": ratio})
        atomic_pickle_gzip(shard, model_shard_path(directory, r))


def reshard_checkpoint(src_dir: str, dst_dir: str, new_world_size: int, with_optimizer: bool = True):
    """Rewrite a checkpoint for a different number of ranks (offline elastic recovery). Model
    shards and, if present, the sharded optimizer state (m, v, fp32 master) are re-cut; replicated
    parameters are carried over unchanged."""
    first = read_pickle_gzip(model_shard_path(src_dir, 0))
    old_W = first["world_size"]
    desc = first["layout"]
    params = shards_to_param_list(src_dir)
    new_lay = _layout_from_desc(desc, new_world_size)
    _write_model_shards(dst_dir, new_lay, params, first.get("dtype", "bf16"),
                        first.get("zero25_replica_ratio", 0.0))
    if with_optimizer and os.path.exists(optimizer_path(src_dir, 0)):
        old_lay = _layout_from_desc(desc)
        opts = [read_pickle_gzip(optimizer_path(src_dir, r)) for r in range(old_W)]
        new_opts = [{"t": opts[0]["t"]} for _ in range(new_world_size)]
        for key in ("m", "v", "w_fp32"):
            outs = [np.zeros(new_lay.shard_size, dtype=np.float32) for _ in range(new_world_size)]
            for uid, unit in enumerate(old_lay.units):
                if unit.empty:
                    continue
                sl = unit.padded // old_W
                full = np.concatenate([np.asarray(o[key])[unit.shard_offset:unit.shard_offset + sl] for o in opts])
                nu = new_lay.units[uid]
                nfull = np.zeros(nu.padded, dtype=np.float32)
                n = min(len(full), nu.padded)
                nfull[:n] = full[:n]
                nsl = nu.padded // new_world_size
                for r in range(new_world_size):
                    outs[r][nu.shard_offset:nu.shard_offset + nsl] = nfull[r * nsl:(r + 1) * nsl]
            for r in range(new_world_size):
                new_opts[r][key] = outs[r]
        if "replica_m" in opts[0]:
            n_old = old_lay.replica_opt_shard_size
            n_new = new_lay.replica_opt_shard_size
            for key in ("replica_m", "replica_v", "replica_w_fp32"):
                full = np.concatenate([np.asarray(o[key])[:n_old] for o in opts])
                buf = np.zeros(new_lay.replica_padded_total, dtype=np.float32)
                n = min(len(full), len(buf))
                buf[:n] = full[:n]
                for r in range(new_world_size):
                    new_opts[r][key] = buf[r * n_new:(r + 1) * n_new]
            for r in range(new_world_size):
                new_opts[r]["replica_t"] = opts[0]["replica_t"]
        for r in range(new_world_size):
            atomic_pickle_gzip(new_opts[r], optimizer_path(dst_dir, r))
    ts = trainer_state_path(src_dir)
    if os.path.exists(ts):
        os.makedirs(dst_dir, exist_ok=True)
        shutil.copyfile(ts, trainer_state_path(dst_dir))
