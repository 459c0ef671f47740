"""Workers for the multi-process CPU (gloo) tests. Importable so that ``spawn`` can find them."""
import os
import pickle
import sys
import traceback

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

TINY = dict(vocab_size=64, hidden_size=32, layer_num=3, time_size=16, q_head=4, kv_head=2, padding_id=2,
            dropout_rate=0, half_float=False, dtype="fp32", ffn_size=48, tie_embeddings=True, seed=5,
            ce_chunk_size=40)
HP = dict(lr_max=3e-3, lr_mini=3e-4, weight_decay=0.1, warm_up=2, total_steps=8, beta1=0.9, beta2=0.95,
          epsilon=1e-6, max_grads=1.0)
GLOBAL_B = 8


def make_batches(n_steps, rank, world, accum=1):
    import numpy as np
    from create_llm_by_cupy_b200.utils.data import padding_proceccing, synthetic_token_stream

    ids = synthetic_token_stream(n_steps * GLOBAL_B, TINY["time_size"], TINY["vocab_size"], "train", TINY["padding_id"], low=3)
    out = []
    per_rank = GLOBAL_B // world
    micro = per_rank // accum
    for s in range(n_steps):
        chunk = ids[s * GLOBAL_B:(s + 1) * GLOBAL_B][rank * per_rank:(rank + 1) * per_rank]
        out.append([padding_proceccing(chunk[a * micro:(a + 1) * micro], np.full(micro, TINY["time_size"]), TINY["padding_id"])
                    for a in range(accum)])
    return out


def train_worker(rank, world, port, out_dir, cfg):
    try:
        import torch
        from create_llm_by_cupy_b200.parallel.comm import init_distributed, shutdown_distributed
        from create_llm_by_cupy_b200.parallel.trainer import Trainer

        torch.set_num_threads(1)
        comm = init_distributed(rank, world, backend="gloo", master_port=port, timeout_s=cfg.get("timeout_s", 120))
        md = dict(TINY, **cfg.get("model", {}))
        tr = Trainer(md, rank=rank, world_size=world, comm=comm, device="cpu", zero_stage=cfg.get("zero", "3"),
                     optimizer_device=cfg.get("opt", "gpu"), accum_step=cfg.get("accum", 1), **HP)
        losses = []
        for bs in make_batches(cfg.get("steps", 4), rank, world, cfg.get("accum", 1)):
            losses.append(tr.train_step(bs)["loss"])
        if cfg.get("save_dir"):
            tr.save(cfg["save_dir"])
        tr.manager.materialize_all()
        params = [p.detach().clone().numpy() for p in tr.model.params]
        tr.manager.release_all()
        with open(os.path.join(out_dir, f"r{rank}.pkl"), "wb") as f:
            pickle.dump({"losses": losses, "params": params, "gathered": tr.manager.bytes_gathered,
                         "reduced": tr.manager.bytes_reduced, "replicated": tr.manager.replicated_param_indices}, f)
        if world > 1:
            comm.barrier()
            shutdown_distributed()
    except BaseException:
        traceback.print_exc()
        os._exit(3)


def run_spawn(fn, world, *args, timeout=240):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    port = 20000 + (os.getpid() * 7 + world * 131 + run_spawn.counter * 17) % 20000
    run_spawn.counter += 1
    procs = [ctx.Process(target=fn, args=(r, world, port) + args) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    codes = []
    for p in procs:
        if p.is_alive():
            p.terminate()
            p.join(5)
            codes.append("timeout")
        else:
            codes.append(p.exitcode)
    return codes


run_spawn.counter = 0
