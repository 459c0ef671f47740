"""Child of the multi-GPU tests: trains a small bf16 model for a few steps under ZeRO-3 with
either NCCL collectives or the fused peer-memory kernels and saves the loss curve."""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")     # see parallel.trainer.prefer_eager_module_loading

import numpy as np  # noqa: E402
import torch  # noqa: E402


def main():
    mode, out_path = sys.argv[1], sys.argv[2]
    from create_llm_by_cupy_b200.ops import native
    from create_llm_by_cupy_b200.parallel.comm import init_distributed, shutdown_distributed
    from create_llm_by_cupy_b200.parallel.trainer import Trainer
    from create_llm_by_cupy_b200.utils.data import padding_proceccing, synthetic_token_stream

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = init_distributed(rank, world, backend="nccl", device_id=local, master_port=int(os.environ["MASTER_PORT"]),
                            timeout_s=120)
    fused = None
    if mode == "fused":
        from create_llm_by_cupy_b200.parallel.symm import FusedCollectives
        fused = FusedCollectives(comm, dev, heap_bytes=512 << 20, wait_ns=5_000_000_000,
                                 gather_mode=os.environ.get("B200_TEST_GATHER", "copy"),
                                 reduce_mode=os.environ.get("B200_TEST_REDUCE", "copy"),
                                 copy_min_bytes=int(os.environ.get("B200_TEST_COPY_MIN", str(1 << 20))))
    accum = int(os.environ.get("B200_TEST_ACCUM", "2"))
    md = dict(vocab_size=2048, hidden_size=256, layer_num=3, time_size=256, q_head=4, kv_head=2, ffn_size=688,
              padding_id=0, dropout_rate=0, dtype="bf16", half_float=True, tie_embeddings=True, init_std=0.02, seed=1,
              grad_bucket_elems=int(os.environ.get("B200_TEST_BUCKET", "300000")),     # blocks are reduced in parts,
              zero3_early_bucket_flush=True)                                           # the MLP part ahead of the rest
    fused_adam = os.environ.get("B200_TEST_FUSED_ADAM", "0") == "1"
    tr = Trainer(md, rank=rank, world_size=world, comm=comm, device=dev, accum_step=accum, lr_max=1e-3, warm_up=1,
                 total_steps=6, beta2=0.95, fused=fused, profile_comm=True, fused_adam=fused_adam,
                 max_grads=0.0 if fused_adam or os.environ.get("B200_TEST_NOCLIP") == "1" else 1.0)
    assert tr.fused_adam == (fused_adam and fused is not None)
    B = 2
    ids = synthetic_token_stream(6 * accum * B * world, 256, 2048, "train", 0, low=1)[rank::world]
    losses = []
    for s in range(6):
        bs = []
        for a in range(accum):
            chunk = ids[(s * accum + a) * B:(s * accum + a + 1) * B]
            bs.append(tuple(v.to(dev) for v in padding_proceccing(chunk, np.full(B, 256), 0)))
        losses.append(tr.train_step(bs)["loss"])
    tr.manager.synchronize()
    native.raise_on_status()
    loss_t = torch.tensor(losses, device=dev)
    comm.all_reduce(loss_t)
    pn = tr.manager.calculate_global_param_norm()
    if rank == 0:
        torch.save({"losses": (loss_t / world).tolist(), "param_norm": pn,
                    "exposed_ms": tr.manager.exposed_comm_ms()}, out_path)
    comm.barrier()
    tr.close()                      # frees the heap; raises if a guard block around an allocation was overwritten
    shutdown_distributed()


if __name__ == "__main__":
    main()
