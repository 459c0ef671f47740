"""ZeRO-2.5 training entry point (counterpart of the reference's Main/main_sample2.5.py).

A configurable share of the parameters stays replicated on every rank (no gather in forward or
backward); their gradients and optimizer state are still sharded. Defaults describe the ~1.3 B GQA decoder on the GPUs of one NVLink/NVSwitch box; every value can
be overridden on the command line, e.g. a CPU smoke run:

    python Main/main_sample2.5.py --devices 0 --layers 2 --hidden 128 --q-heads 4 --kv-heads 2 \
        --ffn 512 --vocab 512 --seq 128 --batch 4 --data-size 64 --backend gloo

NCCL is left on its defaults: NVLink peer-to-peer through NVSwitch is the transport this stack is
built for (the reference disables P2P and InfiniBand and forces the socket transport because it
targets a PCIe workstation, Main/main_sample3.py:4-14).
"""
import argparse
import os
import sys

sys.path.append(os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

from model.ZeRO2_5 import TrainMultiGPU  # noqa: E402


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--devices", default=None, help="comma-separated device ids (default: all visible GPUs, or 0)")
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--q-heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--ffn", type=int, default=5504)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--accum", type=int, default=1)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--data-size", type=int, default=10_000_000)
    ap.add_argument("--data-dir", default=None, help="directory of *.jsonl.gz with input_ids (default: synthetic)")
    ap.add_argument("--optimizer-device", default="gpu", choices=["gpu", "cpu"])
    ap.add_argument("--save-dir", default=None)
    ap.add_argument("--resume-dir", default=None)
    ap.add_argument("--backend", default=None)
    ap.add_argument("--wandb", action="store_true")
    ap.add_argument("--collectives", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU data plane: peer-memory kernels / copy engines over NVLink (default) or NCCL")
    ap.add_argument("--gather", default="copy", choices=["copy", "pull", "gemm", "nccl"],
                    help="parameter gather with --collectives fused: copy engines, P2P pull kernel, inside the "
                         "consuming GEMM, or ncclAllGather")
    ap.add_argument("--reduce", default="copy", choices=["copy", "pull"],
                    help="gradient reduce-scatter with --collectives fused: copy engines + a local summing kernel, "
                         "or the kernel that pulls the peers' slices while it sums")
    ap.add_argument("--validate-every", type=int, default=0,
                    help="validation loss and a generation sample every N iterations (0: off)")
    ap.add_argument("--replica-ratio", type=float, default=0.25, help="fraction of parameter elements kept replicated")
    ap.add_argument("--replica-policy", default="largest_first",
                    choices=["largest_first", "first", "last", "embedding_first"])
    return ap.parse_args()


if __name__ == "__main__":
    a = parse()
    if a.devices is None:
        import torch
        use_devices = list(range(torch.cuda.device_count())) or [0]
    else:
        use_devices = [int(v) for v in a.devices.split(",")]
    padding_id = 2
    model_dic = {
        "vocab_size": a.vocab, "hidden_size": a.hidden, "dropout_rate": 0, "layer_num": a.layers,
        "time_size": a.seq, "q_head": a.q_heads, "kv_head": a.kv_heads, "padding_id": padding_id,
        "half_float": True, "ffn_size": a.ffn, "tie_embeddings": True, "rope_base": 10000.0,
        # memory / communication knobs (same names as the reference)
        "keep_layer_num": 1, "keep_embedding_until_backward": True, "ce_chunk_size": 8192,
        "gqa_cache_out_value": True, "swiglu_cache_gate": True,
        "zero3_param_prefetch": True, "zero3_grad_bucket": True, "zero3_max_pending_reduces": 8,
        "zero25_replica_ratio": a.replica_ratio, "zero25_replica_policy": a.replica_policy,
        "grad_bucket_elems": 25_000_000, "zero3_sync_gather": False, "flash_backend": "b200",
        "zero3_fused_collectives": a.collectives == "fused", "zero3_gather_mode": a.gather, "zero3_reduce_mode": a.reduce,
    }
    if a.backend == "gloo":
        model_dic.update(dtype="fp32", half_float=False)
    GradScale_dic = {"StartScale": 10, "UpRate": 2.0, "DownRate": 0.7, "Scale_Up_Step": 10, "enabled": False}
    trainer = TrainMultiGPU(
        model_dic, GradScale_dic, use_devices=use_devices, batch_size=a.batch, max_epoch=a.epochs,
        lr_max=3e-4, lr_mini=3e-5, weight_decay=0.1, warm_up=1000, max_grads=1.0, accum_step=a.accum,
        save=a.save_dir is not None, save_step=2000, vali=a.validate_every > 0, vali_step=max(a.validate_every, 1), wand=a.wandb,
        optimizer_device=a.optimizer_device, train_continue_path=None, data_dir=a.data_dir, save_dir=a.save_dir,
        resume_dir=a.resume_dir, backend=a.backend, beta1=0.9, beta2=0.95)
    trainer.fit(a.data_size)
