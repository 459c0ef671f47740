"""Headline benchmark: training tokens/s of the ~1.3 B GQA decoder under ZeRO-3 on N B200s.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (weak scaling, per-GPU work fixed): vocab 32000, d_model 2048, 24 layers, 16 query / 4 KV
heads, head_dim 128, SwiGLU FFN 5504, seq 2048, micro-batch 4 per GPU, bf16 compute with fp32
master weights and AdamW state sharded; synthetic uniform-random token ids (seed 0), random-init
N(0, 0.02) weights. A step = forward + backward + gradient reduction + global-norm clip + AdamW.

Three numbers are measured, each over exactly K steps after W warm-up steps, bracketed by a barrier
and a device synchronise, timed with CUDA events, max over ranks:
  value    : the step with its inputs already resident on the device;
  e2e      : the same step driven through the public ``Trainer.train_step`` API with every step's
             token ids copied from pinned host memory and every step's loss read back to the host;
  baseline : this framework's own plain path on the same box, in the same process, after the two
             above: NCCL all-gather / reduce-scatter instead of the peer-memory collectives, AdamW as
             one kernel after the backward, rotary embedding / SwiGLU / loss statistics as separate
             kernels, weight gradients on the main stream. ``vs_baseline`` = value / baseline value (the
             reference itself cannot run here: it needs CuPy, see ``--impl reference``).
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

CONFIGS = {
    "1.3b": dict(vocab_size=32000, hidden_size=2048, layer_num=24, q_head=16, kv_head=4, ffn_size=5504,
                 time_size=2048, micro_batch=4, accum=1, zero="3", opt="gpu", name="1.3B-GQA-ZeRO3"),
    "125m": dict(vocab_size=32000, hidden_size=768, layer_num=12, q_head=12, kv_head=4, ffn_size=2048,
                 time_size=1024, micro_batch=8, accum=1, zero="2.5", opt="gpu", name="125M-GQA-ZeRO2.5"),
    "7b": dict(vocab_size=32000, hidden_size=4096, layer_num=32, q_head=32, kv_head=8, ffn_size=11008,
               time_size=4096, micro_batch=1, accum=8, zero="3", opt="cpu", name="7B-Llama-ZeRO3-offload"),
    "tiny": dict(vocab_size=512, hidden_size=128, layer_num=2, q_head=4, kv_head=2, ffn_size=512,
                 time_size=128, micro_batch=4, accum=1, zero="3", opt="gpu", name="tiny"),
}


def reference_arm(args):
    """The reference needs CuPy (``cupy``, ``cupy.cuda.nccl``) for every tensor op and collective
    and shells out to ``rclone`` for its data; neither exists in this image and there is no index
    to install from, so its stock code path cannot run here."""
    why = None
    try:
        import cupy  # noqa: F401
    except Exception as e:
        why = f"reference imports cupy at module load (model/ZeRO3.py:1-7) and cupy is not installable offline: {e}"
    if why is None:
        why = "reference harness not wired: its data loader requires the rclone binary and Google Drive"
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="1.3b", choices=sorted(CONFIGS))
    ap.add_argument("--fused", type=int, default=-1, help="1: fused peer-memory collectives, 0: NCCL baseline, -1: auto")
    ap.add_argument("--ag", default="copy", choices=["nccl", "pull", "gemm", "copy"],
                    help="parameter gather with --fused: copy engines (cudaMemcpyAsync per peer slice), P2P pull "
                         "kernel, NCCL all-gather, or pulled inside the consuming GEMM")
    ap.add_argument("--rs", default="copy", choices=["pull", "copy"],
                    help="gradient reduce-scatter: peer loads inside the summing kernel, or copy engines + a local kernel")
    ap.add_argument("--one-comm-stream", action="store_true",
                    help="A/B: parameter gathers on the stream of the gradient reductions instead of their own")
    ap.add_argument("--parallel-copies", action="store_true",
                    help="A/B: the peer copies of a gather / reduction side by side on helper streams")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-baseline", action="store_true", help="skip the plain-path arm (vs_baseline stays null)")
    ap.add_argument("--sync-read", action="store_true", help="read the loss of every step before the next one starts")
    ap.add_argument("--no-adam-overlap", action="store_true", help="AdamW as one kernel after the backward")
    ap.add_argument("--keep-params", action="store_true",
                    help="keep gathered block parameters from the forward until their backward (one GPU only)")
    ap.add_argument("--opt", default=None, choices=["gpu", "cpu"], help="override the config's optimizer tier")
    ap.add_argument("--delayed-offload", action="store_true",
                    help="host optimizer (--opt cpu / config 7b): one-step delayed parameter update, the host AdamW "
                         "runs under the next step's forward and backward")
    ap.add_argument("--graph", action="store_true", help="capture the whole step in a CUDA graph (one GPU)")
    ap.add_argument("--no-phases", action="store_true", help="do not record the per-phase CUDA events")
    ap.add_argument("--comm-blocks", type=int, default=0, help="CTAs of the fused collective kernels (0: default)")
    ap.add_argument("--bucket-elems", type=int, default=25_000_000,
                    help="largest reduce-scatter launch in elements (0: every unit's bucket is reduced in one launch)")
    ap.add_argument("--peer-wait-s", type=float, default=0.0,
                    help="budget of one cross-GPU wait of the fused collectives in seconds (0: the library default)")
    ap.add_argument("--adam-ctas", type=int, default=2, help="AdamW CTAs per SM while it runs beside the next forward")
    ap.add_argument("--early-flush", action="store_true",
                    help="reduce the MLP part of a block's gradient bucket before the block's backward has finished")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    # Libraries (NCCL's version banner, for one) write to file descriptor 1 directly; the contract is
    # ONE JSON line on stdout, so everything before the final print goes to stderr.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    if int(os.environ.get("WORLD_SIZE", 1)) > 1:
        # before CUDA is touched: no kernel is loaded lazily while kernels that wait for a peer are in flight
        os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
    import torch

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from create_llm_by_cupy_b200.ops import functional as F
    from create_llm_by_cupy_b200.ops import native
    from create_llm_by_cupy_b200.parallel.comm import init_distributed, shutdown_distributed
    from create_llm_by_cupy_b200.parallel.trainer import Trainer
    from create_llm_by_cupy_b200.utils.data import BatchStager, synthetic_token_stream
    from create_llm_by_cupy_b200.utils.profiler import ClockSampler

    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    comm = init_distributed(rank, world, backend="nccl", device_id=local_rank,
                            master_port=int(os.environ.get("MASTER_PORT", 29511)))

    c = dict(CONFIGS[args.config])
    if args.opt is not None:
        c["opt"] = args.opt
        c["name"] = c["name"] + ("-offload" if args.opt == "cpu" and "offload" not in c["name"] else "")
    pad = 0
    md = dict(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], layer_num=c["layer_num"],
              time_size=c["time_size"], q_head=c["q_head"], kv_head=c["kv_head"], ffn_size=c["ffn_size"],
              padding_id=pad, dropout_rate=0, half_float=True, dtype="bf16", tie_embeddings=True, init_std=0.02,
              seed=0, grad_bucket_elems=args.bucket_elems, zero3_early_bucket_flush=args.early_flush,
              zero3_gather_stream=not args.one_comm_stream)
    if c["zero"] == "2.5":
        md.update(zero25_replica_ratio=0.5, zero25_replica_policy="largest_first")
    if args.keep_params:
        if world > 1:
            raise SystemExit("--keep-params is a one-GPU option: on multi-GPU runs it is refused (one such run "
                             "did not finish and the cause is not established)")
        md.update(keep_params_until_backward=True)
    B, T, accum = c["micro_batch"], c["time_size"], c["accum"]
    n_steps_total = args.warmup + args.steps
    tokens = B * T * accum * world

    # distinct synthetic batches per rank and per step (seed 0 stream, partitioned by rank)
    ids = synthetic_token_stream(n_steps_total * accum * B * world, T, c["vocab_size"], "train", pad, low=1)
    ids = ids[rank::world]
    stager = BatchStager(B, T, device, depth=max(4, 2 * accum))
    vl = np.full(B, T, dtype=np.int32)

    def host_batch(i):
        return ids[i * B:(i + 1) * B]

    def barrier_sync():
        if world > 1:
            comm.barrier()
        torch.cuda.synchronize()

    dev_batches = [[stager.stage(host_batch(i * accum + a), vl, pad) for a in range(accum)] for i in range(n_steps_total)]
    torch.cuda.synchronize()

    def make_trainer(plain: bool):
        """The product configuration, or (``plain``) the framework's own baseline path."""
        fused = None
        if world > 1 and args.fused != 0 and not plain:
            try:
                from create_llm_by_cupy_b200.parallel.symm import FusedCollectives
                kw = dict(rs_blocks=args.comm_blocks, ag_blocks=args.comm_blocks) if args.comm_blocks > 0 else {}
                if args.peer_wait_s > 0:
                    kw["wait_ns"] = int(args.peer_wait_s * 1e9)
                fused = FusedCollectives(comm, device, gather_mode=args.ag, reduce_mode=args.rs, **kw)
                if args.parallel_copies:
                    fused.lib.b200_symm_parallel_copies(1)
            except Exception as e:  # the NCCL path is the fallback only when the fused runtime cannot start
                if args.fused == 1:
                    raise
                if rank == 0:
                    print(f"[bench] fused collectives unavailable ({e}); using NCCL", file=sys.stderr)
        F.set_unfused_baseline(plain)
        tr = Trainer(md, rank=rank, world_size=world, comm=comm, device=device, zero_stage=c["zero"],
                     optimizer_device=c["opt"], accum_step=accum, lr_max=3e-4, lr_mini=3e-5, weight_decay=0.1,
                     warm_up=100, total_steps=10000, beta1=0.9, beta2=0.95, max_grads=1.0, fused=fused,
                     profile_comm=world > 1, profile_phases=not (args.no_phases or args.graph),
                     cuda_graph=args.graph and not plain, adam_overlap=not (args.no_adam_overlap or plain),
                     defer_host_read=not (args.sync_read or plain), adam_overlap_ctas_per_sm=args.adam_ctas,
                     offload_delayed_update=args.delayed_offload and not plain)
        return tr, fused

    def timed(trainer, run_step):
        for w in range(args.warmup):
            run_step(w)
        trainer.flush_host_read()
        barrier_sync()
        native.raise_on_status()
        trainer.phase_times()                 # drop the warm-up steps' marks
        trainer.manager.exposed_comm_ms()
        launches0 = native.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(args.steps):
            run_step(args.warmup + k)
        trainer.flush_host_read()             # the last step's scalars are read inside the timed region
        trainer.join_optimizer()              # the last step's pipelined AdamW belongs to the timed region
        e1.record()
        barrier_sync()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            comm.all_reduce(ms, op="max")
        exposed = trainer.manager.exposed_comm_ms() / max(args.steps, 1) if world > 1 else 0.0
        return float(ms) / args.steps, (native.launch_count() - launches0) // args.steps, exposed, trainer.phase_times()

    def dev_step(trainer):
        return lambda i: trainer.train_step(dev_batches[i % n_steps_total])

    def e2e_step(trainer):
        def step(i):
            batches = [stager.stage(host_batch((i % n_steps_total) * accum + a), vl, pad) for a in range(accum)]
            return trainer.train_step(batches)["loss"]
        return step

    def note(msg):
        print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    # ---- product arm: device-resident inputs, then end to end through the public API ------------------------
    trainer, fused = make_trainer(plain=False)
    note("product arm built")
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_dev, launches, exposed, phases = timed(trainer, dev_step(trainer))
    clocks = sampler.stop() if sampler else None
    note(f"device-resident phase done: {ms_dev:.2f} ms/step")
    last = dict(trainer.last)
    e2e = None
    if not args.no_e2e:
        ms_e2e, _, _, _ = timed(trainer, e2e_step(trainer))
        note(f"end-to-end phase done: {ms_e2e:.2f} ms/step")
        e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": stager.h2d_bytes * accum, "d2h_bytes_per_step": 12,
               "host_read": "deferred by one step" if trainer.defer_host_read else "every step before the next"}
    native.raise_on_status()
    n_par = trainer.n_params
    cuda_graph = bool(trainer.cuda_graph)
    collectives = (f"fused reduce-scatter+stats ({args.rs}), gather={args.ag}" if fused is not None
                   else ("nccl" if world > 1 else "none"))
    copies = fused.copies if fused is not None else 0
    trainer.close()
    del trainer, fused
    note("product arm closed")

    # ---- baseline arm: the framework's own plain path on the same box ---------------------------------------
    baseline = None
    if not args.no_baseline:
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        btr, _ = make_trainer(plain=True)
        note("baseline arm built")
        ms_b, launches_b, exposed_b, phases_b = timed(btr, dev_step(btr))
        note(f"baseline arm done: {ms_b:.2f} ms/step")
        native.raise_on_status()
        baseline = {"value": tokens / (ms_b / 1e3), "unit": "tokens/s", "ms_per_step": ms_b, "gpu_launches": launches_b,
                    "exposed_comm_ms_per_step": exposed_b, "phases_ms": phases_b,
                    "what": ("NCCL all-gather / reduce-scatter, " if world > 1 else "") +
                            "AdamW after the backward, separate RoPE / SwiGLU / loss-statistics kernels, "
                            "weight gradients on the main stream; same process, after the product arm"}
        btr.close()
        del btr
        F.set_unfused_baseline(False)

    value = tokens / (ms_dev / 1e3)
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))
        except Exception:
            pass
        flops_tok = 6.0 * n_par + 6.0 * c["layer_num"] * c["hidden_size"] * T
        out = {
            "metric": "train tokens/sec (device-timed, max over ranks)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / baseline["value"]) if baseline else None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": c["name"], "global_batch": B * accum * world, "seq_len": T,
                       "parallelism": f"zero{c['zero']}-dp{world}", "params": n_par, "cuda_graph": cuda_graph,
                       "keep_params_until_backward": bool(args.keep_params), "collectives": collectives,
                       "optimizer": c["opt"] + (" (one-step delayed update)" if args.delayed_offload and c["opt"] == "cpu" else ""),
                       "l2": f"not flushed: a step streams more than {28e-9 * n_par / world + 2e-9 * n_par:.1f} GB of weights and "
                             "optimizer state per GPU, far above the 126 MB L2"},
            "e2e": e2e, "gpu_launches": launches, "copy_engine_transfers_total": copies, "clocks": clocks,
            "exposed_comm_ms_per_step": exposed, "phases_ms": phases, "baseline": baseline,
            "model_tflops_per_gpu": flops_tok * tokens / world / (ms_dev / 1e3) / 1e12,
            "mfu_of_measured_sustained": (flops_tok * tokens / world / (ms_dev / 1e3) / 1e12) /
                                         peaks.get("bf16_tflops_sustained", 1401.9),
            "last_loss": last.get("loss"), "last_grad_norm": last.get("grad_norm"),
            "native_digest": native.source_digest(),
        }
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(out), flush=True)
        os.dup2(2, 1)
    if world > 1:
        comm.barrier()
        shutdown_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
