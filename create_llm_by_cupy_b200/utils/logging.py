"""Metrics and console logging (reference: wandb + prints, model/ZeRO3.py:120-166,440-467,499-501).

``MetricsLogger`` fans a dict of scalars out to the console (rank 0), a JSON-lines file and, when
the package is importable and ``wand=True``, Weights & Biases under the reference's project
name. On top of the reference's GradScale / Grad Norm / loss / Perplexity / learning_rate /
validation it records what the reference never measures: tokens per second, model FLOP/s
utilisation and exposed-communication milliseconds per step.
"""
from __future__ import annotations

import json
import math
import os
import time

WANDB_PROJECT = "zero-scrach-1B LLM"


def model_flops_per_token(n_params_no_embed: int, layers: int, hidden: int, seq_len: int, vocab: int) -> float:
    """Training FLOPs per token: 6 * (weights incl. LM head) + causal attention (12 * L * H * T / 2)."""
    return 6.0 * (n_params_no_embed + vocab * hidden) + 6.0 * layers * hidden * seq_len


class MetricsLogger:
    def __init__(self, rank: int = 0, wand: bool = False, config: dict | None = None, jsonl_path: str | None = None,
                 console: bool = True):
        self.rank = rank
        self.console = console and rank == 0
        self.jsonl = open(jsonl_path, "a") if (jsonl_path and rank == 0) else None
        self.wandb = None
        self.history = []
        if wand and rank == 0:
            try:
                import wandb  # noqa: WPS433 (optional dependency, as in the reference)
                wandb.init(project=WANDB_PROJECT, config=config or {}, mode=os.environ.get("WANDB_MODE", "offline"))
                self.wandb = wandb
            except Exception as e:  # missing package / no network: keep training
                print(f"[log] wandb disabled: {e}")

    def log(self, metrics: dict, step: int | None = None):
        rec = dict(metrics)
        if step is not None:
            rec["step"] = step
        rec["time"] = time.time()
        self.history.append(rec)
        if self.jsonl is not None:
            self.jsonl.write(json.dumps(rec) + "\n")
            self.jsonl.flush()
        if self.wandb is not None:
            self.wandb.log(metrics, step=step)

    def line(self, text: str):
        if self.console:
            print(text, flush=True)

    def step_line(self, epoch: int, it: int, max_iters: int, loss: float, extra: dict | None = None):
        if not self.console:
            return
        ppl = math.exp(min(loss, 30.0)) if math.isfinite(loss) else float("nan")
        parts = [time.strftime("%H:%M:%S"), f"epoch {epoch}", f"iter {it}/{max_iters}", f"loss {loss:.4f}",
                 f"ppl {ppl:.2f}"]
        for k, v in (extra or {}).items():
            parts.append(f"{k} {v:.4g}" if isinstance(v, float) else f"{k} {v}")
        print(" | ".join(parts), flush=True)

    def close(self):
        if self.jsonl is not None:
            self.jsonl.close()
        if self.wandb is not None:
            self.wandb.finish()
