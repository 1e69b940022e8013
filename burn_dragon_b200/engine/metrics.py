"""Training metrics: JSONL log, console lines, end-of-run summary.

The reference relies on burn-train's metric loggers (loss for train and valid, learning rate, a
summary at the end; src/bin/train.rs:397-400). Here every record is one JSON line in
`<run>/metrics.jsonl` with device-timed throughput next to the loss.
"""
from __future__ import annotations

import json
import math
import time
from pathlib import Path
from typing import Dict, List


class MetricsLogger:
    def __init__(self, run_dir=None, log_frequency: int = 100, rank: int = 0, quiet: bool = False):
        self.path = Path(run_dir) / "metrics.jsonl" if run_dir is not None and rank == 0 else None
        if self.path is not None:
            self.path.parent.mkdir(parents=True, exist_ok=True)
        self.freq = max(1, log_frequency)
        self.rank, self.quiet = rank, quiet
        self.history: Dict[str, List[float]] = {}
        self.t0 = time.time()

    def log(self, split: str, step: int, **values) -> None:
        rec = dict(split=split, step=step, time=round(time.time() - self.t0, 3), **values)
        for k, v in values.items():
            if isinstance(v, (int, float)) and not (isinstance(v, float) and math.isnan(v)):
                self.history.setdefault(f"{split}/{k}", []).append(float(v))
        if self.path is not None:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        if self.rank == 0 and (split != "train" or step % self.freq == 0):
            body = "  ".join(f"{k}={v:.5g}" if isinstance(v, float) else f"{k}={v}" for k, v in values.items())
            line = f"[{split} {step:>7}] {body}"
            if self.path is not None:
                # the run's text log (burn-train writes `experiment.log` beside its checkpoints)
                with open(self.path.with_name("experiment.log"), "a") as f:
                    f.write(time.strftime("%Y-%m-%d %H:%M:%S ") + line + "\n")
            if not self.quiet:
                print(line, flush=True)

    def summary(self) -> str:
        """min / max / last of every metric, as burn-train's `.summary()` prints at the end of a run."""
        lines = [f"{'metric':<28}{'min':>12}{'max':>12}{'last':>12}{'n':>8}"]
        for k in sorted(self.history):
            v = self.history[k]
            lines.append(f"{k:<28}{min(v):>12.5g}{max(v):>12.5g}{v[-1]:>12.5g}{len(v):>8}")
        return "\n".join(lines)


def theoretical_profile(cfg, batch: int, T: int) -> Dict[str, float]:
    """Analytic FLOPs of one training step. The reference logs a version that counts one encoder
    GEMM and no LM head (src/bin/train.rs:635-659); this one counts both encoders, the causal half
    of the attention products and the head, and assumes backward = 2 x forward."""
    fwd = cfg.flops_per_token_forward(T) * batch * T
    return dict(forward_flops=fwd, backward_flops=2 * fwd, step_flops=3 * fwd, params=cfg.num_params())
