"""Structured run metrics: JSON-lines file + optional TensorBoard scalars with the reference's tag
names (``Train/Loss``, ``Train/PSNR``, ``Test/PSNR`` ...; reference:
benchmarks/nerf/gridnerf/gridnerf_trainer.py:355-364), CUDA-event stage timers and NVTX ranges."""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Dict, Optional

import torch


class MetricsLogger:
    def __init__(self, logfolder: Optional[str], tensorboard: bool = False, enabled: bool = True, wandb: bool = False,
                 run_name: Optional[str] = None, run_config: Optional[dict] = None):
        self.enabled = enabled and logfolder is not None
        self._fh = None
        self.writer = None
        self.wandb = None
        if self.enabled and wandb:
            # the reference starts a wandb run when ``TrainConfig.wandb`` is set (landmark/train/nerf_trainer.py:95-97);
            # the package is optional here: without it the flag only costs a warning
            try:
                import wandb as _wandb

                _wandb.init(project="landmarksystem_b200", name=run_name, dir=logfolder, config=run_config or {})
                self.wandb = _wandb
            except Exception as exc:  # noqa: BLE001 - not installed, or no network
                print(f"[metrics] wandb logging requested but unavailable ({type(exc).__name__}); continuing without it")
        if self.enabled:
            os.makedirs(logfolder, exist_ok=True)
            self._fh = open(os.path.join(logfolder, "metrics.jsonl"), "a", encoding="utf-8")
            if tensorboard:
                try:
                    from torch.utils.tensorboard import SummaryWriter

                    self.writer = SummaryWriter(log_dir=os.path.join(logfolder, "runs"))
                except Exception:  # tensorboard is optional
                    self.writer = None

    def log(self, step: int, scalars: Dict[str, float]) -> None:
        if not self.enabled:
            return
        rec = {"step": int(step), "time": time.time()}
        rec.update({k: float(v) for k, v in scalars.items()})
        self._fh.write(json.dumps(rec) + "\n")
        self._fh.flush()
        if self.writer is not None:
            for k, v in scalars.items():
                self.writer.add_scalar(k, float(v), global_step=step)
        if self.wandb is not None:
            self.wandb.log({k: float(v) for k, v in scalars.items()}, step=int(step))

    def close(self) -> None:
        if self._fh is not None:
            self._fh.close()
            self._fh = None
        if self.writer is not None:
            self.writer.close()


class StageTimer:
    """Accumulates device time per named stage with CUDA events (wall clock on CPU)."""

    def __init__(self, enabled: bool = False):
        self.enabled = enabled
        self.totals: Dict[str, float] = {}
        self.counts: Dict[str, int] = {}
        self._pending = []

    @contextlib.contextmanager
    def stage(self, name: str):
        if not self.enabled:
            yield
            return
        cuda = torch.cuda.is_available()
        if cuda:
            torch.cuda.nvtx.range_push(name)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            yield
            end.record()
            torch.cuda.nvtx.range_pop()
            self._pending.append((name, start, end))
        else:
            t0 = time.perf_counter()
            yield
            self._add(name, (time.perf_counter() - t0) * 1e3)

    def _add(self, name, ms):
        self.totals[name] = self.totals.get(name, 0.0) + ms
        self.counts[name] = self.counts.get(name, 0) + 1

    def summary(self) -> Dict[str, float]:
        if self._pending:
            torch.cuda.synchronize()
            for name, s, e in self._pending:
                self._add(name, s.elapsed_time(e))
            self._pending.clear()
        return {k: self.totals[k] / max(self.counts[k], 1) for k in self.totals}
