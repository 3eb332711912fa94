"""Pipeline workers: a callable run by a host thread, optionally on its own CUDA stream, optionally
under the PyTorch profiler (reference: landmark/render/easy_pipeline/worker.py:1-157)."""
from __future__ import annotations

import threading
from queue import SimpleQueue
from typing import Callable, Optional

import torch

from .task import EmptyTask, StopTask, Task


class Worker:
    """Stage interface: ``process(payload)`` returns the stage's output."""

    def process(self, payload):
        raise NotImplementedError


class SimpleWorker(Worker):
    """A callable as a stage.  With ``init_fn`` the worker builds a private resource once (a model replica, a buffer
    pool) and the callable receives it first: ``fn(resource, payload)``."""

    def __init__(self, fn: Callable, init_fn: Optional[Callable] = None):
        self.fn = fn
        self.has_resource = init_fn is not None
        self.resource = init_fn() if init_fn is not None else None

    def process(self, payload):
        return self.fn(self.resource, payload) if self.has_resource else self.fn(payload)


class WorkerThread(threading.Thread):
    def __init__(self, worker: SimpleWorker, in_queue: SimpleQueue, out_queue: SimpleQueue, use_cuda_stream: bool = False):
        super().__init__(daemon=True)
        self.worker, self.in_queue, self.out_queue = worker, in_queue, out_queue
        self.stream = torch.cuda.Stream() if (use_cuda_stream and torch.cuda.is_available()) else None
        self.device = torch.cuda.current_device() if torch.cuda.is_available() else None

    def _run_one(self, task: Task):
        if self.stream is None:
            return self.worker.process(task.payload)
        with torch.cuda.stream(self.stream):
            out = self.worker.process(task.payload)
        self.stream.synchronize()
        return out

    def loop(self):
        while True:
            task = self.in_queue.get()
            if isinstance(task, StopTask):
                self.out_queue.put(task)
                return
            if isinstance(task, EmptyTask):
                self.out_queue.put(task)
                continue
            try:
                self.out_queue.put(Task(self._run_one(task)))
            except Exception as exc:  # surface the failure to the consumer instead of dying silently
                self.out_queue.put(Task(exc))

    def run(self):
        if self.device is not None:
            torch.cuda.set_device(self.device)
        self.loop()

    # -- queue access under the reference's method names (worker.py:101-124) ---------------------------------
    def get_from_job_queue(self):
        return self.in_queue.get()

    def put_to_result_queue(self, result):
        self.out_queue.put(result)

    def put_stop_task(self):
        self.in_queue.put(StopTask())

    def wait_stop(self, timeout: float = 10.0):
        self.join(timeout=timeout)


class ProfileWorkerThread(WorkerThread):
    """Same loop under ``torch.profiler`` (wait / warm-up / active schedule, TensorBoard trace handler)."""

    def __init__(self, *args, trace_dir: str = "./landmark_traces", wait: int = 120, warmup: int = 120, active: int = 10,
                 **kwargs):
        super().__init__(*args, **kwargs)
        self.trace_dir, self.schedule = trace_dir, (wait, warmup, active)

    def run(self):
        from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler

        if self.device is not None:
            torch.cuda.set_device(self.device)
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        wait, warmup, active = self.schedule
        with profile(activities=acts, schedule=schedule(wait=wait, warmup=warmup, active=active),
                     on_trace_ready=tensorboard_trace_handler(self.trace_dir), with_stack=True) as prof:
            original = self._run_one

            def stepped(task):
                out = original(task)
                prof.step()
                return out

            self._run_one = stepped
            self.loop()
