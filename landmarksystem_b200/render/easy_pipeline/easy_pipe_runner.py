"""Front end of the stage pipeline: submit a batch of jobs, get results back in order (reference:
landmark/render/easy_pipeline/easy_pipe_runner.py:1-74)."""
from __future__ import annotations

from queue import SimpleQueue
from typing import List

from .pipeline import PipelineItem, SimplePipeline
from .task import StopTask, Task


class EasyPipeRunner:
    def __init__(self, items: List[PipelineItem]):
        self.job_queue, self.result_queue = SimpleQueue(), SimpleQueue()
        self.pipeline = SimplePipeline(items, self.job_queue, self.result_queue)
        self.pipeline.start()
        self.pending = 0

    def run_batch(self, payloads) -> None:
        for p in payloads:
            self.job_queue.put(Task(p))
            self.pending += 1

    def get_result(self):
        assert self.pending > 0, "no job in flight"
        task = self.result_queue.get()
        self.pending -= 1
        if isinstance(task, StopTask):
            raise RuntimeError("pipeline stopped")
        if isinstance(task.payload, Exception):
            raise task.payload
        return task.payload

    def stop(self) -> None:
        self.pipeline.stop()
