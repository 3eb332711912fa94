"""Front end of the stage pipeline: submit a batch of jobs, get results back in order (reference:
landmark/render/easy_pipeline/easy_pipe_runner.py:1-74)."""
from __future__ import annotations

from queue import SimpleQueue
from typing import List

from .pipeline import PipelineItem, SimplePipeline
from .task import StopTask, Task


class EasyPipeRunner:
    def __init__(self, items: List[PipelineItem]):
        self.items = items
        self.job_queue, self.result_queue = SimpleQueue(), SimpleQueue()
        self.pipeline = self.create_pipe()
        self.pipeline.start()
        self.pending = 0

    def create_pipe(self) -> SimplePipeline:
        return SimplePipeline(self.items, self.job_queue, self.result_queue)

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

    def get_from_result_queue(self):
        """The next raw task of the result queue (blocking)."""
        return self.result_queue.get()

    def get_result_task(self, block: bool = False):
        """The next finished task, or ``None`` when ``block`` is false and none is ready."""
        if not block and self.result_queue.empty():
            return None
        task = self.get_from_result_queue()
        self.pending = max(self.pending - 1, 0)
        return task

    def stop(self) -> None:
        self.pipeline.stop()

    def wait_stop(self) -> None:
        self.pipeline.wait_stop()
