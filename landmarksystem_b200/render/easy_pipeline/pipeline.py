"""Chain of worker pools connected by queues (reference: landmark/render/easy_pipeline/pipeline.py:1-99)."""
from __future__ import annotations

from dataclasses import dataclass
from queue import SimpleQueue
from typing import Callable, List, Optional

from .task import StopTask
from .worker import ProfileWorkerThread, SimpleWorker, WorkerThread


@dataclass
class PipelineItem:
    fn: Callable
    n_workers: int = 1
    use_cuda_stream: bool = False
    profile: bool = False
    init_fn: Optional[Callable] = None          # builds a per-worker resource; ``fn(resource, payload)`` then


class SimplePipeline:
    def __init__(self, items: List[PipelineItem], job_queue: SimpleQueue, result_queue: SimpleQueue):
        self.items, self.threads = items, []
        queues = [job_queue] + [SimpleQueue() for _ in items[:-1]] + [result_queue]
        for i, item in enumerate(items):
            for _ in range(item.n_workers):
                cls = ProfileWorkerThread if item.profile else WorkerThread
                self.threads.append(cls(SimpleWorker(item.fn, item.init_fn), queues[i], queues[i + 1],
                                        use_cuda_stream=item.use_cuda_stream))
        self.job_queue, self.result_queue = job_queue, result_queue

    def start(self):
        for t in self.threads:
            t.start()

    def stop(self):
        for _ in range(max(self.items[0].n_workers, 1)):
            self.job_queue.put(StopTask())
        self.wait_stop()

    def wait_stop(self, timeout: float = 10.0):
        for t in self.threads:
            t.join(timeout=timeout)

    def get_result_queue(self) -> SimpleQueue:
        return self.result_queue
