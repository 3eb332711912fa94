from .easy_pipe_runner import EasyPipeRunner
from .pipeline import PipelineItem, SimplePipeline
from .task import EmptyTask, StopTask, Task
from .worker import ProfileWorkerThread, SimpleWorker, Worker, WorkerThread

__all__ = ["EasyPipeRunner", "PipelineItem", "SimplePipeline", "EmptyTask", "StopTask", "Task", "ProfileWorkerThread",
           "SimpleWorker", "Worker", "WorkerThread"]
