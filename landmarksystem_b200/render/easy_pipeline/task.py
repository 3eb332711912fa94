"""Work items of the stage pipeline (reference: landmark/render/easy_pipeline/task.py:1-29)."""


class Task:
    def __init__(self, payload=None):
        self.payload = payload


class EmptyTask(Task):
    """Keeps a stage's output slot aligned when a worker produced nothing."""


class StopTask(Task):
    """Tells a worker to exit and is forwarded down the pipeline."""
