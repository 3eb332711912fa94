"""Sharded, asynchronous, atomic checkpoints (internal format; the public ``state_dict.th`` /
``kwargs.th`` / ``point_cloud.ply`` formats of the reference stay the trainers' default).

The reference saves with blocking ``torch.save`` on the training thread
(``landmark/nerf_components/model/base_model.py:89-132``, ``benchmarks/nerf/gridnerf/gridnerf_trainer.py:
156-164, 384-404``) and has no atomicity, sharding or RNG state.  Here:

* each rank writes only its own shard ``shard-{rank:05d}-of-{world:05d}.pt`` (tensors it owns:
  its spatial block, its channel slice, its optimiser partition) plus, on rank 0, ``meta.json``;
* tensors are first copied device-to-host into pinned buffers on a side stream, so the training stream
  continues as soon as the copies are enqueued, and the file is written by a background thread;
* a checkpoint becomes visible atomically: files go to ``<dir>.tmp-<nonce>`` and the directory is renamed
  when every shard and the metadata are complete (``COMPLETE`` marker written last);
* RNG states (torch CPU / CUDA, numpy, python) and arbitrary JSON metadata are part of the checkpoint.
"""
from __future__ import annotations

import json
import os
import random
import shutil
import threading
import time
import uuid
from typing import Any, Dict, Optional

import numpy as np
import torch


def _rng_state() -> Dict[str, Any]:
    state = {"torch": torch.get_rng_state(), "numpy": np.random.get_state(), "python": random.getstate()}
    if torch.cuda.is_available():
        state["cuda"] = torch.cuda.get_rng_state()
    return state


def restore_rng_state(state: Dict[str, Any]) -> None:
    torch.set_rng_state(state["torch"])
    np.random.set_state(state["numpy"])
    random.setstate(state["python"])
    if "cuda" in state and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["cuda"])


def _to_host(obj, stream=None, pinned_pool: Optional[Dict] = None):
    """Recursively copy tensors to (pinned, when on CUDA) host memory; returns a structure of the same shape."""
    if isinstance(obj, torch.Tensor):
        if obj.is_cuda:
            key = (tuple(obj.shape), obj.dtype)
            buf = None
            if pinned_pool is not None:
                free = pinned_pool.setdefault(key, [])
                buf = free.pop() if free else None
            if buf is None:
                buf = torch.empty(obj.shape, dtype=obj.dtype, pin_memory=True)
            buf.copy_(obj.detach(), non_blocking=True)
            return buf
        return obj.detach().clone()
    if isinstance(obj, dict):
        return {k: _to_host(v, stream, pinned_pool) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_host(v, stream, pinned_pool) for v in obj)
    return obj


def _shard_name(rank: int, world: int) -> str:
    return f"shard-{rank:05d}-of-{world:05d}.pt"


def save_sharded(directory: str, state: Dict[str, Any], rank: int = 0, world: int = 1, meta: Optional[Dict] = None,
                 barrier=None) -> str:
    """Blocking sharded save.  ``barrier`` (callable, optional) synchronises the ranks around the rename."""
    return AsyncCheckpointer(directory_root=None).save(directory, state, rank, world, meta, barrier=barrier, wait=True)


def load_sharded(directory: str, rank: int = 0, map_location="cpu", restore_rng: bool = False) -> Dict[str, Any]:
    if not os.path.exists(os.path.join(directory, "COMPLETE")):
        raise FileNotFoundError(f"{directory} is not a complete checkpoint")
    with open(os.path.join(directory, "meta.json"), encoding="utf-8") as fh:
        meta = json.load(fh)
    world = int(meta["world"])
    shard = torch.load(os.path.join(directory, _shard_name(rank % world, world)), map_location=map_location, weights_only=False)
    if restore_rng and "rng" in shard:
        restore_rng_state(shard["rng"])
    return {"state": shard["state"], "meta": meta, "rng": shard.get("rng")}


def latest_checkpoint(root: str) -> Optional[str]:
    """Newest complete ``step-*`` directory under ``root`` (incomplete ones are ignored)."""
    best = None
    if not os.path.isdir(root):
        return None
    for name in os.listdir(root):
        path = os.path.join(root, name)
        if name.startswith("step-") and os.path.exists(os.path.join(path, "COMPLETE")):
            step = int(name.split("-")[1])
            if best is None or step > best[0]:
                best = (step, path)
    return best[1] if best else None


class AsyncCheckpointer:
    """``save()`` returns after the device-to-host copies are enqueued; a worker thread waits for them,
    serialises the shard and publishes the directory.  ``wait()`` blocks until pending saves are on disk."""

    def __init__(self, directory_root: Optional[str] = None, keep_last: int = 0):
        self.root, self.keep_last = directory_root, keep_last
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        self._pinned: Dict = {}
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            err, self._error = self._error, None
            raise err

    def save_step(self, step: int, state, rank=0, world=1, meta=None, barrier=None, wait=False) -> str:
        assert self.root is not None
        return self.save(os.path.join(self.root, f"step-{step:08d}"), state, rank, world, dict(meta or {}, step=step),
                         barrier=barrier, wait=wait)

    def save(self, directory: str, state, rank=0, world=1, meta=None, barrier=None, wait=False) -> str:
        self.wait()                                                   # one save in flight at a time
        nonce = uuid.uuid4().hex[:8] if world == 1 else "shared"
        tmp = f"{directory}.tmp-{nonce}"
        os.makedirs(tmp, exist_ok=True)
        event = None
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())     # the copies see the state of "now"
            with torch.cuda.stream(self._stream):
                host_state = _to_host(state, pinned_pool=self._pinned)
                event = torch.cuda.Event()
                event.record(self._stream)
        else:
            host_state = _to_host(state)
        rng = _rng_state()
        payload_meta = dict(meta or {}, world=world, time=time.time(), format="lmb200-sharded-v1")

        def work():
            try:
                if event is not None:
                    event.synchronize()
                torch.save({"state": host_state, "rng": rng, "rank": rank}, os.path.join(tmp, _shard_name(rank, world)))
                if rank == 0:
                    with open(os.path.join(tmp, "meta.json"), "w", encoding="utf-8") as fh:
                        json.dump(payload_meta, fh)
                if barrier is not None:
                    barrier()                                         # every shard is on disk
                if rank == 0:
                    with open(os.path.join(tmp, "COMPLETE"), "w", encoding="utf-8") as fh:
                        fh.write("ok\n")
                    if os.path.isdir(directory):
                        shutil.rmtree(directory)
                    os.replace(tmp, directory)                        # atomic publish
                    self._prune(os.path.dirname(directory))
                if barrier is not None:
                    barrier()
                self._recycle(host_state)
            except BaseException as exc:                              # surfaced by the next wait()
                self._error = exc

        if wait or barrier is not None:
            work()                                                    # collectives must stay on the calling thread
            if self._error is not None:
                self.wait()
        else:
            self._thread = threading.Thread(target=work, name="lmb-checkpoint", daemon=True)
            self._thread.start()
        return directory

    def _recycle(self, host_state) -> None:
        if isinstance(host_state, torch.Tensor):
            if host_state.is_pinned():
                self._pinned.setdefault((tuple(host_state.shape), host_state.dtype), []).append(host_state)
        elif isinstance(host_state, dict):
            for v in host_state.values():
                self._recycle(v)
        elif isinstance(host_state, (list, tuple)):
            for v in host_state:
                self._recycle(v)

    def _prune(self, root: str) -> None:
        if self.keep_last <= 0 or not root or not os.path.isdir(root):
            return
        steps = sorted(n for n in os.listdir(root) if n.startswith("step-") and os.path.exists(os.path.join(root, n, "COMPLETE")))
        for name in steps[:-self.keep_last]:
            shutil.rmtree(os.path.join(root, name), ignore_errors=True)
