"""Sharded, asynchronous, atomic checkpoints (internal format; the public ``state_dict.th`` /
``kwargs.th`` / ``point_cloud.ply`` formats of the reference stay the trainers' default).

The reference saves with blocking ``torch.save`` on the training thread
(``landmark/nerf_components/model/base_model.py:89-132``, ``benchmarks/nerf/gridnerf/gridnerf_trainer.py:
156-164, 384-404``) and has no atomicity, sharding or RNG state.  Here:

* each rank writes only its own shard ``shard-{rank:05d}-of-{world:05d}.pt`` (tensors it owns:
  its spatial block, its channel slice, its optimiser partition) plus, on rank 0, ``meta.json``;
* a snapshot is taken ON THE TRAINING STREAM first (device-to-device clones into reusable staging tensors, a few
  milliseconds even for tens of GB), then the staging tensors are copied to pinned host memory on a side stream and the
  file is written by a background thread - later in-place updates of parameters and optimiser moments cannot leak into
  the checkpoint.  When the staging clones do not fit in device memory the save falls back to copying the live tensors
  and makes the training stream wait for those copies (correct, but the next step starts after the copies);
* a checkpoint becomes visible atomically: files go to ``<dir>.tmp-<nonce>`` and the directory is renamed
  when every shard and the metadata are complete (``COMPLETE`` marker written last).  With more than one rank the
  publishing rank learns that the other shards are on disk through a host-side rendezvous: a ``barrier`` callable run on
  the calling thread, or a key-value ``store`` (the process group's rendezvous store) polled from the writer thread;
  a multi-rank save with neither is refused;
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


def capture_rng_state() -> Dict[str, Any]:
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


def _snapshot_on_device(obj, pool: Dict):
    """Device-to-device clones (current stream) of every CUDA tensor into reusable staging tensors."""
    if isinstance(obj, torch.Tensor):
        if not obj.is_cuda:
            return obj
        key = (tuple(obj.shape), obj.dtype, obj.device.index)
        free = pool.setdefault(key, [])
        buf = free.pop() if free else torch.empty(obj.shape, dtype=obj.dtype, device=obj.device)
        buf.copy_(obj.detach())
        return buf
    if isinstance(obj, dict):
        return {k: _snapshot_on_device(v, pool) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_snapshot_on_device(v, pool) for v in obj)
    return obj


def _release_staging(obj, pool: Dict) -> None:
    if isinstance(obj, torch.Tensor):
        if obj.is_cuda:
            pool.setdefault((tuple(obj.shape), obj.dtype, obj.device.index), []).append(obj)
    elif isinstance(obj, dict):
        for v in obj.values():
            _release_staging(v, pool)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            _release_staging(v, pool)


def _to_host(obj, stream=None, pinned_pool: Optional[Dict] = None):
    """Recursively copy tensors to (pinned, when on CUDA) host memory; returns a structure of the same shape.
    ``stream`` is the stream the copies run on: every CUDA source is marked as used there, so the caching allocator
    does not hand its memory to someone else while the copy is still reading it."""
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
            if stream is not None:
                obj.record_stream(stream)
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
                 barrier=None, store=None) -> str:
    """Blocking sharded save.  ``barrier`` (callable) or ``store`` (key-value store shared by the ranks) tells the
    publishing rank when every shard is on disk; one of them is required when ``world > 1``."""
    return AsyncCheckpointer(directory_root=None).save(directory, state, rank, world, meta, barrier=barrier, store=store,
                                                       wait=True)


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
    """``save()`` returns after the snapshot (device clones on the caller's stream) and the device-to-host copies
    (side stream) are enqueued; a worker thread waits for them, serialises the shard and publishes the directory.
    ``wait()`` blocks until pending saves are on disk."""

    RENDEZVOUS_TIMEOUT_S = 1800.0

    def __init__(self, directory_root: Optional[str] = None, keep_last: int = 0, snapshot: str = "clone"):
        assert snapshot in ("clone", "block")
        self.root, self.keep_last, self.snapshot = directory_root, keep_last, snapshot
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        self._pinned: Dict = {}
        self._staging: Dict = {}
        self._saves = 0
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            err, self._error = self._error, None
            raise err

    def save_step(self, step: int, state, rank=0, world=1, meta=None, barrier=None, store=None, wait=False) -> str:
        assert self.root is not None
        return self.save(os.path.join(self.root, f"step-{step:08d}"), state, rank, world, dict(meta or {}, step=step),
                         barrier=barrier, store=store, wait=wait)

    def save(self, directory: str, state, rank=0, world=1, meta=None, barrier=None, store=None, wait=False) -> str:
        if world > 1 and barrier is None and store is None:
            raise ValueError("a checkpoint of more than one rank needs a host-side rendezvous: pass barrier= (a callable "
                             "every rank runs) or store= (a key-value store shared by the ranks); without one the "
                             "publishing rank cannot know that the other shards are on disk")
        self.wait()                                                   # one save in flight at a time
        self._saves += 1
        tag = f"lmb-ckpt/{os.path.basename(directory)}/{self._saves}"  # same on every rank: ranks save in lock step
        nonce = uuid.uuid4().hex[:8] if world == 1 else "shared"
        tmp = f"{directory}.tmp-{nonce}"
        os.makedirs(tmp, exist_ok=True)
        event = None
        staged = None
        if self._stream is not None:
            cur = torch.cuda.current_stream()
            src, blocked = state, self.snapshot == "block"
            if not blocked:
                try:
                    staged = src = _snapshot_on_device(state, self._staging)      # on the training stream: a true snapshot
                except torch.cuda.OutOfMemoryError:
                    self._staging.clear()
                    torch.cuda.empty_cache()
                    staged, src, blocked = None, state, True
            self._stream.wait_stream(cur)
            with torch.cuda.stream(self._stream):
                host_state = _to_host(src, stream=self._stream, pinned_pool=self._pinned)
                event = torch.cuda.Event()
                event.record(self._stream)
            if blocked:
                cur.wait_event(event)        # no staging copy: later work of the training stream waits for the reads
        else:
            host_state = _to_host(state)
        rng = capture_rng_state()
        payload_meta = dict(meta or {}, world=world, time=time.time(), format="lmb200-sharded-v1")

        def rendezvous(phase: str):
            """Every rank announces ``phase``; rank 0 returns once all ranks have (other ranks do not wait)."""
            if barrier is not None:
                barrier()
                return
            if store is None:
                return
            store.set(f"{tag}/{phase}/{rank}", "1")
            if rank == 0:
                deadline = time.time() + self.RENDEZVOUS_TIMEOUT_S
                for r in range(world):
                    key = f"{tag}/{phase}/{r}"
                    while True:
                        try:
                            if store.check([key]):
                                break
                        except (RuntimeError, NotImplementedError):
                            store.wait([key])                  # stores without check(): blocking wait
                            break
                        if time.time() > deadline:
                            raise TimeoutError(f"checkpoint {directory}: rank {r} did not report '{phase}'")
                        time.sleep(0.01)

        def work():
            try:
                if event is not None:
                    event.synchronize()
                if staged is not None:
                    _release_staging(staged, self._staging)
                torch.save({"state": host_state, "rng": rng, "rank": rank}, os.path.join(tmp, _shard_name(rank, world)))
                if rank == 0:
                    with open(os.path.join(tmp, "meta.json"), "w", encoding="utf-8") as fh:
                        json.dump(payload_meta, fh)
                rendezvous("written")                                 # every shard is on disk
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
