"""Failure detection (host-side heartbeats, no GPU involved) and sharded / asynchronous checkpoints."""
import multiprocessing as mp
import os
import time

import pytest
import torch
import torch.distributed as dist

from landmarksystem_b200.runtime import AsyncCheckpointer, HeartbeatMonitor, PeerFailure, StatusWords, load_sharded
from landmarksystem_b200.runtime.checkpoint import latest_checkpoint


def _store():
    return dist.HashStore()


def test_heartbeat_detects_silent_reported_and_departed_peers():
    store = _store()
    now = [1000.0]
    a = HeartbeatMonitor(store, 0, 3, timeout=5.0, clock=lambda: now[0])
    b = HeartbeatMonitor(store, 1, 3, timeout=5.0, clock=lambda: now[0])
    with pytest.raises(PeerFailure) as e:
        a.check()                                   # rank 2 never joined
    assert e.value.rank == 2 and "never joined" in e.value.reason
    c = HeartbeatMonitor(store, 2, 3, timeout=5.0, clock=lambda: now[0])
    a.check()
    now[0] += 3.0
    a._publish(); b._publish()                      # rank 2 stays silent
    a.check()
    now[0] += 3.0
    a._publish(); b._publish()
    with pytest.raises(PeerFailure) as e:
        a.check()
    assert e.value.rank == 2 and "no heartbeat" in e.value.reason
    c._publish()
    a.check()
    b.fail("RuntimeError: out of memory")
    with pytest.raises(PeerFailure) as e:
        a.check()
    assert e.value.rank == 1 and "out of memory" in e.value.reason
    b._state = "ok"; b._publish()
    c.leave()
    with pytest.raises(PeerFailure) as e:
        a.check()
    assert e.value.rank == 2 and "left" in e.value.reason


def test_heartbeat_step_lag():
    store = _store()
    a = HeartbeatMonitor(store, 0, 2, max_step_lag=3)
    b = HeartbeatMonitor(store, 1, 2, max_step_lag=3)
    b.beat(10); b._publish()
    a.guard(12)
    with pytest.raises(PeerFailure) as e:
        a.guard(14)
    assert "stalled at step 10" in e.value.reason


def _rank_main(rank, world, port, die_at, out):
    store = dist.TCPStore("127.0.0.1", port, is_master=False, timeout=__import__("datetime").timedelta(seconds=30))
    mon = HeartbeatMonitor(store, rank, world, interval=0.05, timeout=3.0).start()
    store.set(f"ready/{rank}", "1")
    store.wait([f"ready/{r}" for r in range(world)])   # everybody has published once
    try:
        for step in range(200):
            if rank == 1 and step == die_at:
                os._exit(17)                         # dies between steps without a word
            mon.guard(step)
            time.sleep(0.02)
        out.put((rank, "finished"))
    except PeerFailure as exc:
        out.put((rank, f"peer {exc.rank}: {exc.reason}"))
    finally:
        mon.stop()


def test_heartbeat_across_processes_when_a_rank_dies():
    """Three host processes; rank 1 exits between steps.  The survivors notice through the store (no collective
    is in flight) and leave their loops with a PeerFailure naming rank 1."""
    import datetime

    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 29000 + os.getpid() % 900
    # the key-value store lives outside the ranks (as with a launcher-hosted rendezvous store), so it survives them
    master = dist.TCPStore("127.0.0.1", port, is_master=True, wait_for_workers=False, timeout=datetime.timedelta(seconds=30))
    procs = [ctx.Process(target=_rank_main, args=(r, 3, port, 20, out)) for r in range(3)]
    for p in procs:
        p.start()
    got = {}
    deadline = time.time() + 120
    while len(got) < 2 and time.time() < deadline:
        if not out.empty():
            r, msg = out.get()
            got[r] = msg
        else:
            time.sleep(0.05)
    for p in procs:
        p.join(timeout=20)
    assert procs[1].exitcode == 17
    assert set(got) == {0, 2}, got
    assert all("peer 1" in m and "no heartbeat" in m for m in got.values()), got
    del master


def test_status_words_poll():
    words = StatusWords()
    ok, bad = torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32)
    words.register("barrier", ok)
    words.register("fused_mlp", bad, lambda c: {2: "input tile wait expired"}.get(c, str(c)))
    words.poll()
    bad.fill_(2)
    with pytest.raises(RuntimeError, match="fused_mlp: input tile wait expired"):
        words.poll()


def test_async_sharded_checkpoint_roundtrip(tmp_path):
    ck = AsyncCheckpointer(str(tmp_path), keep_last=2)
    state = {"model": {"w": torch.randn(4, 5), "nested": [torch.arange(3), {"b": torch.ones(2)}]}, "iteration": 7}
    torch.manual_seed(123)
    expect = None
    for step in (10, 20, 30):
        state["iteration"] = step
        path = ck.save_step(step, state, meta={"expname": "t"})
        if step == 30:
            expect = torch.rand(3)                   # drawn right after the RNG state was captured
    ck.wait()
    assert sorted(os.listdir(tmp_path)) == ["step-00000020", "step-00000030"]      # oldest pruned, no temp dirs left
    assert latest_checkpoint(str(tmp_path)) == path
    got = load_sharded(path, restore_rng=True)
    assert got["meta"]["step"] == 30 and got["meta"]["world"] == 1 and got["state"]["iteration"] == 30
    assert torch.equal(got["state"]["model"]["w"], state["model"]["w"])
    assert torch.equal(got["state"]["model"]["nested"][1]["b"], torch.ones(2))
    assert torch.equal(torch.rand(3), expect)        # RNG stream continues where the checkpoint was taken


def test_incomplete_checkpoint_is_ignored(tmp_path):
    os.makedirs(tmp_path / "step-00000005")
    (tmp_path / "step-00000005" / "meta.json").write_text("{}")
    assert latest_checkpoint(str(tmp_path)) is None
    with pytest.raises(FileNotFoundError):
        load_sharded(str(tmp_path / "step-00000005"))


def _ckpt_rank(rank, world, root, store_file, delay, q):
    """One rank of a two-rank save: rank 1 is slow; rank 0 must not publish before rank 1's shard exists."""
    import time

    import torch.distributed as dist

    store = dist.FileStore(store_file, world)
    ck = AsyncCheckpointer(root)
    if delay:
        real_save = torch.save

        def slow_save(obj, path, *a, **k):
            time.sleep(delay)
            return real_save(obj, path, *a, **k)

        torch.save = slow_save
    try:
        path = ck.save_step(3, {"w": torch.full((4,), float(rank))}, rank=rank, world=world, store=store)
        ck.wait()
        q.put((rank, "ok", path))
    except BaseException as exc:  # noqa: BLE001 - reported to the parent
        q.put((rank, "error", repr(exc)))


def test_multi_rank_checkpoint_waits_for_the_slow_rank(tmp_path):
    import multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    store_file = str(tmp_path / "store")
    root = str(tmp_path / "ck")
    procs = [ctx.Process(target=_ckpt_rank, args=(r, 2, root, store_file, 1.5 if r == 1 else 0.0, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict((r, (s, m)) for r, s, m in (q.get(timeout=60) for _ in procs))
    for p in procs:
        p.join(timeout=20)
    assert got[0][0] == "ok" and got[1][0] == "ok", got
    path = got[0][1]
    assert sorted(os.listdir(path)) == ["COMPLETE", "meta.json", "shard-00000-of-00002.pt", "shard-00001-of-00002.pt"]
    for r in range(2):
        assert float(load_sharded(path, rank=r)["state"]["w"][0]) == float(r)


def test_multi_rank_checkpoint_without_rendezvous_is_refused(tmp_path):
    with pytest.raises(ValueError, match="rendezvous"):
        AsyncCheckpointer(str(tmp_path)).save_step(1, {"w": torch.zeros(1)}, rank=0, world=2)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["clone", "block"])
def test_async_checkpoint_from_device_is_a_snapshot(tmp_path, mode):
    """A 1 GiB tensor is saved and then updated in place many times right away (each update is far shorter than the
    device-to-host copy): the checkpoint must hold the value at the time of the call, in the staging-clone mode and in
    the mode where the training stream waits for the copies.  A temporary that is freed right after the call (what a
    ``state_dict`` hook produces) must survive until its copy has been read."""
    ck = AsyncCheckpointer(str(tmp_path), snapshot=mode)
    w = torch.full((1 << 28,), 1.0, device="cuda")
    tmp = torch.full((1 << 24,), 5.0, device="cuda")
    path = ck.save_step(1, {"w": w, "tmp": tmp * 1.0})
    del tmp
    for _ in range(64):
        w.add_(1.0)
        junk = torch.full((1 << 24,), -1.0, device="cuda")      # would reuse the freed temporary's memory
        del junk
    ck.wait()
    state = load_sharded(path)["state"]
    assert float(state["w"].max()) == 1.0 and float(state["w"].min()) == 1.0
    assert float(state["tmp"].min()) == 5.0 and float(state["tmp"].max()) == 5.0
    assert float(w[0]) == 65.0


@pytest.mark.gpu
def test_peer_barrier_wait_gives_up_and_reports_the_missing_peer():
    """A barrier among two ranks of which only rank 0 exists: nothing ever sets the flag that rank 1 would write, the
    wait for it runs out after a few milliseconds of SM clocks, the kernel returns and the status word names the peer
    (100 + 1).  A bounded wait, not a hang: the context stays usable and a second barrier reports again."""
    import ctypes

    from landmarksystem_b200.comm import symmetric  # noqa: F401  (registers the signatures)
    from landmarksystem_b200.ops import native

    dev = torch.device("cuda")
    flags = torch.zeros(64, dtype=torch.int32, device=dev)                      # this rank's flag array
    sink = torch.zeros(64, dtype=torch.int32, device=dev)                       # stands in for the absent peer's array
    table = torch.tensor([flags.data_ptr(), sink.data_ptr()], dtype=torch.int64, device=dev)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    limit = 10_000_000                                                          # ~5 ms at 2 GHz
    for expect_epoch in (1, 2):
        status.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        native.check(native.lib().lmb_peer_barrier(flags.data_ptr(), table.data_ptr(), 0, 2, epoch.data_ptr(),
                                                   status.data_ptr(), ctypes.c_longlong(limit), native.stream_ptr()),
                     "peer_barrier")
        end.record()
        torch.cuda.synchronize()
        assert int(status) == 101
        assert int(epoch) == expect_epoch
        assert int(flags[0]) == expect_epoch          # the rank's own signal to itself did arrive
        assert start.elapsed_time(end) < 1000.0       # gave up after milliseconds, not the one-second default
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0                 # the context still works


def test_multicast_probe_is_false_without_a_gpu():
    """The NVLink-multicast probe only reads a driver attribute; on a machine without a GPU it answers False."""
    from landmarksystem_b200.comm.symmetric import multicast_supported

    if not torch.cuda.is_available():
        assert multicast_supported() is False
    else:
        assert multicast_supported() in (True, False)
