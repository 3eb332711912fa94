"""Worker launched by torch.distributed.run on 2 GPUs: dynamic loading with the NVLink fan-out.  Every rank reads half
of each new block from its pinned host copy and receives the other half from its peer; the windows must equal the
blocks, and the host link must carry half the bytes per rank."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from landmarksystem_b200.render.offload.block import Block  # noqa: E402
from landmarksystem_b200.render.offload.buffer_manager import BufferManager  # noqa: E402


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    group = dist.new_group(list(range(world)))
    torch.manual_seed(0)                      # every rank holds the same blocks in its own pinned memory
    blocks = []
    for b in range(6):
        sd = {"plane": torch.randn(1, 256, 256, 16).to(torch.bfloat16).pin_memory(),     # 2 MiB: fanned out
              "line": torch.randn(1, 16, 300).pin_memory(),                              # 19 KB: read whole by every rank
              "odd": torch.randn(1, 70001).pin_memory()}                                 # not divisible: read whole
        blocks.append(Block(b, (b // 3, b % 3), state_dict=sd))
    mgr = BufferManager(blocks, [2, 3], [1, 2], "cuda", use_nccl=True, group=group, fanout=True)
    assert mgr.fanout

    def check(idxes):
        torch.cuda.synchronize()
        buf = mgr.get_buffer()
        assert buf.local_block_idxes == idxes
        for slot, b in enumerate(idxes):
            for key, t in buf.state_dict.items():
                want = blocks[b].state_dict[key].cuda().reshape(t[slot].shape)
                assert torch.equal(t[slot], want), (key, slot, b)

    assert mgr.update_buffer([0, 1], init=True)
    mgr.wait_update_done()
    check([0, 1])
    plane_bytes = 256 * 256 * 16 * 2
    small = 16 * 300 * 4 + 70001 * 4
    assert mgr.bytes_h2d == 2 * (plane_bytes // world + small), mgr.bytes_h2d
    assert mgr.bytes_pushed == 2 * (plane_bytes // world) * (world - 1)
    for window in ([1, 2], [4, 5], [5, 3]):            # block 1 / 5 stay resident: device-to-device, no host read
        h0 = mgr.bytes_h2d
        assert mgr.update_buffer(window)
        while not mgr.update_done():
            pass
        mgr.change_buffer()
        check(window)
        new = len(set(window) - set(mgr.buffers[mgr.active ^ 1].local_block_idxes))
        assert mgr.bytes_h2d - h0 == new * (plane_bytes // world + small), (window, new)
    mgr.barrier.check()
    # device-timed streaming of a two-block window of 64 MiB planes, fan-out against every rank reading everything
    big = [Block(b, (0, b), state_dict={"plane": torch.empty(1, 2048, 1024, 16, dtype=torch.bfloat16).pin_memory()})
           for b in range(4)]
    res = {}
    for name, fan in (("fanout", True), ("every_rank_reads_all", False)):
        m = BufferManager(big, [1, 4], [1, 2], "cuda", use_nccl=False, group=group if fan else None, fanout=fan)
        m.update_buffer([0, 1], init=True); m.wait_update_done(); torch.cuda.synchronize(); dist.barrier()
        times = []
        for window in ([2, 3], [0, 1], [2, 3]):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier(); torch.cuda.synchronize()
            s.record(m.copy_stream)
            m.update_buffer(window)
            e.record(m.copy_stream)
            m.change_buffer(); torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        ms = torch.tensor([min(times)], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        res[name + "_ms"] = round(float(ms), 3)
    res["window_MiB"] = 2 * 2048 * 1024 * 16 * 2 / 2 ** 20
    if rank == 0:
        print("OFFLOAD_FANOUT_RESULTS " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
