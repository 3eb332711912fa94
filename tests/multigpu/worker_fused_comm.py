"""Worker launched by torch.distributed.run on >= 2 GPUs: checks the peer-memory kernels against NCCL /
PyTorch references and prints device-timed throughput (max over ranks)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from landmarksystem_b200.parallel.composite_merge import CompositeMerger, merge_reference, pack_partial  # noqa: E402
from landmarksystem_b200.parallel.zero_adam import NcclZeroAdam, P2PZeroAdam  # noqa: E402


def timed(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    ms = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    results = {}

    # ---- ZeRO Adam over peer memory vs the NCCL statement of the same algorithm -----------------------------
    torch.manual_seed(0)
    shapes = [(1000, 64), (37,), (128, 128), (5, 3, 7)]
    pa = [torch.nn.Parameter(torch.randn(*s, device="cuda")) for s in shapes]
    pb = [torch.nn.Parameter(p.detach().clone()) for p in pa]
    opt_a = P2PZeroAdam(pa, lr=0.01, betas=(0.9, 0.99), eps=1e-8, shadow=True)
    opt_b = NcclZeroAdam(pb, lr=0.01, betas=(0.9, 0.99), eps=1e-8)
    for step in range(4):
        g = torch.Generator(device="cuda").manual_seed(100 * step + rank)
        for a, b in zip(pa, pb):
            grad = torch.randn(a.shape, device="cuda", generator=g)
            a._lmb_grad_sink.copy_(grad)
            b.grad = grad.clone()
        opt_a.step()
        opt_b.step()
    opt_a.barrier.check()
    for a, b in zip(pa, pb):
        assert torch.allclose(a, b, atol=2e-6), (a - b).abs().max()
        assert torch.allclose(a._lmb_shadow.float(), a.detach().bfloat16().float())
        assert a._lmb_grad_sink.abs().sum() == 0
    # replicas agree bit for bit
    flat = opt_a.flat.flat_param.clone()
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref)

    # throughput on a grid-sized buffer (256 Mi params = 1 GiB fp32 per replica)
    n = 256 * 1024 * 1024
    big = [torch.nn.Parameter(torch.zeros(n, device="cuda"))]
    opt_big = P2PZeroAdam(big, lr=0.01, shadow=True)
    ms = timed(opt_big.step, iters=5)
    shard = n // world
    nvlink = (world - 1) * shard * 6     # outgoing per rank: new fp32 value + bf16 shadow to every peer
    hbm = shard * (world * 8 + 4 + 8 + 8 + world * 6)
    results["zero_adam_p2p"] = {"ms": ms, "params": n, "nvlink_GBps_per_rank": nvlink / ms / 1e6,
                                "hbm_GBps_per_rank": hbm / ms / 1e6}
    nccl_big = NcclZeroAdam([torch.nn.Parameter(torch.zeros(n, device="cuda"))], lr=0.01)
    nccl_big.params[0].grad = torch.zeros(n, device="cuda")

    def nccl_step():
        nccl_big.params[0].grad = nccl_big.params[0].grad if nccl_big.params[0].grad is not None else torch.zeros(n, device="cuda")
        nccl_big.step()

    results["zero_adam_nccl"] = {"ms": timed(nccl_step, iters=3)}
    del opt_big, nccl_big, big
    torch.cuda.empty_cache()

    # ---- cross-GPU ordered composite ----------------------------------------------------------------------------
    R = 1920 * 1080
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    rgb = torch.rand(R, 3, device="cuda", generator=g) * 0.5
    trans = torch.rand(R, device="cuda", generator=g)
    depth = torch.rand(R, device="cuda", generator=g)
    acc = 1 - trans
    # entry distances are distinct across ranks for every ray (a tie would leave the composite order undefined)
    t_entry = (torch.randint(0, 1 << 20, (R,), device="cuda", generator=g) * 8 + rank).float() * (100.0 / (1 << 23))
    empty = torch.rand(R, device="cuda", generator=g) < 0.3          # rays that miss this rank's blocks
    t_entry[empty] = float("inf")
    rgb[empty], trans[empty], depth[empty], acc[empty] = 0.0, 1.0, 0.0, 0.0
    mine = pack_partial(rgb, trans, depth, acc, t_entry)
    merger = CompositeMerger(R)
    out = merger.merge(mine, bg=1.0, root=-1).clone()
    merger.barrier.check()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    ref = merge_reference(torch.stack(gathered), bg=1.0)
    assert torch.allclose(out, ref, atol=1e-5), (out - ref).abs().max()
    ms = timed(lambda: merger.merge(mine, bg=1.0, root=-1), iters=20)
    per_rank_rays = R // world
    nvlink = (world - 1) * per_rank_rays * (32 + 24)
    results["composite_merge_p2p"] = {"ms": ms, "rays": R, "nvlink_GBps_per_rank": nvlink / ms / 1e6}

    def nccl_merge():
        dist.all_gather(gathered, mine)
        return merge_reference(torch.stack(gathered), bg=1.0)

    results["composite_merge_nccl_torch"] = {"ms": timed(nccl_merge, iters=5)}

    # small all-reduce over peer staging buffers (gradients of replicated heads) vs the NCCL collective
    from landmarksystem_b200.parallel.grad_sync import GradSynchronizer

    shapes = [(128, 150), (128,), (128, 128), (3, 128), (27, 48), (1, 16), (5,)]
    gg = torch.Generator(device="cuda").manual_seed(50 + rank)
    params = []
    for shp in shapes:
        p = torch.nn.Parameter(torch.zeros(shp, device="cuda"))
        p.grad = torch.randn(shp, device="cuda", generator=gg)
        params.append(p)
    want = []
    for p in params:
        t = p.grad.clone()
        dist.all_reduce(t)
        want.append(t)
    sync = GradSynchronizer(None, average=False, p2p_small=True)
    keep = [p.grad.clone() for p in params]

    def p2p_sync():
        for p, k in zip(params, keep):
            p.grad.copy_(k)
        sync.sync(params)

    p2p_sync()
    for p, t in zip(params, want):
        assert torch.allclose(p.grad, t, atol=1e-5), (p.grad - t).abs().max()
    sync._p2p.check()
    results["allreduce_small_p2p"] = {"ms": timed(p2p_sync, iters=20), "floats": sum(p.numel() for p in params)}

    if rank == 0:
        print("FUSED_COMM_RESULTS " + json.dumps({"world": world, **results}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
