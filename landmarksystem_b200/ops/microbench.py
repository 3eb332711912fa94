"""Kernel micro-benchmarks: ``python -m landmarksystem_b200.ops.microbench <name> [--rows N] [--iters K]``.

Each case times one library kernel in isolation with CUDA events (after warm-up, inputs larger than the
126 MB L2 or an L2 flush between launches) and prints one JSON line with the algorithmic bytes / FLOPs,
the achieved rate and its fraction of the measured peaks (``MEASURED_PEAKS.json`` at the repository root
when present: STREAM-style copy bandwidth and cuBLAS bf16 throughput on the same GPU model).  The same
command line is what the profiler captures are taken from.

Cases: ``adam`` (dense fused Adam), ``lazy_adam`` (deferred Adam step over the touched texels of a plane),
``vm_fwd`` / ``vm_bwd`` (plane x line lookup), ``mlp_fwd`` / ``mlp_bwd`` (tcgen05 colour head),
``composite`` (volume-render weights + colour), ``hash_fwd`` (multiresolution hash grid), ``zero_adam_emulated`` /
``merge_emulated`` (the peer-memory kernels with all eight "peers" on one GPU).
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Callable, Dict

import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def measured_peaks() -> Dict[str, float]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path, encoding="utf-8") as fh:
            data = json.load(fh)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS)


class _L2Flush:
    def __init__(self, enabled: bool):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if enabled else None

    def __call__(self):
        if self.buf is not None:
            self.buf.zero_()


def time_kernel(fn: Callable[[], None], iters: int, warmup: int = 3, flush_l2: bool = False, setup: Callable[[], None] = None):
    """Median and best device time (ms) of ``fn`` over ``iters`` launches; ``setup`` runs untimed before each."""
    flush = _L2Flush(flush_l2)
    for _ in range(warmup):
        if setup:
            setup()
        fn()
    times = []
    for _ in range(iters):
        if setup:
            setup()
        flush()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    times.sort()
    return times[len(times) // 2], times[0]


def _report(name, ms, best, bytes_=0.0, flops=0.0, **extra):
    peaks = measured_peaks()
    out = {"kernel": name, "ms_median": round(ms, 4), "ms_best": round(best, 4)}
    if bytes_:
        gbs = bytes_ / (ms * 1e-3) / 1e9
        out.update(algorithmic_gb=round(bytes_ / 1e9, 3), gbs=round(gbs, 1),
                   frac_of_hbm_peak=round(gbs / peaks["hbm_gbs"], 3))
    if flops:
        tf = flops / (ms * 1e-3) / 1e12
        out.update(algorithmic_gflop=round(flops / 1e9, 2), tflops=round(tf, 1),
                   frac_of_bf16_peak=round(tf / peaks["bf16_tflops"], 3))
    out["peaks"] = f'{peaks["source"]}: {peaks["hbm_gbs"]} GB/s, {peaks["bf16_tflops"]} TFLOP/s'
    out.update(extra)
    print(json.dumps(out), flush=True)
    return out


# -- cases ----------------------------------------------------------------------------------------
def case_adam(args):
    from . import FusedAdam

    n = args.rows * 64
    p = torch.nn.Parameter(torch.randn(n, device="cuda"))
    FusedAdam.attach_sink(p, shadow=True)
    opt = FusedAdam([p], lr=1e-3)
    p._lmb_grad_sink.normal_()
    ms, best = time_kernel(opt.step, args.iters)
    return _report("adam_kernel<shadow>", ms, best, bytes_=n * 34.0, params=n)


def case_lazy_adam(args):
    from . import FusedAdam

    C, side = args.channels, args.plane
    p = torch.nn.Parameter(torch.randn(1, side, side, C, device="cuda") * 0.1)
    FusedAdam.attach_sink(p, shadow=True, lazy=True)
    opt = FusedAdam([{"params": [p], "lr": 0.02, "lr_decay": 0.999}])
    state = p._lmb_lazy
    gen = torch.Generator(device="cuda").manual_seed(0)
    touched = [0]

    def setup():
        coords = torch.rand(args.rows, 4, device="cuda", generator=gen) * 2 - 1
        coords[:, 3] = 0
        state.prepare(p, coords)
        mask = state.need != 0
        touched[0] = int(mask.sum())
        p._lmb_grad_sink.view(-1, C)[mask] = 0.01

    ms, best = time_kernel(opt.step, args.iters, warmup=6, setup=setup)
    # per touched texel: read p, g, m, v; write p, g, m, v (fp32) + bf16 shadow + flag/last-step; plus one flag byte per texel
    bytes_ = touched[0] * (C * 4 * 8 + C * 2 + 6) + side * side
    return _report("lazy_scan_kernel<step>", ms, best, bytes_=float(bytes_), touched_texels=touched[0],
                   touched_fraction=round(touched[0] / side ** 2, 3), channels=C)


def _vm_setup(args):
    C, side = args.channels, args.plane
    planes = [torch.nn.Parameter(torch.randn(1, side, side, C, device="cuda") * 0.1)]
    lines = [torch.nn.Parameter(torch.randn(1, 512, C, device="cuda") * 0.1)]
    from . import FusedAdam

    for t in planes + lines:
        FusedAdam.attach_sink(t, shadow=True)
    coords = torch.rand(args.rows, 4, device="cuda") * 2 - 1
    coords[:, 3] = 0
    return planes, lines, coords.contiguous()


def case_vm_fwd(args):
    from .vm import vm_encode

    planes, lines, coords = _vm_setup(args)
    C = args.channels
    with torch.no_grad():
        fn = lambda: vm_encode(coords, planes, lines, [p._lmb_shadow for p in planes], [l._lmb_shadow for l in lines],
                               out_dtype=torch.bfloat16)
        ms, best = time_kernel(fn, args.iters)
    # per sample: 4 plane texels + 2 line entries (bf16) in, one bf16 feature row out, 16 B coordinate
    return _report("vm_encode_fwd_kernel<bf16,bf16>", ms, best, bytes_=args.rows * (6 * C * 2 + C * 2 + 16.0), channels=C)


def case_vm_bwd(args):
    from .vm import vm_encode

    planes, lines, coords = _vm_setup(args)
    C = args.channels
    out = vm_encode(coords, planes, lines, [p._lmb_shadow for p in planes], [l._lmb_shadow for l in lines], out_dtype=torch.bfloat16)
    dout = torch.randn_like(out)
    ms, best = time_kernel(lambda: out.backward(dout, retain_graph=True), args.iters)
    # per sample: re-read 6 bf16 rows + bf16 dout row, reduce 6 fp32 rows into the accumulators
    return _report("vm_encode_bwd_kernel<bf16,bf16>", ms, best, bytes_=args.rows * (6 * C * 2 + C * 2 + 6 * C * 4 + 16.0), channels=C)


def case_vm_bwd_sorted(args):
    from . import vm
    from .vm import vm_encode

    planes, lines, coords = _vm_setup(args)
    C = args.channels
    out = vm_encode(coords, planes, lines, [p._lmb_shadow for p in planes], [l._lmb_shadow for l in lines], out_dtype=torch.bfloat16)
    dout = torch.randn_like(out)
    vm.DETERMINISTIC_BACKWARD = True
    try:
        ms, best = time_kernel(lambda: out.backward(dout, retain_graph=True), args.iters)
    finally:
        vm.DETERMINISTIC_BACKWARD = False
    return _report("vm_encode backward, atomic-free (2 radix sorts + 4 plane colours + 2 line colours)", ms, best,
                   bytes_=args.rows * (6 * C * 2 + C * 2 + 6 * C * 4 + 16.0), channels=C)


def _rgb_decoder(n_feat: int):
    from ..models.gridnerf.gridnerf import RGBDecoder

    torch.manual_seed(0)
    return RGBDecoder([n_feat], [1], 27, view_pe=2, fea_pe=2, featureC=128).cuda()


def _mlp_flops(n_feat: int, rows: int, backward: bool) -> float:
    fwd = 2.0 * rows * (n_feat * 27 + 150 * 128 + 128 * 128 + 128 * 3)
    return fwd * 3.0 if backward else fwd       # recompute + data gradients + weight gradients


def case_mlp_fwd(args):
    from . import fused_mlp

    dec = _rgb_decoder(args.channels)
    x = (torch.randn(args.rows, fused_mlp.RGB_IN_WIDTH, device="cuda") * 0.3).to(torch.bfloat16)
    with torch.no_grad():
        ms, best = time_kernel(lambda: fused_mlp.rgb_decoder_forward(dec, None, x), args.iters)
    dec._lmb_packed.check_status()
    return _report("fused_mlp_kernel", ms, best, flops=_mlp_flops(args.channels, args.rows, False),
                   bytes_=args.rows * (fused_mlp.RGB_IN_WIDTH * 2 + 12.0), rows=args.rows)


def case_mlp_bwd(args):
    from . import fused_mlp

    dec = _rgb_decoder(args.channels)
    x = (torch.randn(args.rows, fused_mlp.RGB_IN_WIDTH, device="cuda") * 0.3).to(torch.bfloat16)
    dout = torch.randn(args.rows, 3, device="cuda")
    ms, best = time_kernel(lambda: fused_mlp.rgb_decoder_backward(dec, x, dout), args.iters)
    dec._lmb_packed.check_status()
    return _report("rgb_mlp_bwd_kernel", ms, best, flops=_mlp_flops(args.channels, args.rows, True),
                   bytes_=args.rows * (fused_mlp.RGB_IN_WIDTH * 4 + 12.0), rows=args.rows)


def case_mlp3_bwd(args):
    """Backward of a hash-grid colour head (39 -> 64 -> 64 -> 3, sigmoid, no bias) in one tcgen05 launch; the time
    includes building the kernel's 160-wide input rows and clearing the gradient buffer."""
    from ..components.fields.mlp_decoder import MLPDecoder
    from . import fused_mlp

    dec = MLPDecoder(inChanel=39, layer_width=64, num_layers=3, out_dim=3, out_activation=torch.nn.Sigmoid(), mlp_bias=False).cuda()
    x = (torch.randn(args.rows, 39, device="cuda") * 0.5)
    dout = torch.randn(args.rows, 3, device="cuda")
    with torch.no_grad():
        fused_mlp.mlp_forward(dec, x)                      # packs the weights
    packed = dec._lmb_packed
    xb = torch.nn.functional.pad(x, (0, packed.in_width - 39)).to(torch.bfloat16).contiguous()
    ms, best = time_kernel(lambda: fused_mlp.mlp3_backward(packed, xb, dout), args.iters)
    packed.check_status()
    flops = 2.0 * args.rows * (39 * 64 + 64 * 64 + 64 * 3) * 3          # recompute + data + weight gradients, true widths
    return _report("mlp_bwd_kernel<false> 39-64-64-3", ms, best, flops=flops, bytes_=args.rows * (48 * 2 + 160 * 2 * 3 + 12.0),
                   rows=args.rows)


def case_composite(args):
    from .composite import composite_render, composite_weights

    rays, S = max(args.rows // 128, 1), 128
    sigma = torch.rand(rays, S, device="cuda")
    dists = torch.full((rays, S), 0.1, device="cuda")
    rgbs = torch.rand(rays, S, 3, device="cuda")
    z = torch.rand(rays, S, device="cuda").sort(-1).values

    def fn():
        w, _ = composite_weights(sigma, dists)
        composite_render(w, rgbs, z, 0.0)

    with torch.no_grad():
        ms, best = time_kernel(fn, args.iters, flush_l2=True)
    return _report("composite weights+render", ms, best, bytes_=rays * S * (4 * 3 + 4 * 5.0), rays=rays)


def case_ray_losses(args):
    """Distortion loss (value + gradient) and proposal inter-level loss, one warp per ray."""
    from .ray_losses import distortion_per_ray, interlevel_per_ray

    rays, S, E = max(args.rows // 128, 1), 128, 256
    edges = torch.rand(rays, S + 1, device="cuda").sort(-1).values
    w = (torch.rand(rays, S, device="cuda") * 0.05).requires_grad_(True)
    m, d = (edges[:, 1:] + edges[:, :-1]) / 2, edges[:, 1:] - edges[:, :-1]
    ms, best = time_kernel(lambda: distortion_per_ray(w, m, d), args.iters, flush_l2=True)
    out = [_report("distortion loss fwd+grad", ms, best, bytes_=rays * S * 4 * 4.0, rays=rays)]
    env = torch.rand(rays, E + 1, device="cuda").sort(-1).values
    w_env = (torch.rand(rays, E, device="cuda") * 0.02).requires_grad_(True)
    ms, best = time_kernel(lambda: interlevel_per_ray(edges, w.detach(), env, w_env), args.iters, flush_l2=True)
    out.append(_report("interlevel loss fwd+grad", ms, best, bytes_=rays * (2 * S + 3 * E) * 4.0, rays=rays))
    return out


def case_prop_resample(args):
    from .pdf import prop_resample

    rays, E, B = max(args.rows // 128, 1), 256, 97
    existing = torch.rand(rays, E + 1, device="cuda").sort(-1).values
    w = torch.rand(rays, E, device="cuda")
    u = ((torch.arange(B, device="cuda") + torch.rand(rays, B, device="cuda")) / B).contiguous()
    ms, best = time_kernel(lambda: prop_resample(w, existing, u, 0.01, 1e-5, True), args.iters, flush_l2=True)
    return _report("proposal resample + merge", ms, best, bytes_=rays * (2 * E + 1 + B + B + E + 1) * 4.0, rays=rays)


def case_alpha_pool(args):
    from .resize import alpha_mask_pool

    n = 320
    alpha = torch.rand(n, n, n, device="cuda") ** 6
    ms, best = time_kernel(lambda: alpha_mask_pool(alpha, 0.3), args.iters, flush_l2=True)
    return _report("alpha-mask pool 320^3", ms, best, bytes_=n ** 3 * 8.0)


def case_hash_fwd(args):
    import math

    from .hashgrid import hashgrid_encode, make_meta

    meta = make_meta(16, 2, 22, 16, math.exp(math.log(8192 / 16) / 15))
    table = torch.rand(meta.n_params, device="cuda") * 2e-4 - 1e-4
    table._lmb_shadow = table.to(torch.bfloat16)          # the kernels read the bf16 copy
    x = torch.rand(args.rows, 3, device="cuda")
    with torch.no_grad():
        ms, best = time_kernel(lambda: hashgrid_encode(x, table, meta), args.iters)
    # per sample and level: 8 corners x 2 bf16 features in, 2 fp32 features out
    return _report("hashgrid fwd", ms, best, bytes_=args.rows * 16 * (8 * 4 + 8.0), rows=args.rows)


# -- peer-memory kernels with the peers emulated on one GPU --------------------------------------------------
# The fused compute+collective kernels take a table of peer addresses.  Here every "peer" is another buffer on the
# SAME GPU and ONE launch plays one rank of an 8-rank job (no barrier is needed: nothing else writes the buffers), so
# the kernel's own behaviour - instruction mix, access pattern, traffic per element - can be profiled on a single
# GPU.  The loads that would cross NVLink hit local HBM instead; link-level figures come from the multi-GPU tests.
def _ptr_table(tensors):
    import ctypes

    return (ctypes.c_longlong * len(tensors))(*[t.data_ptr() for t in tensors])


def case_zero_adam_emulated(args):
    from . import native
    from ..parallel import zero_adam  # noqa: F401  (registers the entry point's signature)

    world, n = 8, args.rows * 64
    grads = [torch.randn(n, device="cuda") for _ in range(world)]
    params = [torch.zeros(n, device="cuda") for _ in range(world)]
    shadows = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    m = torch.zeros(n // world, device="cuda")
    v = torch.zeros(n // world, device="cuda")
    gt, pt, st = _ptr_table(grads), _ptr_table(params), _ptr_table(shadows)
    step = [0]

    def fn():
        step[0] += 1
        native.check(native.lib().lmb_zero_adam_p2p(gt, pt, st, m.data_ptr(), v.data_ptr(), n, 0, world, 1e-3, 0.9, 0.99, 1e-8,
                                                    step[0], 1.0, native.stream_ptr()), "zero_adam_p2p")

    ms, best = time_kernel(fn, args.iters)
    shard = n // world
    # per shard element: world gradient loads, p / m / v read and written, the new value + bf16 shadow stored to every rank
    bytes_ = shard * (world * 4 + 12 + 8 + world * 6.0)
    return _report("zero_adam_p2p_kernel (8 ranks emulated on one GPU, rank 0's shard)", ms, best, bytes_=bytes_,
                   params=n, shard=shard)


def case_merge_emulated(args):
    from . import native
    from ..parallel import composite_merge  # noqa: F401

    world, R = 8, 1920 * 1080
    gen = torch.Generator(device="cuda").manual_seed(0)
    partials = []
    for r in range(world):
        p = torch.rand(R, 8, device="cuda", generator=gen)
        p[:, 6] = (torch.randint(0, 1 << 20, (R,), device="cuda", generator=gen) * 8 + r).float()
        partials.append(p.contiguous())
    outs = [torch.zeros(R, 6, device="cuda") for _ in range(world)]
    pt, ot = _ptr_table(partials), _ptr_table(outs)

    def fn():
        native.check(native.lib().lmb_composite_merge_p2p(pt, ot, R, 0, world, -1, 1.0, native.stream_ptr()), "composite_merge_p2p")

    ms, best = time_kernel(fn, args.iters, flush_l2=True)
    rays = (R + world - 1) // world
    return _report("composite_merge_p2p_kernel (8 ranks emulated on one GPU, rank 0's ray slice)", ms, best,
                   bytes_=rays * (world * 32 + world * 24.0), rays=rays)


def case_a2a_emulated(args):
    """The spatial-block all-to-all on one GPU (the rank is its own and only peer: same kernels, flags and waits as the
    multi-GPU runs, peer stores landing in local memory): one sigma-shaped query - 16-byte records out, 4 bytes back."""
    from ..parallel.branch_dispatch import BlockDispatcher

    n = args.rows
    gen = torch.Generator(device="cuda").manual_seed(0)
    disp = BlockDispatcher(n, max_w=6, max_v=3)
    payload = torch.rand(n, 4, device="cuda", generator=gen)
    payload[:, 3] = 0.0
    owner = torch.zeros(n, dtype=torch.int32, device="cuda")
    w = torch.randn(3, 1, device="cuda", generator=gen)

    class Owner:
        def parameters_for_autograd(self):
            return []

        def __call__(self, coords, extra, m):
            return torch.tanh(coords[:, :3] @ w)

    fn = Owner()
    with torch.no_grad():
        ms, best = time_kernel(lambda: disp.query(payload, owner, fn, 1, channel="bench"), args.iters)
    disp.check()
    # dispatch: 16 B read + 16 B stored to the owner; collect: 16 B read + 16 B written; combine / result: 4 B each way twice
    return _report("a2a dispatch + collect + owner map + combine + result (1 rank, peers emulated)", ms, best,
                   bytes_=n * (32 + 32 + 16.0), rows=n)


def case_mlp_fwd_sources(args):
    """The colour head with its input assembled from two sources (feature block + direction block), the path the
    channel-parallel gather uses for peer slices; both sources are local here."""
    from ..parallel.channel_gather_mlp import ChannelGatherColourHead

    dec = _rgb_decoder(args.channels)                  # one level of `channels` appearance features
    assert dec.basis_mat.weight.shape[1] == args.channels
    head = ChannelGatherColourHead(dec, n_levels=1, channels_per_rank=args.channels, max_rows=args.rows)
    feat = (torch.randn(args.rows, args.channels, device="cuda") * 0.3).to(torch.bfloat16)
    dirs = torch.nn.functional.normalize(torch.randn(args.rows, 3, device="cuda"), dim=-1)
    ms, best = time_kernel(lambda: head(feat, dirs), args.iters)
    return _report("fused_mlp_kernel, two input sources (copy into the symmetric buffer and two barriers included)", ms, best,
                   flops=_mlp_flops(args.channels, args.rows, False), bytes_=args.rows * (args.channels * 2 * 3 + 32 + 12.0),
                   rows=args.rows)


CASES = {"a2a_emulated": case_a2a_emulated, "mlp_fwd_sources": case_mlp_fwd_sources, "mlp3_bwd": case_mlp3_bwd, "ray_losses": case_ray_losses, "prop_resample": case_prop_resample, "alpha_pool": case_alpha_pool,
         "zero_adam_emulated": case_zero_adam_emulated, "merge_emulated": case_merge_emulated, "adam": case_adam, "lazy_adam": case_lazy_adam, "vm_fwd": case_vm_fwd, "vm_bwd": case_vm_bwd, "vm_bwd_sorted": case_vm_bwd_sorted,
         "mlp_fwd": case_mlp_fwd, "mlp_bwd": case_mlp_bwd, "composite": case_composite, "hash_fwd": case_hash_fwd}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--rows", type=int, default=1 << 20, help="samples / rows per launch")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--channels", type=int, default=48, help="feature channels of the plane / appearance features")
    ap.add_argument("--plane", type=int, default=4096, help="plane side length (lazy_adam, vm_*)")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    names = sorted(CASES) if args.case == "all" else [args.case]
    for name in names:
        CASES[name](args)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
