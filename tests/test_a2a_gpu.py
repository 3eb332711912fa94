"""All-to-all dispatcher and the small all-reduce on ONE GPU (world 1: the rank is its own and only peer).  The kernels,
the epoch flags raised by a kernel's last block, the waits in the consumers' prologues and the device-side state are the
ones the multi-GPU runs use; only the peers' addresses all point at this GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


class _Fn:
    """Owner-side function: a small differentiable map of (coords, extra) with one parameter."""

    def __init__(self, w):
        self.w = w

    def parameters_for_autograd(self):
        return [self.w]

    def __call__(self, coords, extra, m):
        # rows at and beyond the device-side count m hold whatever was in memory: they are masked with `where`, whose
        # backward also drops the (equally undefined) gradient rows
        x = coords[:, :3] if extra is None else torch.cat((coords[:, :3], extra), -1)
        live = (torch.arange(x.shape[0], device=x.device) < m[0])[:, None]
        x = torch.where(live, x, torch.zeros_like(x))
        return torch.where(live, torch.tanh(x @ self.w[: x.shape[1]]), torch.zeros(1, device=x.device))


def _direct(fn, payload, owner, count):
    n = payload.shape[0]
    k = n if count is None else int(count)
    x = payload
    vals = torch.tanh(x @ fn.w[: x.shape[1]])
    keep = (owner >= 0) & (torch.arange(n, device=payload.device) < k)
    return vals * keep[:, None]


@pytest.mark.parametrize("W,V,use_count", [(3, 1, False), (6, 3, True)])
def test_query_on_one_gpu_matches_direct_evaluation_and_replays_in_a_graph(W, V, use_count):
    side = torch.cuda.Stream()          # everything, leaf creation included, lives on one non-default stream so that the
    side.wait_stream(torch.cuda.current_stream())        # later capture never touches the legacy stream
    with torch.cuda.stream(side):
        _query_case(W, V, use_count, side)
    torch.cuda.current_stream().wait_stream(side)


def _query_case(W, V, use_count, side):
    from landmarksystem_b200.parallel.branch_dispatch import BlockDispatcher

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(5)
    n = 5000
    disp = BlockDispatcher(n, max_w=6, max_v=3)
    w = torch.randn(6, V, device=dev, generator=g, requires_grad=True)
    fn = _Fn(w)
    payload = torch.randn(n, W, device=dev, generator=g)
    owner = torch.where(torch.rand(n, device=dev, generator=g) < 0.2, -1, 0).to(torch.int32)
    count = torch.tensor([3777], dtype=torch.int32, device=dev) if use_count else None
    gout = torch.randn(n, V, device=dev, generator=g)

    def run():
        w.grad = None
        out = disp.query(payload, owner, fn, V, count=count, channel="t")
        (out * gout).sum().backward()
        return out.detach().clone(), w.grad.clone()

    want = _direct(fn, payload, owner, count)
    (want * gout).sum().backward()
    want_grad, w.grad = w.grad.clone(), None
    for _ in range(2):                                  # the second call starts from the first call's epochs and buffers
        out, grad = run()
        torch.testing.assert_close(out, want.detach(), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(grad, want_grad, rtol=1e-4, atol=1e-5)
    # the same sequence recorded once and replayed: epochs live on the device, so a replay is a new hand-over
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    static = {}
    with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):    # the backward runs on autograd's thread
        static["out"], static["grad"] = run()
    for _ in range(3):
        graph.replay()
        torch.cuda.synchronize()
        torch.testing.assert_close(static["out"], want.detach(), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(static["grad"], want_grad, rtol=1e-4, atol=1e-5)
    disp.check()
    assert disp.channels["t"].state[:3].tolist() == [5, 5, 5]     # hand-over epochs (two eager calls, three replays) live on the device


def test_small_all_reduce_on_one_gpu_double_buffers_by_epoch():
    from landmarksystem_b200.parallel.grad_sync import _P2PSmallAllReduce

    ar = _P2PSmallAllReduce(1 << 12)
    for k in range(5):
        x = torch.full((1001,), float(k + 1), device="cuda")
        y = ar(x, 0.5)
        assert y.shape == (1001,) and float(y.min()) == float(y.max()) == 0.5 * (k + 1)
    ar.check()
    assert int(ar.state[0]) == 5
