"""PyTorch reference implementations of the ops, checked against independent formulations."""
import torch
import torch.nn.functional as F

from landmarksystem_b200.ops import FusedAdam, composite_render, composite_weights, vm_encode_reference
from landmarksystem_b200.ops.hashgrid import hashgrid_reference, make_meta


def test_vm_reference_matches_grid_sample():
    """The channels-last lookup equals the two F.grid_sample calls + product of the stacked-plane layout."""
    torch.manual_seed(0)
    B, H, W, Z, C, N = 3, 9, 7, 5, 8, 200
    plane = torch.randn(B, H, W, C)
    line = torch.randn(B, Z, C)
    coords = torch.rand(N, 4) * 2 - 1
    block = torch.randint(0, B, (N,)).float()
    coords[:, 3] = block
    got = vm_encode_reference(coords, [plane], [line])
    plane_ref = plane.permute(3, 0, 1, 2)[None]                      # [1,C,B,H,W]
    line_ref = line.permute(2, 1, 0)[None]                           # [1,C,Z,B]
    bnorm = -1 + 2 * block / (B - 1)
    g3 = torch.stack((coords[:, 0], coords[:, 1], bnorm), -1).view(1, N, 1, 1, 3)
    pf = F.grid_sample(plane_ref, g3, align_corners=True).view(C, N).t()
    g2 = torch.stack((bnorm, coords[:, 2]), -1).view(1, N, 1, 2)
    lf = F.grid_sample(line_ref, g2, align_corners=True).view(C, N).t()
    assert torch.allclose(got, pf * lf, atol=1e-5)


def test_vm_reference_invalid_block_is_zero():
    plane, line = torch.randn(2, 4, 4, 8), torch.randn(2, 4, 8)
    coords = torch.tensor([[0.0, 0.0, 0.0, -1.0], [0.1, 0.2, 0.3, 5.0]])
    assert vm_encode_reference(coords, [plane], [line]).abs().sum() == 0


def test_weights_and_render_reference():
    torch.manual_seed(0)
    sigma, dists = torch.rand(4, 16) * 3, torch.rand(4, 16) * 0.2
    w, bg = composite_weights(sigma, dists)
    alpha = 1 - torch.exp(-sigma * dists)
    T = torch.ones(4)
    for s in range(16):
        assert torch.allclose(w[:, s], alpha[:, s] * T, atol=1e-6)
        T = T * (1 - alpha[:, s] + 1e-10)
    assert torch.allclose(bg, T, atol=1e-6)
    rgb, depth, acc = composite_render(w, torch.rand(4, 16, 3), torch.rand(4, 16), 1.0)
    assert rgb.shape == (4, 3) and depth.shape == (4,) and torch.allclose(acc, w.sum(-1))


def test_fused_adam_cpu_matches_torch_adam():
    torch.manual_seed(0)
    a = torch.nn.Parameter(torch.randn(37))
    b = torch.nn.Parameter(a.detach().clone())
    o1 = FusedAdam([a], lr=0.02, betas=(0.9, 0.99), eps=1e-8)
    o2 = torch.optim.Adam([b], lr=0.02, betas=(0.9, 0.99), eps=1e-8)
    for _ in range(5):
        g = torch.randn(37)
        a.grad, b.grad = g.clone(), g.clone()
        o1.step(); o2.step()
    assert torch.allclose(a, b, atol=1e-6)


def test_fused_radam_cpu_matches_torch_radam():
    from landmarksystem_b200.ops import FusedRAdam

    torch.manual_seed(0)
    a = torch.nn.Parameter(torch.randn(37))
    b = torch.nn.Parameter(a.detach().clone())
    o1, o2 = FusedRAdam([a], lr=0.02, eps=1e-8), torch.optim.RAdam([b], lr=0.02, eps=1e-8)
    for _ in range(10):          # crosses the switch to the rectified update (step 6)
        g = torch.randn(37)
        a.grad, b.grad = g.clone(), g.clone()
        o1.step(); o2.step()
    assert torch.allclose(a, b, atol=1e-6)


def test_hashgrid_reference_dense_level_interpolates():
    meta = make_meta(2, 2, 10, 4, 2.0)
    assert meta.resolutions[0] == 4 and meta.offsets[1] == 64   # 4^3 dense entries
    table = torch.zeros(meta.offsets[-1], 2)
    table[: meta.offsets[1], 0] = 1.0
    x = torch.rand(50, 3)
    out = hashgrid_reference(x, table, meta)
    assert out.shape == (50, 4) and torch.allclose(out[:, 0], torch.ones(50), atol=1e-5)
    assert out[:, 1].abs().max() == 0


def test_cat_pad_bf16_concatenates_pads_and_routes_gradients():
    """Input assembly of the fused MLP path: parts -> one zero-padded bf16 row block; each part gets its gradient slice."""
    from landmarksystem_b200.ops.fused_mlp import _CatPadBf16

    torch.manual_seed(0)
    a = torch.randn(7, 3, requires_grad=True)
    b = torch.randn(7, 5)                                   # no gradient wanted
    c = torch.randn(7, 2, requires_grad=True)
    out = _CatPadBf16.apply(16, a, b, c)
    assert out.dtype == torch.bfloat16 and out.shape == (7, 16)
    ref = torch.cat((a, b, c), -1).detach().to(torch.bfloat16)
    assert torch.equal(out[:, :10], ref) and out[:, 10:].abs().max() == 0
    g = torch.randn(7, 16).to(torch.bfloat16)
    out.backward(g)
    assert torch.equal(a.grad, g[:, :3].float()) and torch.equal(c.grad, g[:, 8:10].float()) and b.grad is None


def test_small_helpers_under_reference_names():
    """``gaussian / create_window`` (SSIM filter), ``build_covariance_from_scaling_rotation``, ``getNeRFppNorm``,
    ``PILtoTorch``, ``activation_to_tcnn_string`` and ``contract``."""
    from types import SimpleNamespace

    import numpy as np
    import pytest

    from landmarksystem_b200.components.data.datasets.dataset_utils import PILtoTorch, getNeRFppNorm
    from landmarksystem_b200.components.fields.encodings.gaussian_encoding import build_covariance_from_scaling_rotation
    from landmarksystem_b200.components.fields.fused_mlp_decoder import activation_to_tcnn_string
    from landmarksystem_b200.components.ray_samplers.proposal_network_sampler import contract
    from landmarksystem_b200.components.utils.loss_utils import create_window, gaussian

    g = gaussian(11, 1.5)
    w = create_window(11, 3)
    assert abs(float(g.sum()) - 1) < 1e-6 and int(g.argmax()) == 5 and torch.allclose(w[1, 0], torch.outer(g, g))
    cov = build_covariance_from_scaling_rotation(torch.tensor([[1.0, 2.0, 3.0]]), 2.0, torch.tensor([[1.0, 0, 0, 0]]))
    assert torch.allclose(cov, torch.tensor([[4.0, 0, 0, 16.0, 0, 36.0]]))
    cams = [SimpleNamespace(camera_center=torch.tensor(c)) for c in ([0.0, 0, 0], [2.0, 0, 0], [1.0, 3.0, 0])]
    norm = getNeRFppNorm(cams)
    assert np.allclose(norm["translate"], [-1.0, -1.0, 0.0]) and abs(norm["radius"] - 1.1 * 2.0) < 1e-6
    assert PILtoTorch(np.full((4, 5), 255, np.uint8)).shape == (1, 4, 5)
    assert float(PILtoTorch(np.full((4, 5, 3), 51, np.uint8)).max()) == pytest.approx(0.2)
    assert activation_to_tcnn_string(torch.nn.LeakyReLU()) == "Leaky ReLU" and activation_to_tcnn_string(None) == "None"
    with pytest.raises(ValueError):
        activation_to_tcnn_string(torch.nn.GELU())
    assert torch.allclose(contract(torch.tensor([[0.5, 0, 0], [4.0, 0, 0]])), torch.tensor([[0.5, 0, 0], [1.75, 0, 0]]))


def test_tcnn_shaped_front_end():
    """``tcnn.Encoding`` / ``tcnn.Network`` descriptions of the reference's call sites (hash_encoding.py:97-107,
    sh_encoding.py:35-38, fused_mlp_decoder.py:86-90) served by this package's own components."""
    import pytest

    from landmarksystem_b200.components.utils.tcnn_utils import TCNN_EXISTS, tcnn
    from landmarksystem_b200.ops.ngp_field import sh_encode

    assert TCNN_EXISTS
    torch.manual_seed(0)
    enc = tcnn.Encoding(3, {"otype": "HashGrid", "n_levels": 4, "n_features_per_level": 2, "log2_hashmap_size": 10,
                            "base_resolution": 4, "per_level_scale": 1.5}, device="cpu")
    with torch.no_grad():
        enc.params.normal_()
    x = torch.rand(7, 5, 3)
    ref = hashgrid_reference(x.reshape(-1, 3), enc.params.view(-1, 2), make_meta(4, 2, 10, 4, 1.5)).reshape(7, 5, 8)
    assert enc.n_output_dims == 8 and torch.allclose(enc(x), ref, atol=1e-6)
    enc(x).sum().backward()
    assert enc.params.grad is not None and enc.params.grad.abs().sum() > 0

    sh = tcnn.Encoding(3, {"otype": "SphericalHarmonics", "degree": 4}, device="cpu")
    d = F.normalize(torch.randn(6, 3), dim=-1)
    assert sh.n_output_dims == 16 and torch.allclose(sh((d + 1) / 2), sh_encode(d, 4, False), atol=1e-5)

    net = tcnn.Network(32, 16, {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None",
                                "n_neurons": 64, "n_hidden_layers": 1}, device="cpu")
    w0, w1 = [p for p in net.inner.parameters()]
    h = torch.randn(3, 4, 32)
    assert net.params.numel() == 32 * 64 + 64 * 16
    assert torch.allclose(net(h), torch.relu(h @ w0.T) @ w1.T, atol=1e-5)
    both = tcnn.NetworkWithInputEncoding(3, 4, {"otype": "HashGrid", "n_levels": 2, "base_resolution": 4,
                                                "per_level_scale": 2.0, "log2_hashmap_size": 8},
                                         {"otype": "CutlassMLP", "n_neurons": 16, "n_hidden_layers": 2,
                                          "output_activation": "Sigmoid"}, device="cpu")
    out = both(torch.rand(9, 3))
    assert out.shape == (9, 4) and float(out.detach().min()) > 0 and float(out.detach().max()) < 1
    with pytest.raises(ValueError):
        tcnn.Encoding(3, {"otype": "Frequency"})
    with pytest.raises(ValueError):
        tcnn.Network(3, 3, {"otype": "FullyFusedMLP", "activation": "Tanh"})


def test_pose_rotate_translate_both_calling_conventions():
    """Camera-to-world in / out with vectors, or the reference's world-to-view in / out with three angles (positional
    or by keyword, graphics_utils.py:88-123): the same rigid motion."""
    import numpy as np

    from landmarksystem_b200.components.data import pose_utils as pu
    from landmarksystem_b200.components.utils.graphics_utils import pose_rotate_translate

    c2w = np.concatenate((pu.viewmatrix([0.2, 1, 0.1], [0, 0, 1], [1, -3, 0.5]), [[0, 0, 0, 1]]))
    moved = pose_rotate_translate(c2w, [10, 20, 30], [1, 2, 3])
    assert np.allclose(moved[:3, 3], (moved[:3, :3] @ np.linalg.inv(c2w[:3, :3])) @ c2w[:3, 3] + [1, 2, 3], atol=1e-5)
    w2v = np.linalg.inv(c2w)
    for out in (pose_rotate_translate(w2v, 10, 20, 30, [1, 2, 3]),
                pose_rotate_translate(w2v, rot_x=10, rot_y=20, rot_z=30, trans=[1, 2, 3])):
        assert np.allclose(np.linalg.inv(out.astype(np.float64)), moved, atol=1e-5)
