"""COLMAP readers / datasets, pose helpers and ray-shard preprocessing (CPU)."""
import math
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from landmarksystem_b200.components.data import pose_utils as pu
from landmarksystem_b200.components.data.datasets import colmap_loader as cl
from landmarksystem_b200.components.data.datasets import gaussian_dataset_dict
from landmarksystem_b200.components.data.datasets.processed_dataset import PreprocessedDataset, dist_preprocess, preprocess


def _toy_model(n_images=17):
    rng = np.random.default_rng(0)
    cameras = {1: cl.ColmapCamera(1, "PINHOLE", 64, 48, np.array([80.0, 82.0, 32.0, 24.0])),
               2: cl.ColmapCamera(2, "SIMPLE_RADIAL", 32, 24, np.array([40.0, 16.0, 12.0, 0.01]))}
    images = {}
    for k in range(n_images):
        ang = 2 * math.pi * k / n_images
        c2w = pu.viewmatrix(lookat=-np.array([math.cos(ang), math.sin(ang), 0.3]), up=np.array([0, 0, 1.0]),
                            pos=3 * np.array([math.cos(ang), math.sin(ang), 0.3]))
        c2w = np.concatenate((c2w, [[0, 0, 0, 1]]))
        c2w[:3, 1:3] *= -1                                    # OpenGL -> COLMAP axes
        w2c = np.linalg.inv(c2w)
        n_pts = int(rng.integers(0, 5))
        images[k + 1] = cl.ColmapImage(k + 1, cl.rotmat2qvec(w2c[:3, :3]), w2c[:3, 3], 1 + k % 2, f"img_{k:03d}.png",
                                       rng.random((n_pts, 2)) * 40, rng.integers(-1, 50, n_pts))
    xyz = rng.normal(size=(50, 3))
    rgb = rng.integers(0, 255, (50, 3)).astype(np.uint8)
    return cameras, images, (xyz, rgb, rng.random(50))


@pytest.mark.parametrize("binary", [True, False])
def test_colmap_model_roundtrip(tmp_path, binary):
    cameras, images, points = _toy_model()
    (cl.write_model_binary if binary else cl.write_model_text)(str(tmp_path), cameras, images, points)
    c2, i2, (xyz, rgb, err) = cl.read_model(str(tmp_path))
    assert set(c2) == {1, 2} and c2[2].model == "SIMPLE_RADIAL" and c2[1].focal() == (80.0, 82.0)
    assert np.allclose(c2[2].params, cameras[2].params)
    assert set(i2) == set(images)
    for k, im in images.items():
        assert i2[k].name == im.name and i2[k].camera_id == im.camera_id
        assert np.allclose(i2[k].qvec, im.qvec) and np.allclose(i2[k].tvec, im.tvec)
        assert np.allclose(i2[k].xys, im.xys) and np.array_equal(i2[k].point3D_ids, im.point3D_ids)
        assert np.allclose(i2[k].rotation(), cl.qvec2rotmat(im.qvec))
        assert np.allclose(cl.qvec2rotmat(cl.rotmat2qvec(i2[k].rotation())), i2[k].rotation())
    assert np.allclose(xyz, points[0]) and np.array_equal(rgb, points[1]) and np.allclose(err, points[2])


def test_colmap_gaussian_dataset_splits_and_geometry(tmp_path):
    cameras, images, points = _toy_model()
    cl.write_model_binary(str(tmp_path / "sparse" / "0"), cameras, images, points)
    args = SimpleNamespace(datadir=str(tmp_path), eval=True, white_bkgd=False)
    train = gaussian_dataset_dict["colmap"]("train", 1.0, args)
    test = gaussian_dataset_dict["Colmap"]("test", 1.0, args)
    assert len(test) == 3 and len(train) == 14                 # every 8th of 17 images is held out
    cam = train.cameras[0]
    assert cam.image_name == "img_001.png" and (cam.image_width, cam.image_height) == (32, 24)
    assert abs(cam.FoVx - 2 * math.atan(32 / 80.0)) < 1e-6
    assert abs(float(cam.camera_center.norm()) - 3 * math.sqrt(1 + 0.09)) < 1e-4      # cameras sit on the ring
    assert abs(train.cameras_extent - 1.1 * float(np.linalg.norm(
        np.array([c.camera_center.numpy() for c in train.cameras]) + train.translate, axis=1).max())) < 1e-4
    xyz, rgb = train.initial_point_cloud()
    assert xyz.shape == (50, 3) and rgb.max() <= 1.0
    zj = gaussian_dataset_dict["zhangjiang"]("train", 1.0, SimpleNamespace(datadir=str(tmp_path), eval=False, lb=[-2, -2, -9], ub=[9, 9, 9]))
    assert 0 < len(zj) < 17 and np.allclose(zj.world_shift, -np.array(
        [-(im.rotation().T @ im.tvec) for im in images.values()]).mean(0))


def test_pose_interpolation_and_orientation():
    a = np.concatenate((pu.viewmatrix([0, 1, 0], [0, 0, 1], [0, -3, 0]), [[0, 0, 0, 1]]))
    b = np.concatenate((pu.viewmatrix([-1, 0, 0], [0, 0, 1], [3, 0, 1]), [[0, 0, 0, 1]]))
    path = pu.get_interpolated_poses(a, b, steps=5)
    assert np.allclose(path[0], a[:3]) and np.allclose(path[-1], b[:3], atol=1e-9)
    mid = path[2]
    assert np.allclose(mid[:, 3], [1.5, -1.5, 0.5]) and abs(np.linalg.det(mid[:, :3]) - 1) < 1e-9
    q = pu.quaternion_from_matrix(mid[:, :3])
    assert np.allclose(pu.quaternion_matrix(q), mid[:, :3])
    many, ks = pu.get_interpolated_poses_many([a, b, a], [np.eye(3), 2 * np.eye(3), np.eye(3)], 4)
    assert many.shape == (8, 3, 4) and ks.shape == (8, 3, 3) and np.allclose(ks[3], 2 * np.eye(3))
    fly = pu.catmull_rom_path([a, b, a, b], 1000)
    assert fly.shape == (1000, 3, 4) and np.allclose(fly[0], a[:3]) and np.allclose(fly[-1], b[:3], atol=1e-6)
    assert np.abs(np.diff(fly[:, :, 3], axis=0)).max() < 0.05            # no jumps
    ring = np.stack([pu.viewmatrix(-np.array([math.cos(t), 0.2, math.sin(t)]), [0, 1, 0], 2 * np.array([math.cos(t), 0.2, math.sin(t)]))
                     for t in np.linspace(0, 2 * math.pi, 12, endpoint=False)])
    new, tf = pu.auto_orient_and_center_poses(ring, method="up", center_method="poses")
    assert np.allclose(new[:, :, 3].mean(0), 0, atol=1e-9)
    assert np.allclose(pu.normalize(new[:, :, 1].mean(0)), [0, 0, 1], atol=1e-6)       # mean up is +z now
    focus = pu.focus_of_attention(np.concatenate((ring, np.tile([[[0, 0, 0, 1.0]]], (12, 1, 1))), 1), np.zeros(3))
    assert np.allclose(focus, 0, atol=1e-6)


def test_shard_preprocessing_single_and_distributed(tmp_path):
    n = 3 * 512 + 100
    ds = SimpleNamespace(all_rays=torch.arange(n * 6, dtype=torch.float32).view(n, 6), all_rgbs=torch.rand(n, 3),
                         all_idxs=torch.arange(n, dtype=torch.float32))
    assert preprocess(ds, str(tmp_path / "single"), shard_rays=512) == 3
    loaded = PreprocessedDataset(str(tmp_path / "single"))
    assert len(loaded) == 3 and loaded[0][0].shape == (512, 6)
    # two "ranks" run one after the other in this process (world 1 calls exercise the same numbering logic)
    total = dist_preprocess(ds, str(tmp_path / "dist"), rank=0, world=1, shard_rays=512)
    assert total == 3
    rows = torch.cat([PreprocessedDataset(str(tmp_path / "dist"))[k][2] for k in range(3)])
    assert rows.unique().numel() == 3 * 512                  # no ray is duplicated across shards
    # the loader under data parallelism: the replicas' shards of an epoch are disjoint, batch divided among them
    from landmarksystem_b200.components.data.datasets.dataset_utils import get_preprocessed_loader
    from landmarksystem_b200.utils import Config

    assert preprocess(ds, str(tmp_path / "many"), shard_rays=128) == 12
    seen = []
    for rank in range(2):
        cfg = Config(preprocessed_dir=str(tmp_path / "many"), processed_data_type="file", batch_size=512, DDP=True,
                     model_parallel_and_DDP=False, world_size=2, rank=rank)
        loader = get_preprocessed_loader(cfg)
        assert loader.batch_size == 2                          # 512 rays = 4 shards of 128, two per replica
        seen.append(torch.cat([b[2].reshape(-1) for b in loader]))
    assert seen[0].numel() == seen[1].numel() == 6 * 128
    assert torch.cat(seen).unique().numel() == 12 * 128
    single = get_preprocessed_loader(Config(preprocessed_dir=str(tmp_path / "many"), processed_data_type="file",
                                            batch_size=512, DDP=False))
    assert single.batch_size == 4


def test_drone_metadata_loader(tmp_path):
    import json

    import numpy as np
    from PIL import Image

    from landmarksystem_b200.components.data.datasets.ray_utils import load_drone_meta

    os.makedirs(tmp_path / "images_4" / "flightA", exist_ok=True)
    os.makedirs(tmp_path / "images_4" / "flightB", exist_ok=True)
    frames = []
    for k, sub in enumerate(("flightA", "flightA", "flightB")):
        name = str(tmp_path / "images_4" / sub / f"{k:03d}.png")
        Image.fromarray(np.zeros((6, 8, 3), dtype=np.uint8)).save(name)
        pose = np.eye(4); pose[0, 3] = k
        frames.append({"file_path": name, "transform_matrix": pose.tolist(), "fl_x": 100.0 + k})
    with open(tmp_path / "transforms_train.json", "w", encoding="utf-8") as fh:
        json.dump({"frames": frames}, fh)
    meta = load_drone_meta(str(tmp_path), "train", 4, subfolder=["flightA"])
    assert meta["poses"].shape == (2, 4, 4) and meta["focals"].tolist() == [100.0, 101.0] and meta["hw"] == [6, 8]
    assert meta["imgfolder"].endswith("images_4")
    with open(tmp_path / "transforms_test.json", "w", encoding="utf-8") as fh:
        json.dump({"fl_x": 55.0, "frames": frames}, fh)
    meta = load_drone_meta(str(tmp_path), "test", 4, stride=2)
    assert float(meta["focals"]) == 55.0 and len(meta["fnames"]) == 2


def _path_args(tmp_path, **over):
    base = dict(datadir=str(tmp_path), lb=[-1, -1, -1], ub=[1, 1, 1], train_near_far=[0.1, 5.0], white_bkgd=False,
                camera="normal", render_px=18, render_fov=60.0, render_nframes=12, render_skip=2, render_spherical=True,
                render_spherical_zdiff=0.5, render_spherical_radius=3.0, render_downward=-30.0, render_ncircle=1,
                render_pathid=3, render_near_far=[0.2, 9.0], render_lb=[-2, -2, -2], render_ub=[2, 2, 2])
    base.update(over)
    return SimpleNamespace(**base)


def test_path_split_spherical_and_trajectory(tmp_path):
    """The ``"path"`` split of the ray datasets: a fly-around built from the ``render_*`` fields, or the frames of
    ``trajectories/path{id}.json`` (reference: base_dataset.py:151-214)."""
    import json

    from landmarksystem_b200.components.data.datasets import dataset_dict
    from landmarksystem_b200.components.data.datasets.ray_utils import pose_spherical

    cls = dataset_dict["matrixcity"] if "matrixcity" in dataset_dict else next(iter(dataset_dict.values()))
    ds = cls(split="path", downsample=1.0, is_stack=True, args=_path_args(tmp_path))
    n, H = 12 // 2, 18
    W = int(1920 / 1080 * H)
    assert ds.all_rgbs is None and tuple(ds.img_wh) == (W, H)
    assert ds.all_rays.shape == (n, H * W, 6) and ds.render_poses.shape == (n, 4, 4)
    assert ds.near_far == [0.2, 9.0] and torch.equal(ds.render_scene_bbox, torch.tensor([[-2.0] * 3, [2.0] * 3]))
    assert math.isclose(ds.focal if not isinstance(ds.focal, tuple) else ds.focal[0],
                        0.5 * H / math.tan(math.radians(30.0)), rel_tol=1e-6)
    # frame k: angle 360 k / n, 30 degrees down, radius 3; height drops by zstep * k in the first half, climbs after
    zstep = 0.5 / n * 2
    for k in range(n):
        want = pose_spherical(360.0 * k / n, -30.0, 3.0)
        want[2, 3] -= zstep * k if k < n // 2 else 0.5 - zstep * (k - n // 2)
        assert torch.allclose(ds.render_poses[k], want, atol=1e-6)
    # ray origins are the camera centres; the centre pixel looks at the (height-shifted) origin side of the sphere
    assert torch.allclose(ds.all_rays[0, :, :3], ds.render_poses[0, :3, 3].expand(H * W, 3), atol=1e-6)

    frames = [{"transform_matrix": (torch.eye(4) + 0.01 * k).tolist()} for k in range(7)]
    os.makedirs(tmp_path / "trajectories")
    with open(tmp_path / "trajectories" / "path3.json", "w", encoding="utf-8") as fh:
        json.dump({"frames": frames}, fh)
    ds2 = cls(split="path", downsample=1.0, is_stack=True, args=_path_args(tmp_path, render_spherical=False, render_skip=3))
    assert ds2.render_poses.shape[0] == 3                                  # frames 0, 3, 6
    assert torch.allclose(ds2.render_poses[1], torch.eye(4) + 0.03)


def test_distributed_ray_sampler_is_disjoint_and_reseeds_per_epoch():
    from landmarksystem_b200.components.data.datasets.dataset_utils import DistributedSampler

    world, batch, total = 3, 4, 40
    samplers = [DistributedSampler(total, batch, r, world, seed=5) for r in range(world)]
    seen, first_epoch = [], None
    for step in range(6):                                   # 3 steps fit into 40 ids; the 4th starts a new epoch
        ids = [s.nextids() for s in samplers]
        flat = torch.cat(ids)
        assert all(i.numel() == batch for i in ids) and flat.unique().numel() == world * batch
        seen.append(flat)
        if step == 0:
            first_epoch = samplers[0].ids.clone()
    assert torch.cat(seen[:3]).unique().numel() == 3 * world * batch          # no id twice within an epoch
    assert samplers[0].epoch == 2 and not torch.equal(samplers[0].ids, first_epoch)
    assert all(torch.equal(s.ids, samplers[0].ids) for s in samplers)


def test_camera_reference_field_names():
    """``width / height / FovX / FovY / c2w / device`` as the reference's camera record names them."""
    from landmarksystem_b200.components.data.cameras import Camera
    from landmarksystem_b200.synthetic import ring_cameras

    pose = ring_cameras(4, 3.0)[1].numpy()
    cam = Camera.from_c2w(pose, 32, 24, 30.0)
    want = pose.copy()
    want[:3, 1:3] *= -1                                       # OpenGL -> COLMAP axes
    assert np.allclose(cam.c2w.numpy(), want, atol=1e-6)
    assert (cam.width, cam.height) == (32, 24) and cam.FovX == cam.FoVx and cam.FovY == cam.FoVy
    assert cam.device == torch.device("cpu") and cam.to("cpu").width == 32


def test_ray_and_pose_helpers(tmp_path):
    """Helper functions under the reference's names (dataloader/utils/ray_utils.py, colmap_loader.py)."""
    from landmarksystem_b200.components.data.datasets import ray_utils as ru

    d = ru.get_ray_directions(4, 6, (10.0, 20.0))
    assert d.shape == (4, 6, 3) and torch.allclose(d[1, 2], torch.tensor([(2 - 3) / 10.0, (1 - 2) / 20.0, 1.0]))
    z = torch.tensor([[1.0, 2.0, 4.0]])
    assert torch.allclose(ru.depth2dist(z, torch.tensor([2.0])), torch.tensor([[2.0, 4.0, 2e10]]))
    H, W, ps = 4, 6, 2
    img = torch.arange(H * W * 3, dtype=torch.float32).view(H * W, 3)
    rgb, rays = ru.patchify(img, img + 1000, img + 2000, H, W, ps)
    assert rgb.shape == (6, 4, 3) and rays.shape == (6, 4, 6)
    full = img.view(H, W, 3)
    assert torch.equal(rgb[4].view(ps, ps, 3), full[2:4, 2:4])            # patch (row 1, column 1)
    assert torch.equal(rays[4, :, :3], rgb[4] + 1000) and torch.equal(rays[4, :, 3:], rgb[4] + 2000)
    assert ru.listify_matrix(np.eye(2)) == [[1.0, 0.0], [0.0, 1.0]]

    rng = np.random.default_rng(0)
    poses = np.tile(np.eye(4)[:3], (30, 1, 1))
    poses[:, :3, 3] = rng.normal(size=(30, 3)) * np.array([0.5, 5.0, 2.0]) + np.array([10.0, -3.0, 2.0])
    out, T = ru.transform_poses_pca(poses)
    c = out[:, :3, 3]
    assert np.isclose(np.abs(c).max(), 1.0) and np.allclose(c.mean(0), 0, atol=1e-9)
    assert c.std(0)[0] > c.std(0)[1] > c.std(0)[2]                          # principal axes, largest spread first
    assert np.allclose(ru.unpad_poses(T @ ru.pad_poses(poses))[:, :3, 3], c)
    assert out.mean(axis=0)[2, 1] >= 0 and ru.pad_poses(out).shape == (30, 4, 4)

    depth = rng.random((5, 7)).astype(np.float32)
    cl.write_colmap_bin_array(str(tmp_path / "depth.bin"), depth)
    assert np.array_equal(cl.read_colmap_bin_array(str(tmp_path / "depth.bin")), depth)
    assert cl.read_extrinsics_binary is cl.read_images_binary and cl.read_intrinsics_text is cl.read_cameras_text


def test_lens_ordering_and_rotation_helpers():
    torch.manual_seed(0)
    assert np.allclose(pu.unit_vector([3.0, 4.0]), [0.6, 0.8])
    assert np.allclose(np.linalg.norm(pu.unit_vector(np.ones((4, 3)), axis=1), axis=1), 1.0)
    v, n = pu.normalize_with_norm(torch.tensor([[3.0, 4.0], [0.0, 0.0]]), dim=-1)
    assert torch.allclose(v[0], torch.tensor([0.6, 0.8])) and float(n[0]) == 5.0 and torch.isfinite(v).all()
    # greedy nearest-neighbour tour along a line visited out of order
    xs = [0.0, 5.0, 1.0, 4.0, 2.0]
    poses = torch.eye(4).repeat(5, 1, 1)
    poses[:, 0, 3] = torch.tensor(xs)
    Ks = torch.arange(5, dtype=torch.float32)[:, None, None] * torch.ones(5, 3, 3)
    op, ok = pu.get_ordered_poses_and_k(poses, Ks)
    assert op[:, 0, 3].tolist() == [0.0, 1.0, 2.0, 4.0, 5.0] and ok[:, 0, 0].tolist() == [0.0, 2.0, 4.0, 3.0, 1.0]
    # undistort inverts the lens model
    params = pu.get_distortion_params(k1=0.1, k2=-0.02, k3=0.003, p1=0.004, p2=-0.003)
    pts = torch.rand(200, 2) * 1.2 - 0.6
    back = pu.radial_and_tangential_undistort(pu.radial_and_tangential_distort(pts, params), params)
    assert torch.allclose(back, pts, atol=1e-5)
    for a, b in ((torch.tensor([1.0, 2.0, 3.0]), torch.tensor([-2.0, 0.5, 1.0])),
                 (torch.tensor([0.0, 0.0, 2.0]), torch.tensor([0.0, 0.0, -1.0]))):
        R = pu.rotation_matrix(a, b)
        assert torch.allclose(R @ (a / a.norm()), b / b.norm(), atol=1e-6)
        assert torch.allclose(R @ R.T, torch.eye(3), atol=1e-6) and abs(float(torch.linalg.det(R)) - 1.0) < 1e-5


def test_dataset_shard_methods_and_merge_type_check(tmp_path):
    from landmarksystem_b200.components.data.datasets import dataset_dict
    from landmarksystem_b200.render.types import MergeType

    assert MergeType.check("Unevenly") and not MergeType.check("Sometimes")
    args = SimpleNamespace(datadir="ring:4:16x16:18:3", lb=[-1, -1, -1], ub=[1, 1, 1], white_bkgd=False,
                           preprocessed_dir=str(tmp_path / "shards"))
    ds = dataset_dict["synthetic"](split="train", downsample=1.0, is_stack=True, args=args)
    assert ds.preprocess(args, batch_size=256) == 4                       # 4 images x 256 rays
    assert PreprocessedDataset(args.preprocessed_dir)[3][1].shape == (256, 3)
    assert ds.distpreprocess(root=str(tmp_path / "dist"), batch_size=512) == 2


def test_camera_dataset_reads_three_intrinsics_layouts(tmp_path):
    """``transforms_*.json`` with one focal length, one field of view, or focal length and size per frame."""
    import json

    from PIL import Image

    pose = np.eye(4).tolist()
    os.makedirs(tmp_path / "images")
    for k, (w, h) in enumerate(((40, 30), (20, 10))):
        Image.fromarray(np.zeros((h, w, 3), np.uint8)).save(tmp_path / "images" / f"image_{k}.png")
    frames = [{"file_path": f"./images/image_{k}.png", "transform_matrix": pose} for k in range(2)]
    args = SimpleNamespace(datadir=str(tmp_path), white_bkgd=False)

    def load(meta):
        with open(tmp_path / "transforms_train.json", "w", encoding="utf-8") as fh:
            json.dump(meta, fh)
        return gaussian_dataset_dict["city"]("train", 1.0, args).cameras

    cams = load({"fl_x": 50.0, "fl_y": 60.0, "w": 40, "h": 30, "frames": frames})
    assert all((c.image_width, c.image_height) == (40, 30) for c in cams)
    assert math.isclose(cams[0].FoVx, 2 * math.atan(40 / 100.0)) and math.isclose(cams[0].FoVy, 2 * math.atan(30 / 120.0))
    cams = load({"camera_angle_x": 0.8, "frames": frames})              # size from the first image
    assert (cams[1].image_width, cams[1].image_height) == (40, 30) and math.isclose(cams[0].FoVx, 0.8, rel_tol=1e-6)
    multi = [dict(f, fl_x=25.0 * (k + 1), fl_y=25.0 * (k + 1), w=w, h=h) for k, (f, (w, h)) in
             enumerate(zip(frames, ((40, 30), (20, 10))))]
    cams = load({"camera_model": "SIMPLE_PINHOLE", "frames": multi})
    assert (cams[1].image_width, cams[1].image_height) == (20, 10)
    assert math.isclose(cams[0].FoVx, 2 * math.atan(40 / 50.0)) and math.isclose(cams[1].FoVx, 2 * math.atan(20 / 100.0))


def test_ray_dataset_with_one_focal_length_per_frame(tmp_path):
    import json

    from PIL import Image

    from landmarksystem_b200.components.data.datasets import dataset_dict
    from landmarksystem_b200.components.data.datasets.ray_utils import get_ray_directions_blender

    os.makedirs(tmp_path / "images")
    frames = []
    for k, fl in enumerate((30.0, 45.0, 60.0)):
        Image.fromarray(np.full((6, 8, 3), 40 * k, np.uint8)).save(tmp_path / "images" / f"image_{k}.png")
        frames.append({"fl_x": fl, "fl_y": fl, "w": 8, "h": 6, "file_path": f"./images/image_{k}.png",
                       "transform_matrix": np.eye(4).tolist()})
    with open(tmp_path / "transforms_train.json", "w", encoding="utf-8") as fh:
        json.dump({"camera_model": "SIMPLE_PINHOLE", "frames": frames}, fh)
    args = SimpleNamespace(datadir=str(tmp_path), lb=[-1, -1, -1], ub=[1, 1, 1], white_bkgd=False, camera="normal")
    ds = dataset_dict["matrixcity"](split="train", downsample=1.0, is_stack=True, args=args)
    assert ds.all_rays.shape == (3, 48, 6) and tuple(ds.img_wh) == (8, 6)
    for k, fl in enumerate((30.0, 45.0, 60.0)):                         # identity pose: ray directions = camera directions
        assert torch.allclose(ds.all_rays[k, :, 3:], get_ray_directions_blender(6, 8, fl).reshape(-1, 3))
    assert torch.allclose(ds.all_rgbs[2], torch.full((48, 3), 80 / 255.0))


def test_colmap_to_transforms_conversion(tmp_path):
    """A sparse model converted to the transforms layout gives the cameras the COLMAP dataset itself gives."""
    import json

    from PIL import Image

    from landmarksystem_b200.components.data.datasets.colmap2nerf import convert, main

    cameras, images, points = _toy_model()
    cl.write_model_binary(str(tmp_path / "sparse" / "0"), cameras, images, points)
    os.makedirs(tmp_path / "images")
    for im in images.values():
        cam = cameras[im.camera_id]
        Image.fromarray(np.zeros((cam.height, cam.width, 3), np.uint8)).save(tmp_path / "images" / im.name)
    n_train, n_test = convert(str(tmp_path / "sparse" / "0"), str(tmp_path), holdout=8)
    assert (n_train, n_test) == (14, 3)
    with open(tmp_path / "transforms_train.json", encoding="utf-8") as fh:
        meta = json.load(fh)
    assert "fl_x" not in meta and meta["frames"][0]["file_path"] == "./images/img_001.png"      # two cameras: per frame
    args = SimpleNamespace(datadir=str(tmp_path), eval=True, white_bkgd=False)
    direct = gaussian_dataset_dict["colmap"]("train", 1.0, args).cameras
    via_json = gaussian_dataset_dict["city"]("train", 1.0, args).cameras
    assert len(direct) == len(via_json) == 14
    for a, b in zip(direct, via_json):
        assert a.image_name == b.image_name and (a.image_width, a.image_height) == (b.image_width, b.image_height)
        assert torch.allclose(a.camera_center, b.camera_center, atol=1e-4)
        assert torch.allclose(a.world_view_transform, b.world_view_transform, atol=1e-4)
        assert abs(a.FoVx - b.FoVx) < 1e-6 and abs(a.FoVy - b.FoVy) < 1e-6
    # one shared camera -> one focal length for the file; the command-line entry point writes the same files
    single = {k: cl.ColmapImage(v.id, v.qvec, v.tvec, 1, v.name, v.xys, v.point3D_ids) for k, v in images.items()}
    cl.write_model_text(str(tmp_path / "one"), {1: cameras[1]}, single, points)
    main(["--recon_dir", str(tmp_path / "one"), "--output_dir", str(tmp_path / "one_out"), "--holdout", "0"])
    with open(tmp_path / "one_out" / "transforms_train.json", encoding="utf-8") as fh:
        meta = json.load(fh)
    assert meta["fl_x"] == 80.0 and meta["fl_y"] == 82.0 and (meta["w"], meta["h"]) == (64, 48) and len(meta["frames"]) == 17


def test_initial_cloud_from_the_sparse_reconstruction(tmp_path):
    """COLMAP datasets seed the Gaussians with their SfM points (reference: ply_utils.py:116-144 picks
    ``init_type="colmap"`` for ``dataset_name="Colmap"``); both calling conventions of the helpers."""
    from landmarksystem_b200.components.utils.ply_utils import get_pcd, init_ply

    cameras, images, points = _toy_model()
    cl.write_model_binary(str(tmp_path / "sparse" / "0"), cameras, images, points)
    args = SimpleNamespace(datadir=str(tmp_path), eval=True, white_bkgd=False, dataset_name="Colmap", point_path=None,
                           init_points_num=77, max_init_points=-1, random_seed=0)
    train = gaussian_dataset_dict["Colmap"]("train", 1.0, args)
    aabb = [[-1.0, -1.0, 0.0], [1.0, 1.0, 1.0]]
    pcd = get_pcd(args, aabb, dataset=train)
    assert pcd.points.shape == (50, 3) and np.allclose(pcd.points, train.initial_point_cloud()[0])
    assert get_pcd(args, aabb).points.shape == (77, 3)                      # no dataset: the random ground-plane cloud
    capped = get_pcd(SimpleNamespace(**dict(vars(args), max_init_points=20)), aabb, dataset=train)
    assert capped.points.shape == (20, 3)

    cloud = init_ply(str(tmp_path), aabb, "colmap", 10)                      # the reference's positional form
    assert cloud.points.shape == (50, 3) and np.allclose(np.sort(cloud.points, 0), np.sort(points[0].astype(np.float32), 0))
    assert os.path.exists(tmp_path / "sparse" / "0" / "points3D.ply")
    flat = init_ply(str(tmp_path), aabb, "ply", 31)
    assert flat.points.shape == (31, 3) and np.allclose(flat.points[:, 2], 0.0)
    assert init_ply(str(tmp_path), aabb, 12).endswith("points3d_init.ply")  # this package's form returns the path
    via_reference = get_pcd(None, args, aabb, str(tmp_path), None)           # (loaded_iter, config, aabb, logfolder, model)
    assert via_reference.points.shape == (50, 3)


def test_get_rays_in_the_reference_form():
    from landmarksystem_b200.components.data.datasets import ray_utils as ru

    H, W, f = 6, 8, 12.0
    K = torch.tensor([[f, 0, W / 2], [0, f, H / 2], [0, 0, 1.0]])
    pose = ru.pose_spherical(40.0, -30.0, 3.0, zval=1.25)
    assert float(pose[2, 3]) == 1.25
    o, d = ru.get_rays(H, W, K, pose)                                 # reference: (H, W, K, c2w)
    assert o.shape == (H * W, 3) and torch.allclose(d.norm(dim=-1), torch.ones(H * W), atol=1e-6)
    dirs = ru.get_ray_directions_blender(H, W, f) - torch.tensor([0.5 / f, -0.5 / f, 0.0])      # integer pixel coordinates
    o2, d2 = ru.get_rays(dirs, pose)                                  # this package: (directions, c2w)
    assert torch.allclose(o, o2) and torch.allclose(d, d2 / d2.norm(dim=-1, keepdim=True), atol=1e-6)
    po, pd = ru.get_rays(H, W, K, pose, "panorama")
    qo, qd = ru.get_rays(dirs, pose, "panorama")
    assert torch.allclose(pd, qd / qd.norm(dim=-1, keepdim=True), atol=1e-5)


def test_interpolation_through_ordered_key_poses_and_args_style_distributed_init(monkeypatch):
    poses = [np.eye(4)[:3] for _ in range(4)]
    for k, x in enumerate((0.0, 3.0, 1.0, 2.0)):
        poses[k] = poses[k].copy()
        poses[k][0, 3] = x
    plain, _ = pu.get_interpolated_poses_many(poses, None, steps_per_transition=2)
    tour, _ = pu.get_interpolated_poses_many(poses, None, steps_per_transition=2, order_poses=True)
    assert plain.shape == tour.shape == (6, 3, 4)
    assert np.all(np.diff(tour[:, 0, 3]) >= -1e-9) and not np.all(np.diff(plain[:, 0, 3]) >= 0)   # the tour never turns back

    from landmarksystem_b200.train.utils import init_distributed_mode

    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(name, raising=False)
    args = SimpleNamespace(env="single_node")
    info = init_distributed_mode(args)                       # the reference passes its configuration object
    assert info == {"rank": 0, "world_size": 1, "local_rank": 0}
    assert (args.rank, args.world_size, args.local_rank, args.distributed) == (0, 1, 0, False)


def test_resolution_field_scales_the_cameras(tmp_path):
    """``resolution``: ``-1`` keeps the size, ``1 / 2 / 4 / 8`` divide it, another number is the target width
    (reference: base_dataset.py:344-358); the field of view does not change, the loaded image follows the camera."""
    from PIL import Image

    cameras, images, points = _toy_model()
    cl.write_model_binary(str(tmp_path / "sparse" / "0"), cameras, images, points)
    os.makedirs(tmp_path / "images")
    for im in images.values():
        cam = cameras[im.camera_id]
        Image.fromarray(np.zeros((cam.height, cam.width, 3), np.uint8)).save(tmp_path / "images" / im.name)

    def first(resolution):
        args = SimpleNamespace(datadir=str(tmp_path), eval=True, white_bkgd=False, resolution=resolution)
        return gaussian_dataset_dict["colmap"]("train", 1.0, args)

    full, half, width16 = first(-1), first(2), first(16)
    a, b, c = full.cameras[0], half.cameras[0], width16.cameras[0]                 # camera 2 of the toy model: 32 x 24
    assert (a.image_width, a.image_height) == (32, 24) and (b.image_width, b.image_height) == (16, 12)
    assert (c.image_width, c.image_height) == (16, 12)
    assert abs(a.FoVx - b.FoVx) < 1e-6 and abs(a.FoVy - c.FoVy) < 1e-6
    assert half.load_image(b).shape == (3, 12, 16)


def test_multi_scale_items_of_the_camera_dataset(tmp_path):
    """``resolution_scales=[1, 2]``: twice as many items; odd items are the same views at half size with
    ``resolution_scale`` set and an image of that size (reference: base_dataset.py:314-331)."""
    from landmarksystem_b200.components.data.datasets import gaussian_dataset_dict as table

    args = SimpleNamespace(datadir="ring:3:16x12:14:3", lb=[-1, -1, -1], ub=[1, 1, 1], white_bkgd=False,
                           resolution_scales=[1.0, 2.0])
    ds = table["synthetic"]("train", 1.0, args)
    assert len(ds) == 2 * len(ds.cameras) == 6
    cam0, img0 = ds[2]
    cam1, img1 = ds[3]
    assert cam0.uid == cam1.uid and cam0.resolution_scale == 1.0 and cam1.resolution_scale == 2.0
    assert (cam1.image_width, cam1.image_height) == (cam0.image_width // 2, cam0.image_height // 2)
    assert img1.shape[-2:] == (cam1.image_height, cam1.image_width) and img0.shape[-2:] == (cam0.image_height, cam0.image_width)
    assert abs(cam0.FoVx - cam1.FoVx) < 1e-9 and torch.equal(cam0.full_proj_transform, cam1.full_proj_transform)
    assert abs(float(img0.mean()) - float(img1.mean())) < 0.05
