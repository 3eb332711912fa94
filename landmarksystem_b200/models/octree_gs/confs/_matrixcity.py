"""MatrixCity block A configurations of Octree-GS (variant set of the reference's benchmarks/nerf/octree_gs/confs/*.py).
Dataset root: ``LMB_MATRIXCITY_ROOT``; the initial point cloud of the anchor-based models defaults to the trained
vanilla-3DGS ``point_cloud.ply`` under ``./log`` and can be moved with ``LMB_INIT_POINT_CLOUD``."""
import os

from landmarksystem_b200.configs import DatasetConfig, RenderConfig, TrainConfig
from landmarksystem_b200.models.octree_gs.gs_model import OctreeGSConfig

DATA_ROOT = os.environ.get("LMB_MATRIXCITY_ROOT", "./data/MatrixCity/small_city/aerial/pose/block_A")
INIT_PLY = os.environ.get("LMB_INIT_POINT_CLOUD",
                          "./log/Gaussian3D_matrix_city_blockA/point_cloud/iteration_30000/point_cloud.ply")
LB = [-1.0378e01, -7.4430e00, -1.1921e-07]
UB = [1.2078e00, 2.4078e00, 9.0000e-01]


def _dataset(downsample):
    return DatasetConfig(datadir=DATA_ROOT, downsample_train=downsample, dataset_type="gaussian", dataset_name="city",
                         preload=True, lb=list(LB), ub=list(UB))

def train(ci: bool = False):
    marks = [10000, 20000, 30000, 40000]
    train_config = TrainConfig(model_name="OctreeGS", expname="OctreeGS_matrix_city_blockA", basedir="./log", batch_size=1,
                               n_iters=40000, test_iterations=marks, save_iterations=marks, tensorboard=True)
    if ci:
        train_config.basedir, train_config.test_iterations, train_config.save_iterations = "./log_for_ci_test", [40000], []
    model_config = OctreeGSConfig(appearance_dim=0, fork=2, base_layer=-1, visible_threshold=0.9, dist2level="round",
                                  update_ratio=0.2, progressive=True, dist_ratio=0.999, levels=-1, init_level=-1, extra_ratio=0.5,
                                  extra_up=0.01, white_bkgd=False, resolution=1, resolution_scales=[1.0], point_path=INIT_PLY)
    return [train_config, _dataset(1), model_config]


def render():
    train_config, dataset_config, model_config = train()
    render_config = RenderConfig(ckpt="log/OctreeGS_matrix_city_blockA/point_cloud/iteration_40000/point_cloud.ply",
                                 ckpt_type="full", batch_size=1, N_vis=20).from_train_config(train_config)
    model_config.enable_lod = True
    return [render_config, dataset_config, model_config]
