"""MatrixCity block A configurations of Scaffold-GS (variant set of the reference's benchmarks/nerf/scaffold_gs/confs/*.py).
Dataset root: ``LMB_MATRIXCITY_ROOT``; the initial point cloud of the anchor-based models defaults to the trained
vanilla-3DGS ``point_cloud.ply`` under ``./log`` and can be moved with ``LMB_INIT_POINT_CLOUD``."""
import os

from landmarksystem_b200.configs import DatasetConfig, RenderConfig, TrainConfig
from landmarksystem_b200.models.scaffold_gs.gs_model import ScaffoldGSConfig

DATA_ROOT = os.environ.get("LMB_MATRIXCITY_ROOT", "./data/MatrixCity/small_city/aerial/pose/block_A")
INIT_PLY = os.environ.get("LMB_INIT_POINT_CLOUD",
                          "./log/Gaussian3D_matrix_city_blockA/point_cloud/iteration_30000/point_cloud.ply")
LB = [-1.0378e01, -7.4430e00, -1.1921e-07]
UB = [1.2078e00, 2.4078e00, 9.0000e-01]


def _dataset(downsample):
    return DatasetConfig(datadir=DATA_ROOT, downsample_train=downsample, dataset_type="gaussian", dataset_name="city",
                         preload=True, lb=list(LB), ub=list(UB))

def train(ci: bool = False):
    train_config = TrainConfig(model_name="ScaffoldGS", expname="ScaffoldGS_matrix_city_blockA", basedir="./log", batch_size=1,
                               n_iters=30000, test_iterations=[7000, 30000], save_iterations=[7000, 30000], tensorboard=True)
    if ci:
        train_config.basedir, train_config.test_iterations, train_config.save_iterations = "./log_for_ci_test", [30000], []
    model_config = ScaffoldGSConfig(white_bkgd=False, resolution=1, resolution_scales=[1.0], point_path=INIT_PLY)
    return [train_config, _dataset(10), model_config]


def render():
    train_config, dataset_config, model_config = train()
    render_config = RenderConfig(ckpt="log/ScaffoldGS_matrix_city_blockA/point_cloud/iteration_30000/point_cloud.ply",
                                 ckpt_type="full", batch_size=1, N_vis=20).from_train_config(train_config)
    return [render_config, dataset_config, model_config]
