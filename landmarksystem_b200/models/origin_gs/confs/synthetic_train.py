"""Vanilla 3DGS on the analytic blob scene (16 ring cameras, 96x96 px)."""
from landmarksystem_b200.configs import DatasetConfig, TrainConfig
from landmarksystem_b200.models.origin_gs.gs_model import Gaussian3DConfig

train_config = TrainConfig(model_name="GaussianModel", expname="gs_synthetic", basedir="./log", n_iters=600,
                           batch_size=1, progress_refresh_rate=100, random_seed=0, test_iterations=[],
                           save_iterations=[], print_timestamp=False)
dataset_config = DatasetConfig(dataset_name="synthetic", dataset_type="gaussian", datadir="ring:16:96x96:110:3",
                               lb=[-1.0, -1.0, -1.0], ub=[1.0, 1.0, 1.0], preload=True)
model_config = Gaussian3DConfig(sh_degree=3, init_points_num=4000, init_points_volume=True, densify_from_iter=100,
                                densify_until_iter=500, densification_interval=100, opacity_reset_interval=300,
                                position_lr_max_steps=600)
config = [train_config, dataset_config, model_config]
