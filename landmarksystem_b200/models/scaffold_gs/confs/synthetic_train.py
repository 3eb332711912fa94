"""Scaffold-GS on the analytic blob scene."""
from landmarksystem_b200.configs import DatasetConfig, TrainConfig
from landmarksystem_b200.models.scaffold_gs.gs_model import ScaffoldGSConfig

train_config = TrainConfig(model_name="ScaffoldGS", expname="scaffold_synthetic", basedir="./log", n_iters=600,
                           batch_size=1, progress_refresh_rate=100, random_seed=0, print_timestamp=False)
dataset_config = DatasetConfig(dataset_name="synthetic", dataset_type="gaussian", datadir="ring:16:96x96:110:3",
                               lb=[-1.0, -1.0, -1.0], ub=[1.0, 1.0, 1.0], preload=True)
model_config = ScaffoldGSConfig(voxel_size=0.08, n_offsets=5, init_points_num=4000, init_points_volume=True,
                                start_stat=50, update_from=150, update_interval=100, update_until=500,
                                position_lr_max_steps=600, offset_lr_max_steps=600, mlp_opacity_lr_max_steps=600,
                                mlp_cov_lr_max_steps=600, mlp_color_lr_max_steps=600)
config = [train_config, dataset_config, model_config]
