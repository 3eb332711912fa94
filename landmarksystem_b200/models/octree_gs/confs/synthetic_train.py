"""Octree-GS on the analytic blob scene (progressive coarse-to-fine levels)."""
from landmarksystem_b200.configs import DatasetConfig, TrainConfig
from landmarksystem_b200.models.octree_gs.gs_model import OctreeGSConfig

train_config = TrainConfig(model_name="OctreeGS", expname="octree_synthetic", basedir="./log", n_iters=600,
                           batch_size=1, progress_refresh_rate=100, random_seed=0, print_timestamp=False)
dataset_config = DatasetConfig(dataset_name="synthetic", dataset_type="gaussian", datadir="ring:16:96x96:110:3",
                               lb=[-1.0, -1.0, -1.0], ub=[1.0, 1.0, 1.0], preload=True)
model_config = OctreeGSConfig(n_offsets=5, appearance_dim=0, init_points_num=4000, init_points_volume=True,
                              base_layer=4, levels=3, progressive=True, coarse_iter=200, start_stat=50,
                              update_from=150, update_interval=100, update_until=500, visible_threshold=0.0)
config = [train_config, dataset_config, model_config]
