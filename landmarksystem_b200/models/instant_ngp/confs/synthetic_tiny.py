"""InstantNGP on the tiny analytic blob scene."""
from landmarksystem_b200.configs import DatasetConfig, TrainConfig
from landmarksystem_b200.models.instant_ngp.instant_ngp import InstantNGPConfig

train_config = TrainConfig(model_name="InstantNGP", expname="ngp_synthetic_tiny", basedir="./log", n_iters=300,
                           batch_size=1024, progress_refresh_rate=50, vis_every=100000, N_vis=2, random_seed=0,
                           print_timestamp=False)
dataset_config = DatasetConfig(dataset_name="synthetic", datadir="ring:8:64x64:80:3", lb=[-1.0, -1.0, -1.0],
                               ub=[1.0, 1.0, 1.0])
model_config = InstantNGPConfig(num_levels=8, base_res=8, max_res=128, log2_hashmap_size=15, grid_resolution=32,
                                grid_levels=1, train_near_far=[1.2, 4.8], appearance_embedding_size=8,
                                render_step_size=0.02, cone_angle=0.0, max_samples_per_ray=160, lr_decay_max_steps=300,
                                background_color="black", runtime="Torch")
config = [train_config, dataset_config, model_config]
