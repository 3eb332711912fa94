"""Nerfacto on the tiny analytic blob scene."""
from landmarksystem_b200.configs import DatasetConfig, TrainConfig
from landmarksystem_b200.models.nerfacto.nerfacto import NerfactoConfig

train_config = TrainConfig(model_name="Nerfacto", expname="nerfacto_synthetic_tiny", basedir="./log", n_iters=300,
                           batch_size=1024, progress_refresh_rate=50, vis_every=100000, N_vis=2, random_seed=0,
                           print_timestamp=False)
dataset_config = DatasetConfig(dataset_name="synthetic", datadir="ring:8:64x64:80:3", lb=[-1.0, -1.0, -1.0],
                               ub=[1.0, 1.0, 1.0])
model_config = NerfactoConfig(num_levels=8, base_res=8, max_res=128, log2_hashmap_size=15,
                              num_proposal_samples_per_ray=(64, 32), num_nerf_samples_per_ray=24,
                              proposal_net_args_list=[{"hidden_dim": 16, "log2_hashmap_size": 13, "num_levels": 4, "max_res": 32},
                                                      {"hidden_dim": 16, "log2_hashmap_size": 13, "num_levels": 4, "max_res": 64}],
                              train_near_far=[1.2, 4.8], appearance_embedding_size=8, lr_decay_max_steps=300,
                              disable_scene_contraction=True, background_color="black", proposal_warmup=100,
                              proposal_weights_anneal_max_num_iters=100, runtime="Torch")
config = [train_config, dataset_config, model_config]
