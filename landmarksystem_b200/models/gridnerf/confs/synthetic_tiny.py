"""GridNeRF on the tiny analytic blob scene: 8 ring cameras of 64x64 px, 128^2 planes / 128 lines,
16 density + 48 appearance channels, 1024-ray batches, 64 samples per ray."""
from landmarksystem_b200.configs import DatasetConfig, TrainConfig
from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRFConfig

train_config = TrainConfig(
    model_name="GridNeRF",
    expname="gridnerf_synthetic_tiny",
    basedir="./log",
    n_iters=200,
    batch_size=1024,
    progress_refresh_rate=20,
    vis_every=100000,
    N_vis=2,
    random_seed=0,
)

dataset_config = DatasetConfig(
    dataset_name="synthetic",
    datadir="ring:8:64x64:80:3",
    lb=[-1.0, -1.0, -1.0],
    ub=[1.0, 1.0, 1.0],
)

model_config = GridNeRFConfig(
    resMode=[1],
    n_lamb_sigma=[16],
    n_lamb_sh=[48],
    nonlinear_density=True,
    view_pe=2,
    fea_pe=2,
    featureC=128,
    N_voxel_init=128 ** 3,
    N_voxel_final=128 ** 3,
    upsamp_list=[],
    update_AlphaMask_list=[],
    nSamples=64,
    step_ratio=2.0,
    train_near_far=[1.5, 4.5],
    lr_init=0.02,
    lr_basis=1e-3,
    distance_scale=25,
    appearance_embedding_size=8,
)

config = [train_config, dataset_config, model_config]
