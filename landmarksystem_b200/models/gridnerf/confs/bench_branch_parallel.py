"""Large-scene GridNeRF benchmark configuration: one 1 km x 1 km x 300 m spatial block per GPU with
4096^2 planes and 512-entry lines, 16 density + 48 appearance channels in bf16 (fp32 masters),
8192 rays per GPU and 128 samples per ray.  ``plane_division`` / ``lb`` / ``ub`` / ``init_grid_size``
are rewritten by ``bench.py`` for the number of GPUs in use ([1,1], [2,1], [2,2], [2,4])."""
from landmarksystem_b200.configs import DatasetConfig, TrainConfig
from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRFConfig

train_config = TrainConfig(
    model_name="GridNeRF",
    expname="gridnerf_bench",
    basedir="./log_bench",
    n_iters=1000000,
    batch_size=8192,
    progress_refresh_rate=1000000,
    vis_every=100000000,
    N_vis=0,
    random_seed=0,
    print_timestamp=False,
    cuda_graph=True,         # single-GPU runs replay the whole step from one CUDA graph
)

dataset_config = DatasetConfig(
    dataset_name="synthetic",
    datadir="aerial:2:8x8:8:400",   # placeholder rig; the benchmark feeds its own ray pool
    lb=[0.0, 0.0, 0.0],
    ub=[1000.0, 1000.0, 300.0],
)

model_config = GridNeRFConfig(
    resMode=[1],
    n_lamb_sigma=[16],
    n_lamb_sh=[48],
    nonlinear_density=True,
    view_pe=2,
    fea_pe=2,
    featureC=128,
    init_grid_size=[4096, 4096, 512],
    upsamp_list=[],
    update_AlphaMask_list=[],
    nSamples=128,
    step_ratio=10.0,
    train_near_far=[10.0, 2000.0],
    lr_init=0.02,
    lr_basis=1e-3,
    distance_scale=25,
    grid_dtype="bf16",
    fused_mlp_train=True,    # colour head forward AND backward run as tcgen05 kernels
    lazy_adam=True,          # exact deferred Adam: only texels the step touched are visited
    runtime="Kernel",
    appearance_embedding_size=8,
)

config = [train_config, dataset_config, model_config]
