"""MatrixCity small-city block A configurations of GridNeRF, built from one table.

Every ``matrixcity_2block_*.py`` file beside this module is two lines that call :func:`train` or
:func:`render` with the variant name; the variants and their switches follow the reference's shipped
configuration set (benchmarks/nerf/gridnerf/confs/*.py): single process, ``DDP``, branch parallel
(``plane_division`` [2,2] / [2,1] / [10,5]), channel parallel (x2), and the render variants that load a
merged checkpoint with a different parallel layout than it was trained with.

The dataset root defaults to ``./data/MatrixCity/small_city/aerial/pose/block_A`` and can be moved with the
``LMB_MATRIXCITY_ROOT`` environment variable; checkpoints are looked up under ``./log/<expname>/``.
"""
import os

from landmarksystem_b200.configs import DatasetConfig, RenderConfig, TrainConfig
from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRFConfig

DATA_ROOT = os.environ.get("LMB_MATRIXCITY_ROOT", "./data/MatrixCity/small_city/aerial/pose/block_A")
LB = [-1.0378e01, -7.4430e00, -1.1921e-07]
UB = [1.2078e00, 2.4078e00, 9.0000e-01]

# quality tiers: iterations, resolution levels, schedule
_TIER = {
    "lowquality": dict(n_iters=8000, vis_every=5000, resMode=[1], add_nerf=5000, lr_decay_iters=8000,
                       upsamp_list=[2000, 3000, 4000, 5500, 7000], update_AlphaMask_list=[2000, 4000, 8000, 10000]),
    "multi": dict(n_iters=50000, vis_every=5000, resMode=[1, 2, 4], add_nerf=40000, lr_decay_iters=50000,
                  upsamp_list=[2000, 3000, 4000, 5500, 7000], update_AlphaMask_list=[2000, 4000, 8000, 10000]),
    "multi_ddp": dict(n_iters=25000, vis_every=2500, resMode=[1, 2, 4], add_nerf=20000, lr_decay_iters=25000,
                      upsamp_list=[1000, 1500, 2000, 2250, 3500], update_AlphaMask_list=[1000, 2000, 4000, 5000]),
}

# variant -> (tier, expname, train-config switches, upper-bound scale of the scene box)
_TRAIN = {
    "lowquality": ("lowquality", "matrix_city_blockA_lowquality", {}, None),
    "lowquality_ddp_train": ("lowquality", "gridnerf_matrix_city_blockA_lowquality_ddp_train", {"DDP": True}, None),
    "lowquality_BranchParallel": ("lowquality", "matrix_city_blockA_lowquality_BranchParallel",
                                  {"branch_parallel": True, "plane_division": [2, 2]}, None),
    "lowquality_ChannelParallel": ("lowquality", "matrix_city_blockA_lowquality_ChannelParallel",
                                   {"channel_parallel": True, "channel_parallel_size": 2}, None),
    "multi": ("multi", "matrix_city_blockA_multi", {}, None),
    "multi_ddp": ("multi_ddp", "matrix_city_blockA_multi_ddp", {}, None),
    "multi_BranchParallel": ("multi", "matrix_city_blockA_multi_BranchParallel",
                             {"branch_parallel": True, "plane_division": [2, 1]}, None),
    "multi_BranchParallel_10x5": ("multi", "matrix_city_blockA_multi_BranchParallel",
                                  {"branch_parallel": True, "plane_division": [10, 5]}, 5),
    "multi_ChannelParallel": ("multi", "matrix_city_blockA_multi_ChannelParallel",
                              {"channel_parallel": True, "channel_parallel_size": 2}, None),
    "single_train_ci": ("lowquality", "matrix_city_blockA_lowquality", {"basedir": "./log_for_ci_test", "N_vis": 0}, None),
}


def train(variant: str):
    tier_name, expname, switches, scale = _TRAIN[variant]
    tier = _TIER[tier_name]
    ub = list(UB)
    if scale:                                   # the 50-block stress scene: footprint enlarged `scale` times in x and y
        ub[0] = UB[0] + (scale - 1) * (UB[0] - LB[0])
        ub[1] = UB[1] + (scale - 1) * (UB[1] - LB[1])
    train_config = TrainConfig(model_name="GridNeRF", expname=expname, basedir="./log", batch_size=8192, debug=False,
                               vis_every=tier["vis_every"], n_iters=tier["n_iters"], N_vis=5)
    for key, value in switches.items():
        setattr(train_config, key, value)
    dataset_config = DatasetConfig(dataset_name="matrixcity", datadir=DATA_ROOT, downsample_train=1, lb=list(LB), ub=ub)
    model_config = GridNeRFConfig(
        ndims=1, resMode=tier["resMode"], encode_app=False, nonlinear_density=True, add_nerf=tier["add_nerf"],
        train_near_far=[0.6, 3.5], N_voxel_init=128 ** 3, N_voxel_final=300 ** 3, upsamp_list=tier["upsamp_list"],
        update_AlphaMask_list=tier["update_AlphaMask_list"], lr_decay_iters=tier["lr_decay_iters"],
        n_lamb_sigma=[16, 16, 16], n_lamb_sh=[48, 48, 48], fea2denseAct="relu", view_pe=2, fea_pe=2,
        L1_weight_inital=8e-5, L1_weight_rest=4e-5, rm_weight_mask_thre=1e-4, TV_weight_density=0.1, TV_weight_app=0.01,
        compute_extra_metrics=1, run_nerf=False, white_bkgd=True, sampling_opt=False, appearance_embedding_size=1063)
    return [train_config, dataset_config, model_config]


# render variant -> (train variant, checkpoint stem relative to ./log, merged?, render switches, sampling_opt)
_RENDER = {
    "lowquality_render": ("lowquality", "matrix_city_blockA_lowquality", False, {}, True),
    "lowquality_BranchParallel_render": ("lowquality_BranchParallel", "matrix_city_blockA_lowquality_BranchParallel", True,
                                         {"branch_parallel": False}, True),
    "lowquality_Branch2ChannelParallel_render": ("lowquality_BranchParallel", "matrix_city_blockA_lowquality_BranchParallel",
                                                 True, {"branch_parallel": False, "channel_parallel": True,
                                                        "channel_parallel_size": 2}, True),
    "lowquality_ChannelParallel_render": ("lowquality_ChannelParallel", "matrix_city_blockA_lowquality_ChannelParallel", True,
                                          {}, True),
    "lowquality_seq2ChannelParallel_render": ("lowquality_ChannelParallel", "matrix_city_blockA_lowquality_ChannelParallel",
                                              True, {"channel_parallel": True, "channel_parallel_size": 2}, True),
    "multi_render": ("multi", "matrix_city_blockA_multi", False, {}, True),
    "multi_ddp_render": ("multi_ddp", "matrix_city_blockA_multi_ddp", False, {}, True),
    "multi_BranchParallel_render": ("multi_BranchParallel", "matrix_city_blockA_multi_BranchParallel", True,
                                    {"branch_parallel": False}, True),
    "multi_BranchParallel_channel_last_render": ("multi_BranchParallel", "matrix_city_blockA_multi_BranchParallel",
                                                 "channel_last", {"branch_parallel": False}, True),
    "multi_Branch2ChannelParallel_render": ("multi_BranchParallel", "matrix_city_blockA_multi_BranchParallel", True,
                                            {"branch_parallel": False, "channel_parallel": True, "channel_parallel_size": 2},
                                            True),
    "multi_BranchParallel_10x5_render": ("multi_BranchParallel_10x5", "merged_gridnerf_5x5", True,
                                         {"branch_parallel": False}, True),
    "multi_BranchParallel_10x5_channel_last_render": ("multi_BranchParallel_10x5", "merged_gridnerf_5x5", "channel_last",
                                                      {"branch_parallel": False}, True),
    "multi_ChannelParallel_render": ("multi_ChannelParallel", "matrix_city_blockA_multi_ChannelParallel", True, {}, False),
    "multi_seq2ChannelParallel_render": ("multi_ChannelParallel", "matrix_city_blockA_multi_ChannelParallel", True,
                                         {"channel_parallel": True, "channel_parallel_size": 2}, False),
}


def render(variant: str):
    train_variant, stem, merged, switches, sampling_opt = _RENDER[variant]
    train_config, dataset_config, model_config = train(train_variant)
    suffix = "-merged" if merged else ""
    state = f"state_dict{suffix}{'_channel_last' if merged == 'channel_last' else ''}.th"
    render_config = RenderConfig(ckpt=f"log/{stem}/{state}", kwargs=f"log/{stem}/kwargs{suffix}.th", ckpt_type="full",
                                 **switches).from_train_config(train_config)
    model_config.sampling_opt = sampling_opt
    return [render_config, dataset_config, model_config]
