"""MatrixCity block A configurations of InstantNGP, built from one table (the variant set of the reference's
benchmarks/nerf/instant_ngp/confs/*.py: ``plconfig`` single process with a 2^24 hash table, data parallel,
branch parallel [2,2] / [2,1] with ``aabb_norm_range=[0,1]``, low-quality / debug sizes, and the render
configurations that load the trained or merged checkpoints).  Dataset root: ``LMB_MATRIXCITY_ROOT``."""
import os

from landmarksystem_b200.configs import DatasetConfig, RenderConfig, TrainConfig
from landmarksystem_b200.models.instant_ngp.instant_ngp import InstantNGPConfig

DATA_ROOT = os.environ.get("LMB_MATRIXCITY_ROOT", "./data/MatrixCity/small_city/aerial/pose/block_A")
LB = [-1.0378e01, -7.4430e00, -1.1921e-07]
UB = [1.2078e00, 2.4078e00, 9.0000e-01]

# variant -> (expname, train switches, model switches)
_TRAIN = {
    "plconfig": ("matrix_city_blockA_ingp", {}, {"log2_hashmap_size": 24, "background_color": "white"}),
    "plconfig_ddp": ("matrix_city_blockA_ingp_ddp", {"vis_every": 500, "n_iters": 50000, "DDP": True},
                     {"log2_hashmap_size": 24, "background_color": "white"}),
    "ddp_train": ("iNGP_matrixcity_blockA_ddp_train", {"DDP": True}, {"log2_hashmap_size": 24}),
    "lowquality_ddp_train": ("iNGP_matrixcity_blockA_lowquality_ddp_train",
                             {"batch_size": 4096, "vis_every": 5000, "n_iters": 30000, "DDP": True}, {}),
    "BranchParallel": ("matrix_city_blockA_instant_ngp_branch",
                       {"branch_parallel": True, "plane_division": [2, 2]},
                       {"log2_hashmap_size": 24, "aabb_norm_range": [0.0, 1.0]}),
    "lowquality_BranchParallel": ("matrix_city_blockA_lowquality_instant_ngp_branch",
                                  {"n_iters": 100, "branch_parallel": True, "plane_division": [2, 1]},
                                  {"log2_hashmap_size": 24, "aabb_norm_range": [0.0, 1.0]}),
    "lowquality_debug": ("matrix_city_blockA_lowquality_debug_new18", {"batch_size": 4096, "vis_every": 5000, "n_iters": 30000},
                         {}),
    "single_train_ci": ("matrix_city_blockA_ingp", {"basedir": "./log_for_ci_test", "N_vis": 0},
                        {"log2_hashmap_size": 24, "background_color": "white"}),
}


def train(variant: str):
    expname, switches, model_switches = _TRAIN[variant]
    train_config = TrainConfig(model_name="InstantNGP", expname=expname, basedir="./log", batch_size=16384, debug=False,
                               vis_every=1000, n_iters=100000, N_vis=5, tensorboard=True)
    for key, value in switches.items():
        setattr(train_config, key, value)
    dataset_config = DatasetConfig(dataset_name="matrixcity", datadir=DATA_ROOT, downsample_train=1, lb=list(LB), ub=list(UB))
    model_config = InstantNGPConfig(train_near_far=[0.05, 1000], appearance_embedding_size=1063, **model_switches)
    return [train_config, dataset_config, model_config]


# render variant -> (train variant, merged checkpoint?, render switches)
_RENDER = {
    "plconfig_render": ("plconfig", False, {}),
    "plconfig_ddp_render": ("plconfig_ddp", False, {}),
    "ddp_train_render": ("ddp_train", False, {}),
    "lowquality_debug_render": ("lowquality_debug", False, {}),
    "BranchParallel_render": ("BranchParallel", True, {"branch_parallel": False}),
    "lowquality_BranchParallel_render": ("lowquality_BranchParallel", True, {"branch_parallel": False}),
}


def render(variant: str):
    train_variant, merged, switches = _RENDER[variant]
    train_config, dataset_config, model_config = train(train_variant)
    suffix = "-merged" if merged else ""
    stem = train_config.expname
    render_config = RenderConfig(ckpt=f"log/{stem}/state_dict{suffix}.th", kwargs=f"log/{stem}/kwargs{suffix}.th",
                                 ckpt_type="full", **switches).from_train_config(train_config)
    return [render_config, dataset_config, model_config]
