"""MatrixCity configurations of Nerfacto, built from one table (variant set of the reference's
benchmarks/nerf/nerfacto/confs/*.py: the "huge" field - 256-wide MLPs, max resolution 8192, 2^21 entries,
proposal samplers (512, 512) -> 64 - single process, data parallel, branch parallel [2,1] / [2,2], debug
lengths, the all-block scene, and their render configurations).  Dataset root: ``LMB_MATRIXCITY_ROOT`` (block A)
and ``LMB_MATRIXCITY_ALL_ROOT`` (all blocks)."""
import os

from landmarksystem_b200.configs import DatasetConfig, RenderConfig, TrainConfig
from landmarksystem_b200.models.nerfacto.nerfacto import NerfactoConfig

ROOT_A = os.environ.get("LMB_MATRIXCITY_ROOT", "./data/MatrixCity/small_city/aerial/pose/block_A")
ROOT_ALL = os.environ.get("LMB_MATRIXCITY_ALL_ROOT", "./data/MatrixCity/small_city/aerial/pose/block_all")
LB = [-1.0378e01, -7.4430e00, -1.1921e-07]
UB = [1.2078e00, 2.4078e00, 9.0000e-01]

# variant -> (expname, train switches, model switches, dataset root)
_TRAIN = {
    "2block_huge": ("matrix_city_blockA_nerfacto", {}, {}, ROOT_A),
    "2block_huge_ddp": ("matrix_city_blockA_nerfacto_ddp", {"vis_every": 500, "n_iters": 50000, "DDP": True}, {}, ROOT_A),
    "2block_huge_debug": ("matrix_city_blockA_huge_nerfacto_debug", {"n_iters": 30000}, {}, ROOT_A),
    "2block_BranchParallel": ("matrix_city_blockA_nerfacto_BranchParallel",
                              {"branch_parallel": True, "plane_division": [2, 1]}, {"aabb_norm_range": [0.0, 1.0]}, ROOT_A),
    "2block_BranchParallel_2x2": ("matrix_city_blockA_nerfacto_BranchParallel_2x2",
                                  {"branch_parallel": True, "plane_division": [2, 2]}, {"appearance_embedding_size": 5621}, ROOT_A),
    "2block_BranchParallel_debug": ("matrix_city_blockA_nerfacto_BranchParallel_debug",
                                    {"n_iters": 30000, "branch_parallel": True, "plane_division": [2, 1]},
                                    {"aabb_norm_range": [0.0, 1.0]}, ROOT_A),
    "2block_lowquality_ddp_train": ("nerfacto_matrix_city_blockA_lowquality_ddp_train", {"DDP": True}, {}, ROOT_A),
    "2block_single_train_ci": ("matrix_city_blockA_nerfacto", {"basedir": "./log_for_ci_test", "N_vis": 0}, {}, ROOT_A),
    "allblock_huge": ("matrix_city_blockall_huge_nerfacto", {"vis_every": 500}, {"appearance_embedding_size": 5621}, ROOT_ALL),
}


def train(variant: str):
    expname, switches, model_switches, root = _TRAIN[variant]
    train_config = TrainConfig(model_name="Nerfacto", expname=expname, basedir="./log", batch_size=16384, debug=False,
                               vis_every=1000, n_iters=100000, N_vis=5, tensorboard=True)
    for key, value in switches.items():
        setattr(train_config, key, value)
    dataset_config = DatasetConfig(dataset_name="matrixcity", datadir=root, downsample_train=1, lb=list(LB), ub=list(UB))
    model_args = dict(
        train_near_far=[0.05, 1000], num_nerf_samples_per_ray=64, num_proposal_samples_per_ray=(512, 512),
        proposal_net_args_list=[
            {"hidden_dim": 16, "log2_hashmap_size": 17, "num_levels": 5, "max_res": 512, "use_linear": False},
            {"hidden_dim": 16, "log2_hashmap_size": 17, "num_levels": 7, "max_res": 2048, "use_linear": False}],
        hidden_dim=256, hidden_dim_color=256, appearance_embedding_dim=32, appearance_embedding_size=1063, max_res=8192,
        proposal_weights_anneal_max_num_iters=5000, log2_hashmap_size=21)
    model_args.update(model_switches)
    return [train_config, dataset_config, NerfactoConfig(**model_args)]


_RENDER = {
    "2block_huge_render": ("2block_huge", False, {"basedir": "./log"}),
    "2block_huge_debug_render": ("2block_huge_debug", False, {}),
    "2block_BranchParallel_render": ("2block_BranchParallel", True, {"branch_parallel": False}),
    "2block_BranchParallel_debug_render": ("2block_BranchParallel_debug", True, {"branch_parallel": False}),
}


def render(variant: str):
    train_variant, merged, switches = _RENDER[variant]
    train_config, dataset_config, model_config = train(train_variant)
    suffix = "-merged" if merged else ""
    stem = train_config.expname
    render_config = RenderConfig(ckpt=f"log/{stem}/state_dict{suffix}.th", kwargs=f"log/{stem}/kwargs{suffix}.th",
                                 ckpt_type="full", **switches).from_train_config(train_config)
    return [render_config, dataset_config, model_config]
