"""``landmarksystem_b200.compat``: the reference's import paths (``landmark.*``, ``benchmarks.nerf.*``) served from this
package.  Runs in a child interpreter so that the import finder does not outlive the test."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import sys, textwrap
import landmarksystem_b200.compat as compat

# the imports a user script of the reference makes (doc/source/rendering_api.rst, tests/utils.py, the conf files)
from landmark import InferenceModule, init_inference
from landmark.communicator import init_communication_context
from landmark.nerf_components.configs import ConfigClass, DatasetConfig, RenderConfig, TrainConfig
from landmark.nerf_components.configs.config_parser import BaseConfig
from landmark.nerf_components.data.data_manager import DatasetManager
from landmark.nerf_components.data.datasets.dataloader.utils.ray_utils import get_ray_directions_blender
from landmark.nerf_components.model import BaseGaussian, BaseNeRF
from landmark.nerf_components.model_components.fields.encodings.tensor_vm_encoding import TensorVMEncoding
from landmark.nerf_components.scene import SceneManager
from landmark.nerf_components.utils.tcnn_utils import tcnn
from landmark.render import InferenceEngine
from landmark.render.scheduler import gen_scheduler
from landmark.render.scheduler.sches import DDPSche
from landmark.render.util import InferenceModuleInitializer, transform_gridnerf_model_to_channel_last
from landmark.render.parameter_loader import OffloadModule
from landmark.train import NeRFTrainer
from landmark.train.utils.distributed_utils import get_dp_group, is_main_rank
from landmark.utils import Config, EnvSetting
from benchmarks.nerf.gridnerf.gridnerf import GridNeRF, GridNeRFConfig
from benchmarks.nerf.octree_gs.gs_model import OctreeGS

import landmarksystem_b200 as lm
import landmarksystem_b200.configs as configs
import landmarksystem_b200.models.gridnerf.gridnerf as gridnerf
assert GridNeRF is gridnerf.GridNeRF and BaseConfig is configs.BaseConfig and init_inference is lm.init_inference
assert compat.resolve("landmark.render.parameter_loader.buffer_manager") == "landmarksystem_b200.render.offload.buffer_manager"
assert compat.resolve("benchmarks.nerf.nerfacto.nerfacto_trainer") == "landmarksystem_b200.models.nerfacto.nerfacto_trainer"

# a configuration file in the reference's own style, render variant importing the training variant with ``*``
folder = sys.argv[1]
open(folder + "/train_conf.py", "w").write(textwrap.dedent("""
    from benchmarks.nerf.gridnerf.gridnerf import GridNeRFConfig
    from landmark.nerf_components.configs import DatasetConfig, TrainConfig

    train_config = TrainConfig(model_name="GridNeRF", expname="compat_run", basedir="./log", batch_size=8192, n_iters=10)
    dataset_config = DatasetConfig(dataset_name="matrixcity", datadir="nowhere", lb=[-1.0, -1.0, 0.0], ub=[1.0, 1.0, 0.9])
    model_config = GridNeRFConfig(ndims=1, resMode=[1, 2, 4], nonlinear_density=True, train_near_far=[0.6, 3.5])
    config = [train_config, dataset_config, model_config]
"""))
open(folder + "/render_conf.py", "w").write(textwrap.dedent("""
    from train_conf import *
    from landmark.nerf_components.configs import RenderConfig

    render_config = RenderConfig(ckpt="log/compat_run/state_dict.th", kwargs="log/compat_run/kwargs.th",
                                 ckpt_type="full").from_train_config(train_config)
    model_config.sampling_opt = True
    config = [render_config, dataset_config, model_config]
"""))
cfg = BaseConfig.from_file(folder + "/render_conf.py")
assert cfg.is_train is False and cfg.sampling_opt is True and cfg.resMode == [1, 2, 4] and cfg.ckpt.endswith("state_dict.th")

# no module was loaded a second time under an alias name
own = set(compat._NAMESPACES) | set(compat._PACKAGE_OVER_MODULE)
twice = [m for m in sys.modules if m.split(".")[0] in ("landmark", "benchmarks") and sys.modules[m].__name__ == m and m not in own]
assert not twice, twice
print("compat ok")
'''


def test_reference_import_paths_resolve_to_this_package(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    done = subprocess.run([sys.executable, "-c", SCRIPT, str(tmp_path)], capture_output=True, text=True, env=env,
                          cwd=str(tmp_path), timeout=300)
    assert done.returncode == 0 and "compat ok" in done.stdout, done.stderr[-3000:]


def test_every_mapped_prefix_points_at_an_existing_module():
    import importlib.util

    from landmarksystem_b200 import compat

    try:
        for ref, here in compat._PREFIXES.items():
            assert importlib.util.find_spec(here) is not None, (ref, here)
    finally:                                     # importing the module registered the finder: take it out again
        sys.meta_path[:] = [f for f in sys.meta_path if not isinstance(f, compat.ReferencePathFinder)]
