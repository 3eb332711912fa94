"""Import paths of the reference under this package.

``import landmarksystem_b200.compat`` registers an import finder that serves the reference's module paths -
``landmark.*`` and ``benchmarks.nerf.*`` - from this package, so scripts written against the reference
(``from landmark.nerf_components.configs.config_parser import BaseConfig``,
``from benchmarks.nerf.gridnerf.gridnerf import GridNeRF``, ``from landmark import init_inference``) run unchanged.
A top-level name (``landmark``, ``benchmarks``) that a real package on the path already provides is left to that package.

``resolve(name)`` gives the module path here for a reference path.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys
from typing import Optional

_P = "landmarksystem_b200"

# reference path -> path here; the longest matching prefix wins, the rest of the dotted path is kept
_PREFIXES = {
    "landmark": _P,
    "landmark.communicator": f"{_P}.comm",
    "landmark.nerf_components": f"{_P}.components",
    "landmark.nerf_components.configs": f"{_P}.configs",
    "landmark.nerf_components.components_convertor": f"{_P}.convertor",
    "landmark.nerf_components.components_convertor.comm_groups": f"{_P}.comm.train_groups",
    "landmark.nerf_components.components_convertor.parallelize": f"{_P}.convertor.convertor_factory",
    "landmark.nerf_components.components_convertor.fusion": f"{_P}.convertor.convertor_factory",
    "landmark.nerf_components.data.datasets.dataloader": f"{_P}.components.data.datasets",
    "landmark.nerf_components.data.datasets.dataloader.utils": f"{_P}.components.data.datasets",
    "landmark.nerf_components.data.datasets.dataloader.utils.utils": f"{_P}.components.data.datasets.dataset_utils",
    "landmark.nerf_components.data.datasets.dataloader.processeddataset": f"{_P}.components.data.datasets.processed_dataset",
    "landmark.nerf_components.data.datasets.dataloader.blender_dataset": f"{_P}.components.data.datasets.json_datasets",
    "landmark.nerf_components.data.datasets.dataloader.city_dataset": f"{_P}.components.data.datasets.json_datasets",
    "landmark.nerf_components.data.datasets.dataloader.matrixcity_dataset": f"{_P}.components.data.datasets.json_datasets",
    "landmark.nerf_components.data.datasets.dataloader.zhangjiang_dataset": f"{_P}.components.data.datasets.colmap_dataset",
    "landmark.nerf_components.data.utils.tensor_dataclass": f"{_P}.components.data.tensor_dataclass",
    "landmark.nerf_components.model_components": f"{_P}.components",
    "landmark.nerf_components.model_components.fields.encodings.fused_tensor_vm_encoding":
        f"{_P}.components.fields.encodings.tensor_vm_encoding",
    "landmark.nerf_components.model_components.fields.fused_anchor_decoder": f"{_P}.components.fields.anchor_decoder",
    "landmark.nerf_components.model_components.renderers.fused_volume_renderer": f"{_P}.components.renderers.volume_renderer",
    "landmark.nerf_components.ray_samplers.fused_uniform_sampler": f"{_P}.components.ray_samplers.uniform_sampler",
    "landmark.nerf_components.utils.comm_utils": f"{_P}.comm.autograd",
    "landmark.render.inference_engine.inference_engine": f"{_P}.render.inference_engine",
    "landmark.render.parallel_module.parallel_module": f"{_P}.render.parallel_module",
    "landmark.render.parallel_module.optimization_manager": f"{_P}.render.optimization_manager",
    "landmark.render.parameter_loader": f"{_P}.render.offload",
    "landmark.render.scheduler": f"{_P}.render.sches",
    "landmark.render.scheduler.sches": f"{_P}.render.sches",
    "landmark.render.scheduler.instructions": f"{_P}.render.instructions",
    "landmark.render.util": f"{_P}.render",
    "landmark.render.util.inference_module": f"{_P}.render.inference_module",
    "landmark.render.util.initializer": f"{_P}.render.initializer",
    "landmark.render.util.types": f"{_P}.render.types",
    "landmark.render.util.utils": f"{_P}.render.utils",
    "landmark.train.utils": f"{_P}.train.utils",
    "landmark.train.utils.distributed_utils": f"{_P}.train.utils",
    "landmark.train.utils.utils": f"{_P}.train.utils",
    "benchmarks": f"{_P}.models",
    "benchmarks.nerf": f"{_P}.models",
}

# packages of the reference whose content is ONE module here: served as an empty package that forwards attribute
# access to that module, so that both ``from landmark.render.scheduler import gen_scheduler`` and
# ``from landmark.render.scheduler.sches import DDPSche`` resolve
_PACKAGE_OVER_MODULE = {"landmark.render.inference_engine", "landmark.render.parallel_module", "landmark.render.scheduler",
                        "landmark.train.utils"}

# packages of the reference that are plain namespaces here (no module of their own)
_NAMESPACES = {"landmark.nerf_components.data.datasets", "landmark.nerf_components.data.utils",
               "landmark.nerf_components.model_components.fields"}


def resolve(name: str) -> Optional[str]:
    """Module path in this package for the reference's module path ``name``."""
    parts = name.split(".")
    for cut in range(len(parts), 0, -1):
        head = ".".join(parts[:cut])
        if head in _PREFIXES:
            return ".".join([_PREFIXES[head]] + parts[cut:])
    return None


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        module = importlib.import_module(self.target)
        # the package root resolves some names on first access: make them real attributes for ``from landmark import X``
        for lazy in getattr(module, "_LAZY", ()):
            getattr(module, lazy)
        return module

    def exec_module(self, module):
        return None


class _ForwardingPackageLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        return None

    def exec_module(self, module):
        real = importlib.import_module(self.target)
        module.__path__ = []
        module.__getattr__ = lambda name: getattr(real, name)
        module.__all__ = [n for n in dir(real) if not n.startswith("__")]


class _NamespaceLoader(importlib.abc.Loader):
    def create_module(self, spec):
        return None

    def exec_module(self, module):
        module.__path__ = []


class ReferencePathFinder(importlib.abc.MetaPathFinder):
    """Serves ``landmark.*`` and ``benchmarks.nerf.*`` from this package.  It sits in front of the path-based finder:
    an alias of a package is the real package object, whose ``__path__`` would otherwise let the path finder load a
    second copy of a sub-module under the alias name."""

    def __init__(self, roots):
        self.roots = tuple(roots)

    def find_spec(self, fullname, path=None, target=None):
        if fullname.split(".")[0] not in self.roots:
            return None
        if fullname in _NAMESPACES:
            return importlib.machinery.ModuleSpec(fullname, _NamespaceLoader(), is_package=True)
        here = resolve(fullname)
        if here is None:
            return None
        try:
            found = importlib.util.find_spec(here)
        except (ImportError, ValueError):
            found = None
        if found is None:
            return None
        if fullname in _PACKAGE_OVER_MODULE:
            return importlib.machinery.ModuleSpec(fullname, _ForwardingPackageLoader(here), is_package=True)
        return importlib.machinery.ModuleSpec(fullname, _AliasLoader(here), is_package=found.submodule_search_locations is not None)


def install() -> None:
    """Register the finder once, for the top-level names no real package provides."""
    if any(isinstance(f, ReferencePathFinder) for f in sys.meta_path):
        return
    roots = [root for root in ("landmark", "benchmarks")
             if root not in sys.modules and importlib.machinery.PathFinder.find_spec(root) is None]
    if roots:
        sys.meta_path.insert(0, ReferencePathFinder(roots))


install()
