"""Nerfacto on MatrixCity: render variant ``2block_BranchParallel_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.nerfacto.confs._matrixcity import render

config = render("2block_BranchParallel_render")
render_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
