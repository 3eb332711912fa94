"""Nerfacto on MatrixCity: render variant ``2block_BranchParallel_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.nerfacto.confs._matrixcity import render

config = render("2block_BranchParallel_render")
