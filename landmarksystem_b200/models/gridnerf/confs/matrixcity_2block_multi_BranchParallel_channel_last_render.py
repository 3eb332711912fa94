"""GridNeRF on MatrixCity block A: render variant ``multi_BranchParallel_channel_last_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import render

config = render("multi_BranchParallel_channel_last_render")
