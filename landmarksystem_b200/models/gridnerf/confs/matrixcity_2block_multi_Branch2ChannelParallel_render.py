"""GridNeRF on MatrixCity block A: render variant ``multi_Branch2ChannelParallel_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import render

config = render("multi_Branch2ChannelParallel_render")
