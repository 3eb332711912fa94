"""GridNeRF on MatrixCity block A: render variant ``multi_seq2ChannelParallel_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import render

config = render("multi_seq2ChannelParallel_render")
render_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
