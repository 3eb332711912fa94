"""InstantNGP on MatrixCity block A: render variant ``lowquality_BranchParallel_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.instant_ngp.confs._matrixcity import render

config = render("lowquality_BranchParallel_render")
render_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
