"""Scaffold-GS on MatrixCity block A: ``matrixcity_2block_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.scaffold_gs.confs._matrixcity import render

config = render()
render_config, dataset_config, model_config = config        # the blocks by name, for files that import this one with *
