"""Scaffold-GS on MatrixCity block A: ``matrixcity_2block_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.scaffold_gs.confs._matrixcity import render

config = render()
