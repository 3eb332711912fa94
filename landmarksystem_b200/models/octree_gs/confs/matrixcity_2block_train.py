"""Octree-GS on MatrixCity block A: ``matrixcity_2block_train`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.octree_gs.confs._matrixcity import train

config = train()
