"""Nerfacto on MatrixCity: training variant ``2block_huge`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.nerfacto.confs._matrixcity import train

config = train("2block_huge")
