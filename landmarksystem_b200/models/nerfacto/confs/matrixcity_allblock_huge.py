"""Nerfacto on MatrixCity: training variant ``allblock_huge`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.nerfacto.confs._matrixcity import train

config = train("allblock_huge")
