"""GridNeRF on MatrixCity block A: training variant ``multi_ddp`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import train

config = train("multi_ddp")
