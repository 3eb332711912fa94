"""GridNeRF on MatrixCity block A: training variant ``multi_BranchParallel_10x5`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import train

config = train("multi_BranchParallel_10x5")
