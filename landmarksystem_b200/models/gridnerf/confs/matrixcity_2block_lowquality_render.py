"""GridNeRF on MatrixCity block A: render variant ``lowquality_render`` (see ``_matrixcity.py``)."""
from landmarksystem_b200.models.gridnerf.confs._matrixcity import render

config = render("lowquality_render")
