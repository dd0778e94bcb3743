"""`import sgd` of the driver scripts: SGD with weight stashing (see stashing_optimizers.py)."""
from .stashing_optimizers import SGDWithWeightStashing  # noqa: F401
