"""`import adam` of the driver scripts: Adam with weight stashing (see stashing_optimizers.py)."""
from .stashing_optimizers import AdamWithWeightStashing  # noqa: F401
