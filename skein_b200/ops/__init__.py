"""Operators: see functional.py (dispatching entry points) and reference.py (fp32 PyTorch oracles)."""
from . import reference
from .functional import *  # noqa: F401,F403
from .functional import workspace, Workspace
