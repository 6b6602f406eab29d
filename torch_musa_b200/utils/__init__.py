"""Developer utilities: numerical debugging modes, extension building, logging."""
import logging

from .compare_tool import CompareWithCPU, ModuleTracker, NanInfTracker  # noqa: F401
from . import extension  # noqa: F401

LOGGER = logging.getLogger("torch_musa_b200")
if not LOGGER.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(logging.Formatter("[%(name)s %(levelname)s] %(message)s"))
    LOGGER.addHandler(_h)
    LOGGER.setLevel(logging.WARNING)
