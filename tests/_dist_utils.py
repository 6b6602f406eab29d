"""Test-side alias of the package's multi-process harness (``torch_musa_b200.testing.distributed``)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from torch_musa_b200.testing.distributed import (MultiProcessTestCase, free_port, run_ranks,  # noqa: E402,F401
                                                 spawn_isolated_test)
