"""Oracle-side helpers of the GPU parity tests: the checker lives in ``oracle/harness.py`` (it is shared with the smoke
entry and the benchmark's checking legs); this module re-exports it under the name the tests use."""
from oracle.harness import *  # noqa: F401,F403
from oracle.harness import MAX_ABS_16BIT, MAX_ABS_F32, MEAN_ABS_16BIT, golden  # noqa: F401
