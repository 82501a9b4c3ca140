"""CPU oracle for the activation-quantized linear path (test infrastructure).

Only tests, the smoke check and the bench's CPU-baseline / reference arm may
import this package; nothing in ``cider_b200`` does.
"""
from .oracle import *  # noqa: F401,F403
