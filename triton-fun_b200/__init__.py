"""splat_b200: B200-native SPLAT sparse-attention path.

The drop-in modules (``acsr_helpers``, ``r_sddmm``, ``r_softmax``, ``r_spmm``, ``r_attention``)
live in the ``SPLAT`` sub-directory and import each other by bare name, exactly like the reference's
``SPLAT`` directory; put that directory on ``sys.path`` (``add_to_path()`` does it) and import them
as you would the reference's.
"""
import os
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
SPLAT_DIR = os.path.join(PACKAGE_DIR, "SPLAT")


def add_to_path() -> str:
    if SPLAT_DIR not in sys.path:
        sys.path.insert(0, SPLAT_DIR)
    return SPLAT_DIR
