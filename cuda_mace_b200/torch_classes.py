"""Registers the reference's TorchScript custom classes, implemented by this package's kernels.

    from cuda_mace_b200 import torch_classes
    torch_classes.load()
    tp = torch.classes.inv_message_passing.InvariantMessagePassingTP()

The class names, namespaces and forward() argument lists are those of cuda-mace (cuda_mace/src/*.cpp), so its
Python layer (cuda_mace/ops/*.py, models/InvariantMACE.py:187) works unchanged once its
torch.classes.load_library(...) line (cuda_mace/ops/__init__.py:7-15) points at LIB_PATH.
"""
import os

import torch

from . import _abi

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libcuda_mace_b200_torch.so")
_loaded = False


def load():
    """Loads the C-ABI library and the class registrations (once); returns the path that was loaded."""
    global _loaded
    if not _loaded:
        _abi.load()  # the binding links against the C-ABI library; make sure it is resolvable first
        if not os.path.isfile(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m cuda_mace_b200.build`")
        torch.classes.load_library(LIB_PATH)
        _loaded = True
    return LIB_PATH
