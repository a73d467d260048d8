"""Writes tests/golden/reference_schemas.json: the TorchScript schemas of `forward` (and of the pickling
methods) of the six custom classes as the REFERENCE's own library registers them.

Needs oracle/_ref/libcuda_mace.so (python -m oracle.build_ref, where the reference checkout is); no GPU.  Must be a
process of its own, because this project's library registers the same class names.

    python tests/golden/make_reference_schemas.py
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CLASSES = [("inv_message_passing", "InvariantMessagePassingTP"), ("symm_contract", "SymmetricContraction"),
           ("linear_wmma", "Linear"), ("linear_wmma", "ElementalLinear"),
           ("spherical_harmonics", "SphericalHarmonics"), ("cubic_spline", "CubicSpline")]


def schemas():
    out = {}
    for ns, cls in CLASSES:
        obj = getattr(getattr(torch.classes, ns), cls)()
        out[f"{ns}.{cls}"] = {m: str(obj._get_method(m).schema) for m in ("forward", "__getstate__", "__setstate__")}
    return out


if __name__ == "__main__":
    lib = os.path.join(HERE, "..", "..", "oracle", "_ref", "libcuda_mace.so")
    if not os.path.isfile(lib):
        raise SystemExit("build the reference library first: python -m oracle.build_ref")
    torch.classes.load_library(lib)
    path = os.path.join(HERE, "reference_schemas.json")
    with open(path, "w") as f:
        json.dump(schemas(), f, indent=1, sort_keys=True)
    print("wrote", path)
    sys.exit(0)
