"""Generates tests/golden/reference_pins.npz by running the reference's OWN host-side Python on seeded inputs.

Two pieces of cuda-mace's Python layer are plain torch and can run in a container that has neither mace nor e3nn
nor a GPU, once their module-level imports are satisfied by empty stand-ins:

* cuda_mace/ops/cubic_spline.py:41-84       CubicSpline.cubic_spline_coefficients(x, y, h)
* cuda_mace/ops/symmetric_contraction.py:91-187   SymmetricContraction.setup_sparse_matrices()
  (the sparse packing of the U tensors: counts, packed int32 indices, values)

The outputs are stored as fixtures; tests/test_oracle.py checks the oracle's and the package's restatements against
them bit for bit (tables) / to rounding (spline).  Run where the reference checkout is available:

    python tests/golden/make_reference_pins.py /path/to/cuda-mace
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))


def load_reference_module(ref_root, rel_path, name):
    # stand-ins for the imports at the top of the reference files (never called here)
    for mod in ("e3nn", "mace", "mace.tools", "mace.tools.cg", "mace.modules", "mace.modules.symmetric_contraction"):
        sys.modules.setdefault(mod, types.ModuleType(mod))
    sys.modules["e3nn"].o3 = types.SimpleNamespace()
    sys.modules["mace.tools.cg"].U_matrix_real = None
    sys.modules["mace.modules.symmetric_contraction"].SymmetricContraction = object
    spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel_path))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def main(ref_root):
    from cuda_mace_b200 import cg

    out = {}
    # ---- cubic spline coefficients ------------------------------------------------------------------------
    spline = load_reference_module(ref_root, "cuda_mace/ops/cubic_spline.py", "ref_cubic_spline")
    g = torch.Generator().manual_seed(11)
    knots = torch.linspace(1e-12, 6.0, 33, dtype=torch.float64)
    values = torch.randn(33, 12, generator=g, dtype=torch.float64).cumsum(0) * 0.1
    h = float(knots[1] - knots[0])
    coeffs = spline.CubicSpline.cubic_spline_coefficients(None, knots, values, h)
    out.update(spline_knots=knots.numpy(), spline_values=values.numpy(), spline_h=np.float64(h),
               spline_coefficients=coeffs.numpy())
    # ---- sparse packing of the U tensors ---------------------------------------------------------------------
    symm = load_reference_module(ref_root, "cuda_mace/ops/symmetric_contraction.py", "ref_symmetric_contraction")
    U3, U2, U1 = (u.to(torch.float32) for u in cg.u_matrices())
    obj = symm.SymmetricContraction.__new__(symm.SymmetricContraction)
    torch.nn.Module.__init__(obj)
    obj.device = "cpu"
    obj.irreps_out = [None]          # one output irrep (L = 0); only its position is used
    obj.U_matrices = {3: {0: U3}, 2: {0: U2}, 1: {0: U1}}
    obj.setup_sparse_matrices()
    out.update(u3_max_nonsparse=np.int64(obj.u3_max_nonsparse),
               U3_num_nonsparse=obj.U3_num_nonsparse.numpy(), U3_indices=obj.U3_indices.numpy(),
               U3_values=obj.U3_values.numpy(), U2_num_nonsparse=obj.U2_num_nonsparse.numpy(),
               U2_indices=obj.U2_indices.numpy(), U2_values=obj.U2_values.numpy(),
               U1_num_values=obj.U1_num_values.numpy(), U1_index=obj.U1_index.numpy())
    path = os.path.join(HERE, "reference_pins.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: getattr(v, "shape", ()) for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_reference_pins.py <path of the cuda-mace checkout>")
    main(sys.argv[1])
