"""Real spherical harmonics up to l=3, float64 torch restatement (test infrastructure).

Follows cuda_mace/cuda/src/spherical_harmonics_impl.cu:62-125 and the e3nn call it
is tested against (tests/spherical_harmonics.py:9-11:
``o3.SphericalHarmonics(l<=3, normalize=True, normalization="component")``):

* the input vector is normalised;
* the axes are permuted before the textbook real harmonics are evaluated, the
  harmonic's (x, y, z) being the input's components (2, 0, 1)
  (spherical_harmonics_impl.cu:62-65), which makes l=1 come out as sqrt(3)*(x, y, z);
* every component is scaled by sqrt(4*pi) (spherical_harmonics_impl.cu:36, :124), so
  that sum_m Y_lm^2 = 2l+1.

The output layout is [16, E] (l-major, edge-minor) like the reference's
(spherical_harmonics_wrapper.cpp:32-55).
"""
import math

import torch

# l value of each of the 16 (l, m) components
L_OF_LM = [0, 1, 1, 1, 2, 2, 2, 2, 2, 3, 3, 3, 3, 3, 3, 3]


def real_sh_l3(vec: torch.Tensor) -> torch.Tensor:
    """vec [E, 3] -> Y [16, E]; differentiable (torch autograd gives dY/dvec)."""
    n = vec / vec.norm(dim=-1, keepdim=True)
    # axis permutation of spherical_harmonics_impl.cu:62-65
    X, Y, Z = n[:, 2], n[:, 0], n[:, 1]
    X2, Y2, Z2 = X * X, Y * Y, Z * Z
    s3, s5, s7, s15 = math.sqrt(3.0), math.sqrt(5.0), math.sqrt(7.0), math.sqrt(15.0)
    s105 = math.sqrt(105.0)
    a = math.sqrt(35.0 / 8.0)
    b = math.sqrt(21.0 / 8.0)
    out = [
        torch.ones_like(X),
        s3 * Y,
        s3 * Z,
        s3 * X,
        s15 * X * Y,
        s15 * Y * Z,
        0.5 * s5 * (2.0 * Z2 - X2 - Y2),
        s15 * X * Z,
        0.5 * s15 * (X2 - Y2),
        a * Y * (3.0 * X2 - Y2),
        s105 * X * Y * Z,
        b * Y * (4.0 * Z2 - X2 - Y2),
        0.5 * s7 * Z * (2.0 * Z2 - 3.0 * X2 - 3.0 * Y2),
        b * X * (4.0 * Z2 - X2 - Y2),
        0.5 * s105 * Z * (X2 - Y2),
        a * X * (X2 - 3.0 * Y2),
    ]
    return torch.stack(out, dim=0)
