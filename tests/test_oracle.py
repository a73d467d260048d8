"""Pins the float64 CPU restatement: committed fixtures, analytic identities, two independent
constructions of the coupling tensors, finite differences."""
import math
import os

import numpy as np
import torch

from cuda_mace_b200 import cg, systems
from oracle import cg as ocg
from oracle import model as omodel
from oracle import ops as oops
from oracle.sh import real_sh_l3

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_sh_norms_and_low_orders():
    v = torch.randn(64, 3, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    Y = real_sh_l3(v)
    n = v / v.norm(dim=-1, keepdim=True)
    for l in range(4):  # component normalisation: sum_m Y_lm^2 = 2l+1
        assert torch.allclose((Y[l * l:(l + 1) ** 2] ** 2).sum(0), torch.full((64,), 2.0 * l + 1, dtype=torch.float64), atol=1e-12)
    # l=1 is sqrt(3) * (x, y, z) in the input's own axis order (e3nn convention)
    assert torch.allclose(Y[1:4].t(), math.sqrt(3.0) * n, atol=1e-13)
    # scale invariance
    assert torch.allclose(real_sh_l3(3.7 * v), Y, atol=1e-13)


def test_sh_orthonormal_on_the_sphere():
    pts, w = ocg._sphere_quadrature()
    Y = real_sh_l3(torch.from_numpy(pts)).numpy()
    gram = np.einsum("iq,jq,q->ij", Y, Y, w)
    assert np.abs(gram - np.eye(16)).max() < 1e-12


def test_u_tensors_two_constructions_agree(U):
    """Gaunt-integral construction (oracle) vs Racah-formula construction (package)."""
    U3o, U2o, U1o = ocg.u_matrices()
    U3, U2, U1 = U
    assert U3.shape == (16, 16, 16, 23) and U2.shape == (16, 16, 4) and U1.shape == (16, 1)
    assert (U3 - U3o).abs().max() < 1e-12 and (U2 - U2o).abs().max() < 1e-14 and (U1 - U1o).abs().max() == 0
    nz = U3 != 0
    assert int(nz.sum()) == 353
    assert int(nz.any(-1).sum(-1).max()) == 3          # at most 3 k per (i, j)
    assert int((nz.any(-1).sum(-1) > 0).sum()) == 234  # non-empty (i, j) pairs
    assert int(nz.sum(-1).max()) == 1                  # one path per (i, j, k)


def test_contraction_is_rotation_invariant(U):
    """Features built from harmonics of rotated vectors give the same contraction: pins the sign and
    axis conventions of the harmonics against those of the coupling tensors."""
    g = torch.Generator().manual_seed(3)
    v = torch.randn(5, 6, 3, generator=g, dtype=torch.float64)
    amp = torch.randn(5, 6, 1, 2, generator=g, dtype=torch.float64)
    q, _ = torch.linalg.qr(torch.randn(3, 3, generator=g, dtype=torch.float64))
    if torch.det(q) < 0:
        q[:, 0] = -q[:, 0]
    W3, W2, W1 = (torch.randn(1, n, 2, generator=g, dtype=torch.float64) for n in (23, 4, 1))

    def feats(vec):
        Y = real_sh_l3(vec.reshape(-1, 3)).t().reshape(5, 6, 16)
        return (Y[..., None] * amp).sum(1)  # [5, 16, 2]

    at = torch.zeros(5, dtype=torch.long)
    a = oops.symmetric_contraction(feats(v), at, *U, W3, W2, W1)
    b = oops.symmetric_contraction(feats(v @ q.t()), at, *U, W3, W2, W1)
    assert (a - b).abs().max() < 1e-10 * a.abs().max()


def test_sparse_packing_round_trip(U):
    """The reference's sparse table layout reproduces the dense contraction (forward nesting of
    symmetric_contraction_impl.cu:108-175 evaluated in numpy)."""
    U3, U2, U1 = U
    maxnz, n3, i3, v3, n2, i2, v2, n1, i1 = oops.pack_sparse_u(U3, U2, U1)
    assert maxnz == 3
    g = torch.Generator().manual_seed(5)
    x = torch.randn(16, generator=g, dtype=torch.float64)
    w3, w2, w1 = (torch.randn(n, generator=g, dtype=torch.float64) for n in (23, 4, 1))
    out = 0.0
    for i in range(16):
        o2 = 0.0
        for j in range(16):
            uw2 = float(v2[i, j]) * w2[int(i2[i, j])] if n2[i, j] > 0 else 0.0
            o3 = 0.0
            for k in range(int(n3[i, j])):
                pk = int(i3[k, i, j])
                o3 += float(v3[k, i, j]) * w3[pk & 0xFF] * x[(pk >> 8) & 0xFF]
            o2 += (o3 + uw2) * x[j]
        out += (o2 + (w1[0] if i == 0 else 0.0)) * x[i]
    dense = oops.symmetric_contraction(x[None, :, None], torch.zeros(1, dtype=torch.long), U3, U2, U1,
                                       w3[None, :, None], w2[None, :, None], w1[None, :, None])
    assert abs(float(out) - float(dense)) < 2e-6 * abs(float(dense))  # the reference's tables are float32


def test_fixtures_ops():
    z = np.load(os.path.join(GOLD, "ops_small.npz"))
    t = {k: torch.from_numpy(z[k]) for k in z.files}
    U = cg.u_matrices()
    N = t["X"].shape[0]
    assert torch.equal(real_sh_l3(t["vec"]), t["Y"])
    assert (oops.invariant_message_passing(t["X"], t["Y"], t["R"], t["send"], t["recv"], N) - t["imp"]).abs().max() < 1e-13
    assert (oops.linear(t["M"], t["W"]) - t["lin"]).abs().max() < 1e-13
    Z = t["WZ"].shape[0]
    assert (oops.elemental_linear(t["M"], t["WZ"], systems.one_hot(t["at"], Z)) - t["elin"]).abs().max() < 1e-13
    con = oops.symmetric_contraction(t["M"], t["at"], *U, t["W3"], t["W2"], t["W1"])
    assert (con - t["con"]).abs().max() < 1e-10 * t["con"].abs().max()
    assert (omodel.radial_embedding(t["vec"].norm(dim=-1), 5.0) - t["bessel"]).abs().max() < 1e-13


def test_fixture_cfg0_energy_forces(U):
    z = np.load(os.path.join(GOLD, "cfg0_energy_forces.npz"))
    s = systems.make_system("cfg0")
    ei, sh = systems.neighbor_list(s["positions"], s["box"], (True, True, True), 5.0)
    assert ei.shape[1] == int(z["n_edges"])
    params = systems.init_params(s["channels"], s["n_species"], 0)
    e, ei_, f = omodel.energy_and_forces(params, U, torch.from_numpy(s["positions"]), systems.one_hot(s["species"], 4),
                                         torch.from_numpy(ei), torch.from_numpy(sh))
    assert abs(float(e) - float(z["energy"])) < 1e-10 * abs(float(z["energy"]))
    assert np.abs(f.numpy() - z["forces"]).max() < 1e-10 * np.abs(z["forces"]).max()
    assert np.abs(f.numpy().sum(0)).max() < 1e-12  # translation invariance


def test_forces_match_finite_differences(U):
    s = systems.make_system("cfg0")
    pos = torch.from_numpy(s["positions"][:192])
    ei, sh = systems.neighbor_list(s["positions"], s["box"], (True, True, True), 5.0)
    ei, sh = torch.from_numpy(ei), torch.from_numpy(sh)
    params = systems.init_params(32, 4, 11)
    attrs = systems.one_hot(s["species"], 4)
    _, _, f = omodel.energy_and_forces(params, U, pos, attrs, ei, sh)

    def energy(p):
        return float(omodel.node_energies(params, U, p, attrs, ei, sh).sum())

    h = 1e-5
    for atom, axis in ((3, 1), (100, 2)):
        pp, pm = pos.clone(), pos.clone()
        pp[atom, axis] += h
        pm[atom, axis] -= h
        fd = -(energy(pp) - energy(pm)) / (2 * h)
        assert abs(fd - float(f[atom, axis])) < 1e-6 * max(1.0, float(f.abs().max()))


def test_neighbor_list_matches_brute_force():
    s = systems.make_system("cfg0")
    pos, L = s["positions"], s["box"][0]
    ei, sh = systems.neighbor_list(pos, s["box"], (True, True, True), 5.0)
    count = 0
    for sx in (-1, 0, 1):
        for sy in (-1, 0, 1):
            for sz in (-1, 0, 1):
                d = pos[None] + np.array([sx, sy, sz]) * L - pos[:, None]
                r2 = (d * d).sum(-1)
                count += int(((r2 < 25.0) & (r2 > 1e-12)).sum())
    assert ei.shape[1] == count
    assert (np.diff(ei[0]) >= 0).all()
    vec = pos[ei[1]] - pos[ei[0]] + sh
    assert np.sqrt((vec * vec).sum(-1)).max() < 5.0
    # full list: every edge has its reverse with the opposite shift
    edges = set(zip(ei[0].tolist(), ei[1].tolist(), map(tuple, np.round(sh, 6).tolist())))
    for a, b, s3 in list(edges)[:500]:
        assert (b, a, tuple(-x + 0.0 for x in s3)) in edges


def test_spline_tabulation_tracks_exact_radial(U):
    params = omodel.add_spline_tables(systems.init_params(32, 2, 5))
    P = params["layers"][0]
    r = torch.linspace(0.9, 4.99, 400, dtype=torch.float64)
    exact = omodel.radial_mlp(omodel.radial_embedding(r, 5.0), P["W_radial"])
    spl = oops.cubic_spline_eval(r, P["spline_knots"], P["spline_coeffs"], P["spline_h"], 5.0)
    assert (spl - exact).abs().max() < 1e-4 * exact.abs().max()
    assert oops.cubic_spline_eval(torch.tensor([5.5], dtype=torch.float64), P["spline_knots"], P["spline_coeffs"],
                                  P["spline_h"], 5.0).abs().max() == 0


def _reference_pins():
    import os

    import numpy as np

    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_pins.npz"))


def test_sparse_u_tables_equal_the_reference_packing(U):
    """The sparse U tables of the oracle and of the package equal, entry for entry, what the reference's own
    setup_sparse_matrices (cuda_mace/ops/symmetric_contraction.py:91-187, run by tests/golden/make_reference_pins.py)
    makes of the same dense U tensors: counts, packed index words (k, path and the two partner paths), values."""
    import numpy as np

    from cuda_mace_b200 import ops
    from oracle import ops as oops

    z = _reference_pins()
    U32 = [u.to(torch.float32) for u in U]
    for pack in (oops.pack_sparse_u, ops.pack_sparse_u):
        maxnz, n3, i3, v3, n2, i2, v2, n1, i1 = pack(*U32)
        assert int(maxnz) == int(z["u3_max_nonsparse"]) == 3
        for mine, ref in ((n3, "U3_num_nonsparse"), (i3, "U3_indices"), (n2, "U2_num_nonsparse"), (i2, "U2_indices"),
                          (n1, "U1_num_values"), (i1, "U1_index")):
            assert np.array_equal(mine.cpu().numpy().astype(np.int64), z[ref].astype(np.int64)), ref
        assert np.array_equal(v3.cpu().numpy().astype(np.float32), z["U3_values"])
        assert np.array_equal(v2.cpu().numpy().astype(np.float32), z["U2_values"])
    assert int(z["U3_num_nonsparse"].sum()) == 353 and int((z["U3_num_nonsparse"] > 0).sum()) == 234


def test_spline_coefficients_equal_the_reference_solve():
    """Natural-spline coefficients against the reference's own tridiagonal solve
    (cuda_mace/ops/cubic_spline.py:41-84) on the same knots and values."""
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    z = _reference_pins()
    x, y, h = torch.from_numpy(z["spline_knots"]), torch.from_numpy(z["spline_values"]), float(z["spline_h"])
    ref = torch.from_numpy(z["spline_coefficients"])
    for solve in (oops.cubic_spline_coefficients, ops.cubic_spline_coefficients):
        got = solve(x, y, h)
        assert got.shape == ref.shape
        assert float((got - ref).abs().max()) < 1e-12 * float(ref.abs().max())
