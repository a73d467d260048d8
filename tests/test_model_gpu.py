"""Whole-model parity on the GPU: energies and forces against the float64 CPU oracle and the
committed fixture; float64 within 1e-10, float32 within 1e-5 (energy) / 1e-4 (forces), relative."""
import os

import numpy as np
import pytest
import torch

from tests.util import rel_err

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def build(name, U, dtype, radial="exact", n_atoms=None, seed=0, channels=None):
    from cuda_mace_b200 import model, systems
    from oracle import model as omodel

    s = systems.make_system(name, n_atoms=n_atoms)
    ei, sh = systems.neighbor_list(s["positions"], s["box"], (True, True, True), 5.0)
    params = systems.init_params(channels or s["channels"], s["n_species"], seed)
    if radial == "spline":
        omodel.add_spline_tables(params)
    m = model.InvariantMACE(params, U, dtype=dtype, device="cuda", radial=radial)
    data = dict(positions=torch.from_numpy(s["positions"]).cuda(),
                species=torch.from_numpy(s["species"]).to(torch.int32).cuda(),
                edge_index=torch.from_numpy(ei).to(torch.int32).cuda(),
                shifts=torch.from_numpy(sh).cuda())
    return s, ei, sh, params, m, data


@pytest.mark.parametrize("dtype,tol_e,tol_f", [(torch.float64, 1e-10, 1e-10), (torch.float32, 1e-5, 1e-4)])
def test_cfg0_matches_fixture_and_oracle(dtype, tol_e, tol_f, U):
    z = np.load(os.path.join(GOLD, "cfg0_energy_forces.npz"))
    s, ei, sh, params, m, data = build("cfg0", U, dtype)
    out = m(data)
    assert abs(float(out["energy"]) - float(z["energy"])) < tol_e * abs(float(z["energy"]))
    assert abs(float(out["interaction_energy"]) - float(z["interaction"])) < tol_e * abs(float(z["interaction"]))
    assert rel_err(out["forces"], torch.from_numpy(z["forces"])) < tol_f
    # a second call reuses the cached topology; the kernels are bitwise reproducible, torch's
    # index_add in the position gradient is not, so compare to rounding
    out2 = m(data)
    assert rel_err(out2["forces"], out["forces"]) < (1e-13 if dtype == torch.float64 else 1e-5)


@pytest.mark.parametrize("dtype,tol_e,tol_f", [(torch.float64, 1e-10, 1e-10), (torch.float32, 1e-5, 1e-4)])
def test_water_like_box_matches_oracle(dtype, tol_e, tol_f, U):
    """The 2-species, 128-channel configuration at a CPU-affordable size (375 atoms)."""
    from cuda_mace_b200 import systems
    from oracle import model as omodel

    s, ei, sh, params, m, data = build("water3000", U, dtype, n_atoms=375, seed=1)
    e, e_inter, f = omodel.energy_and_forces(params, U, torch.from_numpy(s["positions"]),
                                             systems.one_hot(s["species"], 2), torch.from_numpy(ei), torch.from_numpy(sh))
    out = m(data)
    assert abs(float(out["interaction_energy"]) - float(e_inter)) < tol_e * abs(float(e_inter))
    assert rel_err(out["forces"], f) < tol_f
    assert out["forces"].sum(0).abs().max().item() < 1e-3 * out["forces"].abs().max().item()


def test_spline_variant_matches_spline_oracle(U):
    """The reference's tabulated radial path (float32 + cubic spline), checked against the oracle's
    spline variant, and within spline accuracy of the exact model."""
    from cuda_mace_b200 import systems
    from oracle import model as omodel

    s, ei, sh, params, m, data = build("cfg0", U, torch.float64, radial="spline")
    _, e_s, f_s = omodel.energy_and_forces(params, U, torch.from_numpy(s["positions"]), systems.one_hot(s["species"], 4),
                                           torch.from_numpy(ei), torch.from_numpy(sh), radial="spline")
    out = m(data)
    assert abs(float(out["interaction_energy"]) - float(e_s)) < 1e-9 * abs(float(e_s))
    assert rel_err(out["forces"], f_s) < 1e-8
    z = np.load(os.path.join(GOLD, "cfg0_energy_forces.npz"))
    assert abs(float(out["interaction_energy"]) - float(z["interaction"])) < 1e-4 * abs(float(z["interaction"]))


@pytest.mark.parametrize("dtype,tol_e,tol_f", [(torch.float64, 1e-10, 1e-10), (torch.float32, 1e-5, 1e-4)])
def test_water3000_full_size_matches_oracle_fixture(dtype, tol_e, tol_f, U):
    """The 3 000-atom H/O configuration at its full size (156 916 edges, 128 channels) against the float64 CPU
    oracle's energy and forces, committed as tests/golden/water3000_energy_forces.npz (tests/golden/make_golden.py);
    plus the size-independent properties: forces sum to zero, a rigid translation leaves the energy unchanged."""
    z = np.load(os.path.join(GOLD, "water3000_energy_forces.npz"))
    s, ei, sh, params, m, data = build("water3000", U, dtype, seed=1)
    assert ei.shape[1] == int(z["n_edges"])
    out = m(data)
    assert abs(float(out["interaction_energy"]) - float(z["interaction"])) < tol_e * abs(float(z["interaction"]))
    assert abs(float(out["energy"]) - float(z["energy"])) < tol_e * abs(float(z["energy"]))
    f = out["forces"]
    assert rel_err(f, torch.from_numpy(z["forces"])) < tol_f
    if dtype == torch.float64:
        assert f.sum(0).abs().max().item() < 1e-9 * f.abs().max().item() * f.shape[0]
        moved = dict(data, positions=data["positions"] + torch.tensor([0.3, -0.2, 0.1], dtype=torch.float64, device="cuda"))
        assert abs(float(m(moved)["interaction_energy"]) - float(out["interaction_energy"])) < 1e-10 * abs(float(out["interaction_energy"]))


def _cluster_around(pos, species, box, centre, radius):
    """Atoms (with their periodic images) within `radius` of atom `centre`, as an open cluster; the centre is row 0."""
    d = pos - pos[centre]
    d -= np.round(d / box) * box
    keep = np.flatnonzero((d * d).sum(1) < radius * radius)
    keep = np.concatenate([[centre], keep[keep != centre]])
    return d[keep] + 50.0, species[keep]


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-10), (torch.float32, 2e-5)])
def test_slab_64000_node_energies_match_oracle_on_cut_out_clusters(dtype, tol, U):
    """The 64 000-atom slab at its full size.  A node's interaction energy depends only on the atoms within
    2 r_max = 10 A of it, so the oracle evaluated on the open cluster cut out around an atom must give that atom
    the node energy the kernels give it inside the full periodic system.  Three atoms are checked against the
    oracle; the whole system against the size-independent properties (zero net force, in float64)."""
    from cuda_mace_b200 import systems
    from oracle import model as omodel

    s, ei, sh, params, m, data = build("slab", U, dtype, seed=1)
    out = m(data)
    e0 = m.atomic_energies.index_select(0, data["species"].long())
    node_inter = (out["node_energy"] - e0).cpu()
    pos, species, box = s["positions"], s["species"], np.asarray(s["box"])
    scale = float(node_inter.abs().max())
    for centre in (0, 31999, 63999):
        cpos, cspec = _cluster_around(pos, species, box, centre, 10.0 + 1e-6)
        cei, csh = systems.neighbor_list(cpos, np.full(3, 200.0), (False, False, False), 5.0)
        e_nodes = omodel.node_energies(params, U, torch.from_numpy(cpos), systems.one_hot(cspec, 4),
                                       torch.from_numpy(cei), torch.from_numpy(csh))
        assert abs(float(node_inter[centre]) - float(e_nodes[0])) < tol * scale, (centre, len(cspec))
    if dtype == torch.float64:
        f = out["forces"]
        assert f.sum(0).abs().max().item() < 1e-9 * f.abs().max().item() * f.shape[0]


def test_single_gpu_slab_domain_equals_periodic(U):
    """The domain-decomposed driver with one rank reproduces the plain periodic evaluation."""
    from cuda_mace_b200 import domain

    s, ei, sh, params, m, data = build("cfg0", U, torch.float64)
    dom = domain.partition_slabs(s["positions"], s["species"], s["box"], 1, 5.0, 0)
    plan = domain.HaloPlan(dom, "cuda")
    species = torch.from_numpy(dom.species).to(torch.int32).cuda()
    ei_d = torch.from_numpy(dom.edge_index).to(torch.int32).cuda()
    sh_d = torch.from_numpy(dom.shifts).cuda()

    def node_energy(pos_local, exchange):
        return m.node_energies(pos_local, species, ei_d, sh_d, exchange=exchange, n_owned=dom.n_owned)

    e, f = domain.distributed_energy_forces(node_energy, dom, plan, torch.from_numpy(dom.positions).cuda())
    out = m(data)
    assert abs(float(e) - float(out["interaction_energy"])) < 1e-12 * abs(float(e))
    # the domain stores its atoms grouped by species; owned_global maps its rows back
    assert (np.diff(dom.species[: dom.n_owned]) >= 0).all()
    assert rel_err(f, out["forces"][torch.from_numpy(dom.owned_global).cuda()]) < 1e-12


def test_last_radial_layer_inside_message_passing_matches_oracle(U, monkeypatch):
    """The float32 model with R = H @ W formed inside the message-passing kernel (off by default) against the
    oracle, same tolerances as the default path."""
    from cuda_mace_b200 import ops, systems
    from oracle import model as omodel

    monkeypatch.setattr(ops, "FUSED_RADIAL_MESSAGE_PASSING", True)
    s, ei, sh, params, m, data = build("water3000", U, torch.float32, n_atoms=375, seed=1)
    e, e_inter, f = omodel.energy_and_forces(params, U, torch.from_numpy(s["positions"]),
                                             systems.one_hot(s["species"], 2), torch.from_numpy(ei), torch.from_numpy(sh))
    launches = ops._abi.launch_count
    out = m(data)
    ops.check_status()
    assert ops._abi.launch_count > launches
    assert abs(float(out["interaction_energy"]) - float(e_inter)) < 1e-5 * abs(float(e_inter))
    assert rel_err(out["forces"], f) < 1e-4


def test_host_buffer_path_equals_device_resident_path(U):
    """evaluate_host (pinned host inputs, shift vectors as table + byte index, results copied back) gives the
    energy and forces of the device-resident call on the same domain."""
    from cuda_mace_b200 import domain, evaluator

    s, ei, sh, params, m, data = build("cfg0", U, torch.float64)
    dom = domain.partition_slabs(s["positions"], s["species"], s["box"], 1, 5.0, 0)
    ev = evaluator.EnergyForceEvaluator(m, dom, "cuda")
    e_dev, f_dev = ev(ev.load_domain())
    batch = ev.host_batch()
    assert "shift_index" in batch and batch["shift_index"].dtype == torch.uint8
    assert batch["shift_table"].shape[0] <= 27
    assert evaluator.EnergyForceEvaluator.h2d_bytes(batch) < dom.edge_index.nbytes // 2 + 2 * dom.edge_index.shape[1] + 10 ** 5
    e_host, f_host = ev.evaluate_host(batch)
    assert not f_host.is_cuda
    assert abs(e_host - float(e_dev)) < 1e-12 * abs(e_host)
    assert rel_err(f_host, f_dev) < 1e-12


def test_neighbor_list_built_on_the_device_gives_the_same_energy_and_forces(U):
    """The evaluator with its neighbour list rebuilt on the device from the positions (cell-list kernels) against the
    same evaluator fed with the host list: same edge count, energy and forces to rounding (edge order inside a
    receiver differs, so sums are reordered)."""
    from cuda_mace_b200 import domain, evaluator

    s, ei, sh, params, m, data = build("cfg0", U, torch.float64)
    dom = domain.partition_slabs(s["positions"], s["species"], s["box"], 1, 5.0, 0)
    ev = evaluator.EnergyForceEvaluator(m, dom, "cuda")
    pos = ev.load_domain()
    e_host, f_host = ev(pos)
    n_edges_host = ev.edge_index.shape[1]
    ev.rebuild_neighbor_list(pos)
    assert ev.edge_index.shape[1] == n_edges_host and ev.edge_index.dtype == torch.int32
    e_dev, f_dev = ev(pos)
    assert abs(float(e_dev) - float(e_host)) < 1e-11 * abs(float(e_host))
    assert rel_err(f_dev, f_host) < 1e-10


def test_captured_step_replays_with_new_positions(U):
    """The step recorded as a CUDA graph gives, for positions it was not recorded with, the energy and forces of the
    eager step; a new neighbour list drops the recording."""
    from cuda_mace_b200 import domain, evaluator, ops

    s, ei, sh, params, m, data = build("cfg0", U, torch.float32)
    dom = domain.partition_slabs(s["positions"], s["species"], s["box"], 1, 5.0, 0)
    ev = evaluator.EnergyForceEvaluator(m, dom, "cuda")
    pos = ev.load_domain()
    moved = pos + 0.01 * torch.randn(pos.shape, generator=torch.Generator().manual_seed(1), dtype=pos.dtype).cuda()
    e_ref, f_ref = ev(moved)
    ev.capture(pos)
    launches = ops._abi.launch_count
    e_rep, f_rep = ev(moved)
    ops.check_status()
    assert ops._abi.launch_count == launches          # replayed, not re-launched from Python
    assert abs(float(e_rep) - float(e_ref)) < 1e-6 * abs(float(e_ref))
    assert rel_err(f_rep, f_ref) < 1e-5
    ev.set_neighbor_list(ev.species, ev.edge_index, ev.shifts)
    assert ev._graph is None
