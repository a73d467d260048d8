"""Seeded synthetic systems, neighbour lists and random-init model parameters.

The reference measures on ASE-built diamond supercells with upstream MACE's neighbour list
(tests/test_utils.py:85-114); neither package is a dependency here, so the benchmark and the
tests use seeded synthetic boxes of the same densities and a cell-list neighbour search.  The
neighbour list is an *input* of the hot path (``data["edge_index"]``, ``data["shifts"]`` in
cuda_mace/models/InvariantMACE.py:297-301), built on the host.

Edge convention (cuda_mace/models/InvariantMACE.py:99-100): receiver = edge_index[0],
sender = edge_index[1], vector = positions[sender] - positions[receiver] + shift, and the list is
sorted by receiver, as InvariantMessagePassingTP requires.
"""
import math

import numpy as np
import torch


# --------------------------------------------------------------------------------------
# neighbour list
# --------------------------------------------------------------------------------------
def _with_images(pos, box, pbc, r_cut):
    """Appends explicit periodic images lying within r_cut of the box; returns
    (ext_pos [M,3], ext_src [M] index of the original atom, ext_shift [M,3])."""
    ext_pos = pos
    ext_src = np.arange(pos.shape[0])
    ext_shift = np.zeros_like(pos)
    for d in range(3):
        if not pbc[d]:
            continue
        L = box[d]
        if L < r_cut:
            raise ValueError(f"periodic box length {L} is shorter than the cutoff {r_cut}")
        lo = ext_pos[:, d] < r_cut
        hi = ext_pos[:, d] >= L - r_cut
        add_pos, add_src, add_shift = [], [], []
        for mask, sgn in ((lo, +1.0), (hi, -1.0)):
            p = ext_pos[mask].copy()
            s = ext_shift[mask].copy()
            p[:, d] += sgn * L
            s[:, d] += sgn * L
            add_pos.append(p)
            add_src.append(ext_src[mask])
            add_shift.append(s)
        ext_pos = np.concatenate([ext_pos] + add_pos)
        ext_src = np.concatenate([ext_src] + add_src)
        ext_shift = np.concatenate([ext_shift] + add_shift)
    return ext_pos, ext_src, ext_shift


def neighbor_list(pos, box, pbc, r_cut, n_receivers=None):
    """Full (both directions) neighbour list of an orthorhombic box by cell list.

    pos [N,3] float64 numpy inside [0, box) along periodic axes; box (3,); pbc (3,) bools.
    Only the first `n_receivers` atoms receive (default: all).  Returns
    edge_index [2,E] int64 (row 0 receivers, sorted; row 1 senders) and shifts [E,3] float64.
    """
    pos = np.asarray(pos, dtype=np.float64)
    N = pos.shape[0]
    n_recv = N if n_receivers is None else int(n_receivers)
    ext_pos, ext_src, ext_shift = _with_images(pos, np.asarray(box, float), pbc, r_cut)
    lo = ext_pos.min(axis=0) - 1e-9
    cid3 = np.floor((ext_pos - lo) / r_cut).astype(np.int64) + 1  # pad by one cell
    dims = cid3.max(axis=0) + 2
    flat = (cid3[:, 0] * dims[1] + cid3[:, 1]) * dims[2] + cid3[:, 2]
    order = np.argsort(flat, kind="stable")
    ncell = int(dims.prod())
    count = np.bincount(flat, minlength=ncell)
    start = np.concatenate([[0], np.cumsum(count)[:-1]])
    r2 = r_cut * r_cut
    recv_all, send_all = [], []
    rc = cid3[:n_recv]
    ridx = np.arange(n_recv)
    for dx in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dz in (-1, 0, 1):
                ncid = ((rc[:, 0] + dx) * dims[1] + (rc[:, 1] + dy)) * dims[2] + (rc[:, 2] + dz)
                cnt = count[ncid]
                tot = int(cnt.sum())
                if tot == 0:
                    continue
                recv = np.repeat(ridx, cnt)
                base = np.repeat(np.cumsum(cnt) - cnt, cnt)
                send_ext = order[np.repeat(start[ncid], cnt) + (np.arange(tot) - base)]
                d = ext_pos[send_ext] - pos[recv]
                keep = ((d * d).sum(axis=1) < r2) & (send_ext != recv)
                recv_all.append(recv[keep])
                send_all.append(send_ext[keep])
    recv = np.concatenate(recv_all) if recv_all else np.zeros(0, np.int64)
    send_ext = np.concatenate(send_all) if send_all else np.zeros(0, np.int64)
    send = ext_src[send_ext]
    key = np.lexsort((send_ext, send, recv))
    recv, send, send_ext = recv[key], send[key], send_ext[key]
    edge_index = np.stack([recv, send]).astype(np.int64)
    return edge_index, ext_shift[send_ext]


def symmetric_graph(seed, n_nodes, mean_degree):
    """Random undirected graph as a directed, receiver-sorted, duplicate-free, symmetric edge list in which every
    node has at least one edge (a ring guarantees it): the kind of list the reference's message passing needs
    (reverse-edge lookup, no edgeless receivers).  Returns int32 torch tensors (sender, receiver)."""
    rng = np.random.default_rng(seed)
    n_pairs = max(1, int(n_nodes * mean_degree / 2))
    a = rng.integers(0, n_nodes, n_pairs)
    b = rng.integers(0, n_nodes, n_pairs)
    ring = np.arange(n_nodes)
    a = np.concatenate([a, ring])
    b = np.concatenate([b, (ring + 1) % n_nodes])
    keep = a != b
    lo, hi = np.minimum(a[keep], b[keep]), np.maximum(a[keep], b[keep])
    pairs = np.unique(lo.astype(np.int64) * n_nodes + hi)
    lo, hi = pairs // n_nodes, pairs % n_nodes
    recv = np.concatenate([lo, hi])
    send = np.concatenate([hi, lo])
    order = np.lexsort((send, recv))
    return torch.from_numpy(send[order].astype(np.int32)), torch.from_numpy(recv[order].astype(np.int32))


# --------------------------------------------------------------------------------------
# systems
# --------------------------------------------------------------------------------------
def random_box(n_atoms, box, min_dist, seed):
    """Uniform positions in a periodic orthorhombic box with a minimum image distance
    (batched rejection sampling)."""
    from scipy.spatial import cKDTree

    rng = np.random.default_rng(seed)
    box = np.asarray(box, dtype=np.float64)
    acc = np.zeros((0, 3))
    while acc.shape[0] < n_atoms:
        need = n_atoms - acc.shape[0]
        cand = rng.random((int(need * 1.3) + 16, 3)) * box
        cand = np.minimum(cand, np.nextafter(box, 0.0))
        ct = cKDTree(cand, boxsize=box)
        bad = np.zeros(cand.shape[0], dtype=bool)
        pairs = ct.query_pairs(min_dist, output_type="ndarray")
        if pairs.size:
            bad[pairs.max(axis=1)] = True
        if acc.shape[0]:
            at = cKDTree(acc, boxsize=box)
            d, _ = at.query(cand, k=1, distance_upper_bound=min_dist)
            bad |= np.isfinite(d)
        acc = np.concatenate([acc, cand[~bad][:need]])
    return acc


def jittered_lattice(n_side, box_side, sigma, seed):
    """Simple-cubic lattice sites with N(0, sigma) displacements, wrapped into the box."""
    rng = np.random.default_rng(seed)
    g = (np.arange(n_side) + 0.5) * (box_side / n_side)
    pos = np.stack(np.meshgrid(g, g, g, indexing="ij"), axis=-1).reshape(-1, 3)
    pos = pos + rng.normal(0.0, sigma, pos.shape)
    return np.mod(pos, box_side)


def one_hot(species, n_species, dtype=torch.float64):
    out = torch.zeros(len(species), n_species, dtype=dtype)
    out[torch.arange(len(species)), torch.as_tensor(species, dtype=torch.long)] = 1.0
    return out


def make_system(name, seed=None, n_atoms=None):
    """Named synthetic systems.  Returns a dict with numpy `positions`, `species`, `box`,
    `n_species`, and the model size (`channels`) each configuration is quoted on."""
    if name == "cfg0":  # 192 atoms, 12.4 A periodic cube, jittered lattice, 4 species, C=64
        seed = 0 if seed is None else seed
        side = 12.4
        pos = jittered_lattice(6, side, 0.15, seed)[:192]
        rng = np.random.default_rng(seed + 1)
        return dict(positions=pos, species=rng.integers(0, 4, pos.shape[0]), box=np.full(3, side),
                    n_species=4, channels=64)
    if name == "water3000":  # 1000 O + 2000 H at 0.1 atoms/A^3, d_min 0.9 A, C=128
        seed = 1 if seed is None else seed
        n = 3000 if n_atoms is None else n_atoms
        side = (n / 0.1) ** (1.0 / 3.0)
        pos = random_box(n, np.full(3, side), 0.9, seed)
        species = np.zeros(n, dtype=np.int64)
        species[n // 3:] = 1
        return dict(positions=pos, species=species, box=np.full(3, side), n_species=2, channels=128)
    if name == "slab":  # H:C:N:O = 50:30:10:10 at 0.1 atoms/A^3, 80 x 80 A cross-section, C=128
        seed = 4 if seed is None else seed
        n = 64000 if n_atoms is None else n_atoms
        box = np.array([80.0, 80.0, n / 0.1 / 6400.0])
        pos = random_box(n, box, 0.9, seed)
        rng = np.random.default_rng(seed + 1)
        species = rng.choice(4, size=n, p=[0.5, 0.3, 0.1, 0.1])
        return dict(positions=pos, species=species, box=box, n_species=4, channels=128)
    raise KeyError(name)


# --------------------------------------------------------------------------------------
# model parameters
# --------------------------------------------------------------------------------------
def init_params(channels, n_species, seed, r_max=5.0, avg_num_neighbors=None, radial_hidden=64,
                num_bessel=8):
    """Random-init invariant MACE parameters (2 layers, l_max=3, correlation 3) as float64 CPU
    tensors, unit-normal like e3nn's initialisation."""
    g = torch.Generator().manual_seed(seed)

    def rn(*shape, scale=1.0):
        return torch.randn(*shape, generator=g, dtype=torch.float64) * scale

    C, Z = channels, n_species
    if avg_num_neighbors is None:
        avg_num_neighbors = 0.1 * 4.0 / 3.0 * math.pi * r_max**3
    params = dict(r_max=r_max, atomic_energies=rn(Z), W_embed=rn(Z, C), scale=0.8, shift=0.1, layers=[])
    for t in range(2):
        P = dict(
            W_up=rn(C, C),
            W_radial=[rn(num_bessel, radial_hidden), rn(radial_hidden, radial_hidden),
                      rn(radial_hidden, radial_hidden), rn(radial_hidden, 4 * C)],
            W_lin=rn(4, C, C),
            avg_num_neighbors=float(avg_num_neighbors),
            W3=rn(Z, 23, C, scale=1.0 / 23.0),
            W2=rn(Z, 4, C, scale=1.0 / 4.0),
            W1=rn(Z, 1, C),
            W_prod=rn(C, C),
        )
        if t == 0:
            P["W_skip"] = rn(Z, 4, C, C)
            P["W_readout"] = rn(C, 1)
        else:
            P["W_sc"] = rn(C, Z, C)
            P["W_readout1"] = rn(C, 16)
            P["W_readout2"] = rn(16, 1)
        params["layers"].append(P)
    return params
