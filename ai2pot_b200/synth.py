"""Seeded synthetic workloads (host numpy arrays) shaped like the benchmark configurations.

One generator feeds the CUDA path, the CPU checkers and the benchmark, so all of them see
identical arrays. ``numpy.random.default_rng(seed)`` (PCG64) throughout.

  g0: 216 atoms, 6x6x6 simple cubic a=3.0, sigma 0.1, MTP level 10, fp64, rcut 5.0
  g1: 13,824 atoms, 24^3, types 2:2:5, MTP level 16, fp64, rcut 6.0
  g2: same structure in fp32, NEP (n_radial=n_angular=4, 8 Chebyshev, l_max 4, 30 neurons)
  g3: 64 structures of 64..256 atoms, MTP level 16 training batch with random targets
  g4: 64^3 cells x 4 atoms (1,048,576 atoms), a=6.0, NEP as g2 (any cell count for tests)
"""
import numpy as np


def cubic_lattice(n, a, sigma, rng, dtype=np.float64, nocc=None):
    g = np.arange(n, dtype=np.float64) * a
    pos = np.stack(np.meshgrid(g, g, g, indexing="ij"), -1).reshape(-1, 3)
    if nocc is not None:
        pos = pos[:nocc]
    pos = pos + rng.normal(0.0, sigma, pos.shape)
    cell = np.eye(3) * (n * a)
    return cell.astype(dtype), pos.astype(dtype)


def mtp_model(tables, ntypes, rng, dtype, rmax, rmin, chebyshev_size=8, sigma=0.01):
    nmus = tables["nmus"]
    ns = len(tables["alpha_moment_mapping"])
    return dict(kind="mtp", tables=tables, chebyshev_size=chebyshev_size, scaling=1.0, ntypes=ntypes,
                coeffs=rng.normal(0, sigma, ntypes * ntypes * nmus * chebyshev_size).astype(dtype),
                linear_coeffs=rng.normal(0, sigma, ns).astype(dtype),
                type_bias=np.zeros(ntypes, dtype), q_scaler=np.ones(ns, dtype),
                rmax=rmax, rmin=rmin)


def nep_model(ntypes, rng, dtype=np.float32, n_radial=4, n_angular=4, chebyshev_size=8, l_max=4,
              num_neurons=30, rmax_radial=6.0, rmax_angular=4.0, sigma=0.1):
    nd = n_radial + n_angular * l_max
    return dict(kind="nep", ntypes=ntypes, chebyshev_size=chebyshev_size, n_radial=n_radial, n_angular=n_angular,
                l_max=l_max, num_neurons=num_neurons, rmax_radial=rmax_radial, rmax_angular=rmax_angular,
                coeffs=rng.normal(0, sigma, ntypes * ntypes * (n_radial + n_angular) * chebyshev_size).astype(dtype),
                w0=rng.normal(0, sigma, ntypes * num_neurons * nd).astype(dtype),
                b0=rng.normal(0, sigma, ntypes * num_neurons).astype(dtype),
                w1=rng.normal(0, sigma, ntypes * num_neurons).astype(dtype),
                type_bias=np.zeros(ntypes, dtype), q_scaler=np.ones(nd, dtype))


def g0(tables_l10, seed=1000):
    rng = np.random.default_rng(seed)
    cell, pos = cubic_lattice(6, 3.0, 0.1, rng)
    types = rng.integers(0, 3, len(pos)).astype(np.int32)
    model = mtp_model(tables_l10, 3, rng, np.float64, 5.0, 0.5)
    return dict(cell=cell, coords=pos, types=types, rcut=5.0, umax=64, model=model)


def g1(tables_l16, seed=1001, n=24):
    rng = np.random.default_rng(seed)
    cell, pos = cubic_lattice(n, 3.0, 0.1, rng)
    types = rng.choice(3, size=len(pos), p=np.array([2, 2, 5]) / 9.0).astype(np.int32)
    model = mtp_model(tables_l16, 3, rng, np.float64, 6.0, 0.5)
    return dict(cell=cell, coords=pos, types=types, rcut=6.0, umax=64, model=model)


def g2(seed=1001, n=24):
    rng = np.random.default_rng(seed)
    cell, pos = cubic_lattice(n, 3.0, 0.1, rng, np.float32)
    types = rng.choice(3, size=len(pos), p=np.array([2, 2, 5]) / 9.0).astype(np.int32)
    model = nep_model(3, rng)
    return dict(cell=cell, coords=pos, types=types, rcut=6.0, umax=64, model=model)


def g3(tables_l16, seed=1003, batch=64, nmin=64, nmax=256):
    """Training batch. Returns a list of structures plus the model and the random targets."""
    rng = np.random.default_rng(seed)
    structs = []
    for _ in range(batch):
        nb = int(rng.integers(nmin, nmax + 1))
        edge = int(np.ceil(nb ** (1.0 / 3.0) - 1e-9))
        a = float(rng.uniform(2.8, 3.2))
        cell, pos = cubic_lattice(edge, a, 0.15, rng, nocc=nb)
        types = rng.integers(0, 3, nb).astype(np.int32)
        structs.append(dict(cell=cell, coords=pos, types=types))
    model = mtp_model(tables_l16, 3, rng, np.float64, 6.0, 0.5)
    npad = max(len(s["types"]) for s in structs)
    targets = dict(E=rng.normal(0, 1, batch), F=rng.normal(0, 1, (batch, npad, 3)), V=rng.normal(0, 1, (batch, 9)))
    return dict(structs=structs, model=model, targets=targets, rcut=6.0, umax=64, weights=(1.0, 1.0, 1.0))


def g4(seed=1004, ncell=64, dtype=np.float32):
    """4 atoms per cubic cell of a=6.0: sublattice A at (0,0,0),(1/2,1/2,1/2), type 0 with 20 %
    replaced by type 1; sublattice B = A + (1/2,0,0), type 2."""
    rng = np.random.default_rng(seed)
    a = 6.0
    g = np.arange(ncell, dtype=np.float64) * a
    org = np.stack(np.meshgrid(g, g, g, indexing="ij"), -1).reshape(-1, 1, 3)
    basis = np.array([[0, 0, 0], [.5, .5, .5], [.5, 0, 0], [0, .5, .5]]) * a
    pos = (org + basis[None]).reshape(-1, 3)
    types = np.tile(np.array([0, 0, 2, 2], np.int32), ncell ** 3)
    sub = rng.random(len(types)) < 0.2
    types[(types == 0) & sub] = 1
    pos = pos + rng.normal(0, 0.1, pos.shape)
    cell = np.eye(3) * (ncell * a)
    model = nep_model(3, rng)
    return dict(cell=cell.astype(dtype), coords=pos.astype(dtype), types=types, rcut=6.0, umax=32, model=model)


def batch_from_nblist(numneigh, firstneigh, rcs, types, ntypes):
    """Wrap one structure's neighbour list as the batched (B=1) tensors the ops take."""
    n = len(numneigh)
    return dict(binum=np.array([n], np.int32), bilist=np.arange(n, dtype=np.int32)[None],
                bnumneigh=numneigh[None].astype(np.int32), bfirstneigh=firstneigh[None].astype(np.int32),
                brcs=rcs[None], btypes=types[None].astype(np.int32), ntypes=ntypes, nghost=0)


def pad_batch(lists, ntypes, umax):
    """Stack per-structure (numneigh, firstneigh, rcs, types) into padded batch tensors."""
    B = len(lists)
    npad = max(len(l[0]) for l in lists)
    dt = lists[0][2].dtype
    out = dict(binum=np.zeros(B, np.int32), bilist=np.zeros((B, npad), np.int32),
               bnumneigh=np.zeros((B, npad), np.int32), bfirstneigh=np.full((B, npad, umax), -1, np.int32),
               brcs=np.zeros((B, npad, umax, 3), dt), btypes=np.zeros((B, npad), np.int32), ntypes=ntypes, nghost=0)
    for b, (nn, fn, rc, ty) in enumerate(lists):
        n = len(nn)
        out["binum"][b] = n
        out["bilist"][b, :n] = np.arange(n)
        out["bnumneigh"][b, :n] = nn
        out["bfirstneigh"][b, :n] = fn
        out["brcs"][b, :n] = rc
        out["btypes"][b, :n] = ty
    return out
