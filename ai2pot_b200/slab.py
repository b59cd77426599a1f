"""Spatial decomposition of one large periodic system into slabs along the first lattice vector,
one slab per rank / GPU, for energy + force + virial evaluation.

This is the role LAMMPS plays for the reference (`interface/lammps/AI2POT/pair_ai2pot.cpp:177-205,
452-455`: the pair style evaluates local + ghost atoms and returns forces on both; LAMMPS
exchanges ghost positions before and reverse-communicates ghost forces after). Here:

  set-up   each rank keeps the atoms whose fractional coordinate along a0 lies in its slab and
           builds, once, the lists of owned atoms inside the halo (>= cutoff) of either face
  step     1. halo exchange: boundary positions to the two face neighbours (periodic; the wrapped
              copies are shifted by -/+ a0 with the reference's own image arithmetic r + a0*n)
           2. neighbour list over owned + ghost atoms, rows for owned atoms only, open along a0
           3. model evaluation with nghost ghosts: forces on owned and ghost atoms
           4. ghost forces go back to their owners and are added ("ghost-force reduction")
           5. all-reduce of the energy and the nine virial components

`torch.distributed` (NCCL on GPUs, gloo in the CPU tests) carries the messages; message sizes are
fixed at set-up, so a step makes no host synchronisation. The compute of steps 2-3 is injected
(`LocalCompute`), so the partition / exchange / reduction logic can be tested on CPU.
"""
import numpy as np
import torch


def partition(cell, coords, nranks):
    """Rank of every atom: slab index of its fractional coordinate along a0, wrapped into [0,1)."""
    inv = np.linalg.inv(np.asarray(cell, np.float64))
    s = np.asarray(coords, np.float64) @ inv
    wrap = np.floor(s[:, 0])
    fx = s[:, 0] - wrap
    owner = np.minimum((fx * nranks).astype(np.int64), nranks - 1)
    return owner, fx, wrap


class SlabDomain:
    def __init__(self, cell, coords, types, rcut, rank, nranks, device, dist=None, halo_margin=1e-6):
        """cell [3,3], coords [N,3], types [N] describe the WHOLE system (host arrays, identical on
        every rank); each rank keeps only its slab."""
        self.rank, self.P, self.dist, self.device = rank, nranks, dist, device
        self.cell = np.asarray(cell)
        self.dtype = torch.float64 if np.asarray(coords).dtype == np.float64 else torch.float32
        a = np.asarray(cell, np.float64)
        n0 = np.cross(a[1], a[2])
        d0 = abs(a[0] @ (n0 / np.linalg.norm(n0)))          # slab-normal extent of the cell
        self.width = d0 / nranks
        if nranks > 1 and self.width < rcut:
            raise ValueError(f"slab width {self.width:.3f} is below the cutoff {rcut}: use fewer ranks")
        owner, fx, wrap = partition(cell, coords, nranks)
        mine = np.nonzero(owner == rank)[0]
        self.global_index = mine
        self.nlocal = len(mine)
        # positions are brought into the cell along a0 (the input may be unwrapped), so that a slab is contiguous
        inside = np.asarray(coords)[mine] - (wrap[mine, None] * np.asarray(cell)[0][None]).astype(np.asarray(coords).dtype)
        self.owned = torch.from_numpy(np.ascontiguousarray(inside)).to(device)
        self.owned_types = torch.from_numpy(np.ascontiguousarray(types[mine], dtype=np.int32)).to(device)
        self.a0 = torch.from_numpy(np.ascontiguousarray(self.cell[0])).to(self.dtype).to(device)
        h = (rcut + halo_margin) / d0                        # halo in fractional units
        f = fx[mine] * nranks - rank                         # position inside the slab, [0,1)
        hs = h * nranks
        if nranks == 1:
            self.send_left = self.send_right = torch.zeros(0, dtype=torch.int64, device=device)
        else:
            self.send_left = torch.from_numpy(np.nonzero(f < hs)[0]).to(device)          # -> rank-1 (its right ghosts)
            self.send_right = torch.from_numpy(np.nonzero(f >= 1.0 - hs)[0]).to(device)  # -> rank+1 (its left ghosts)
        self.left, self.right = (rank - 1) % nranks, (rank + 1) % nranks
        # ghost counts: what the neighbours send us
        counts = torch.tensor([len(self.send_left), len(self.send_right)], dtype=torch.int64)
        if nranks > 1:
            allc = [torch.zeros(2, dtype=torch.int64) for _ in range(nranks)]
            self._all_gather_cpu(allc, counts)
            self.n_from_left = int(allc[self.left][1])       # left neighbour's right boundary
            self.n_from_right = int(allc[self.right][0])     # right neighbour's left boundary
        else:
            self.n_from_left = self.n_from_right = 0
        self.nghost = self.n_from_left + self.n_from_right
        self.ntotal = self.nlocal + self.nghost
        # ghost types travel once
        self.types = torch.empty(self.ntotal, dtype=torch.int32, device=device)
        self.types[: self.nlocal] = self.owned_types
        if nranks > 1:
            tl, tr = self._exchange(self.owned_types[self.send_left].contiguous(), self.owned_types[self.send_right].contiguous(),
                                    torch.int32, ())
            self.types[self.nlocal: self.nlocal + self.n_from_left] = tl
            self.types[self.nlocal + self.n_from_left:] = tr
        # one buffer [owned | ghosts from the left | ghosts from the right]; `owned` is a view of its head
        self.local = torch.empty(self.ntotal, 3, dtype=self.dtype, device=device)
        self.local[: self.nlocal] = self.owned
        self.owned = self.local[: self.nlocal]
        self.ghost_left = self.local[self.nlocal: self.nlocal + self.n_from_left]
        self.ghost_right = self.local[self.nlocal + self.n_from_left:]
        # Periodic wrap of the end slabs: copies going "around" the cell are shifted by -/+ a0. The sender
        # applies it, with the reference's image arithmetic r + a0 * n (source/nblist/include/structure.h:654-682).
        nl, nr = len(self.send_left), len(self.send_right)
        self.send_idx = torch.cat([self.send_left, self.send_right])
        self.send_buf = torch.empty(nl + nr, 3, dtype=self.dtype, device=device)
        self.back = torch.empty(nl + nr, 3, dtype=self.dtype, device=device)      # ghost forces coming home
        shift = torch.zeros(nl + nr, 3, dtype=self.dtype, device=device)
        if nranks > 1 and rank == 0:
            shift[:nl] = self.a0 * 1.0           # my left neighbour is the last slab: it sees these one cell up
        if nranks > 1 and rank == nranks - 1:
            shift[nl:] = self.a0 * -1.0          # my right neighbour is slab 0
        self.send_shift = shift if (nranks > 1 and (rank == 0 or rank == nranks - 1)) else None
        self.pbc = (nranks == 1, True, True)

    # -- plumbing ----------------------------------------------------------------------------------
    def _all_gather_cpu(self, out, t):
        if self.dist.get_backend() == "nccl":
            dev = [o.to(self.device) for o in out]
            self.dist.all_gather(dev, t.to(self.device))
            for o, d in zip(out, dev):
                o.copy_(d.cpu())
        else:
            self.dist.all_gather(out, t)

    def _exchange(self, to_left, to_right, dtype, tail, from_left=None, from_right=None):
        """Send `to_left` to the left neighbour and `to_right` to the right one; returns what the
        left and the right neighbours sent here (sizes known from set-up)."""
        d = self.dist
        if from_left is None:
            from_left = torch.empty((self.n_from_left,) + tail, dtype=dtype, device=self.device)
            from_right = torch.empty((self.n_from_right,) + tail, dtype=dtype, device=self.device)
        # tag 0: "towards lower x", tag 1: "towards higher x". With two ranks both neighbours are the
        # same peer; the tags (gloo) and the posting order (NCCL, which ignores tags) keep the two
        # messages apart: what the peer sent towards lower x arrives as our right-hand ghosts.
        ops = [d.P2POp(d.isend, to_left, self.left, tag=0), d.P2POp(d.isend, to_right, self.right, tag=1),
               d.P2POp(d.irecv, from_right, self.right, tag=0), d.P2POp(d.irecv, from_left, self.left, tag=1)]
        for r in d.batch_isend_irecv(ops):
            r.wait()
        return from_left, from_right

    # -- one evaluation ------------------------------------------------------------------------------
    def halo_exchange(self):
        """Step 1: boundary positions (already shifted for the wrap) go straight into the neighbours'
        ghost rows of `local`: one gather, one add on the end slabs, one grouped send/receive."""
        if self.P > 1:
            nl = len(self.send_left)
            torch.index_select(self.owned, 0, self.send_idx, out=self.send_buf)
            if self.send_shift is not None:
                self.send_buf.add_(self.send_shift)
            self._exchange(self.send_buf[:nl], self.send_buf[nl:], self.dtype, (3,), self.ghost_left, self.ghost_right)
        return self.local

    def reduce_ghost_forces(self, force):
        """Step 4: force is [ntotal,3]; ghost rows go back to the ranks that own those atoms, which add
        them with one indexed accumulation."""
        owned = force[: self.nlocal]
        if self.P > 1:
            nl = len(self.send_left)
            gl = force[self.nlocal: self.nlocal + self.n_from_left]
            gr = force[self.nlocal + self.n_from_left:]
            d = self.dist
            ops = [d.P2POp(d.isend, gl, self.left, tag=0), d.P2POp(d.isend, gr, self.right, tag=1),
                   d.P2POp(d.irecv, self.back[nl:], self.right, tag=0), d.P2POp(d.irecv, self.back[:nl], self.left, tag=1)]
            for r in d.batch_isend_irecv(ops):
                r.wait()
            owned.index_add_(0, self.send_idx, self.back)
        return owned

    def evaluate(self, compute):
        """compute(local_coords[ntotal,3], types[ntotal], nlocal, pbc) -> (e[1], f[ntotal,3], v[9])."""
        local = self.halo_exchange()
        e, f, v = compute(local, self.types, self.nlocal, self.pbc)
        owned_f = self.reduce_ghost_forces(f.reshape(self.ntotal, 3))
        ev = torch.cat([e.reshape(1), v.reshape(9)])
        if self.P > 1:
            self.dist.all_reduce(ev)
        return ev[0], owned_f, ev[1:]


class LocalCompute:
    """Steps 2-3 on the GPU through the C ABI: ghost-aware neighbour list, then NEP or MTP E/F/V."""

    def __init__(self, model, cell, rcut, umax, dtype):
        from . import capi
        self.capi = capi
        self.kind = model["kind"]
        dev = torch.device("cuda", torch.cuda.current_device())
        self.model = capi.to_device({k: v for k, v in model.items() if k != "tables"}, dev, dtype)
        self.prog = capi.MtpProgram(model["tables"]) if self.kind == "mtp" else None
        self.builder = capi.NeighborBuilder()
        self.cell, self.rcut, self.umax, self.ntypes = np.asarray(cell), float(rcut), int(umax), int(model["ntypes"])
        self.status = None
        self._static = None
        self._graph = None

    def __call__(self, local, types, nlocal, pbc):
        """Neighbour build + E/F/V on the slab. The sequence of launches and every buffer are the same from
        step to step (the halo exchange writes into `local` in place), so after the first call the whole
        sequence is replayed from a CUDA graph; a refused capture leaves the eager path in place."""
        key = (local.data_ptr(), types.data_ptr(), nlocal, local.shape[0], tuple(pbc))
        if self._graph is not None and self._graph[0] == key:
            self._graph[1].replay()
            return self._graph[2]
        out = self._run(local, types, nlocal, pbc)
        if self._graph is None or self._graph[0] not in (key, "refused"):
            try:
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    gout = self._run(local, types, nlocal, pbc)
                self._graph = (key, g, gout)
            except Exception:
                self._graph = ("refused",)
                torch.cuda.synchronize()
        return out

    def _run(self, local, types, nlocal, pbc):
        nn, fn, rcs, status = self.builder.build(self.cell, local, self.rcut, self.umax, pbc=pbc, ncentres=nlocal)
        self.status = status
        ntotal = local.shape[0]
        if self._static is None or self._static[0] != (nlocal, ntotal):
            dev = local.device
            self._static = ((nlocal, ntotal), torch.tensor([nlocal], dtype=torch.int32, device=dev),
                            torch.arange(nlocal, dtype=torch.int32, device=dev)[None].contiguous())
        nb = dict(binum=self._static[1], bilist=self._static[2], bnumneigh=nn[None], bfirstneigh=fn[None], brcs=rcs[None],
                  btypes=types[None], ntypes=self.ntypes, nghost=ntotal - nlocal)
        if self.kind == "mtp":
            e, f, v = self.capi.mtp_efv(self.prog, self.model, nb)
        else:
            e, f, v = self.capi.nep_efv(self.model, nb)
        return e, f[0], v[0]
